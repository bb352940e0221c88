"""Python faces of ``csrc/window_attention.cu``: the row copy that stores a token's keys and values, and
attention over a sliding window of cache rows ``[key | value]`` with the score variants of that file."""

from __future__ import annotations

import torch

from . import _need, _ptr, _stream, dtype_code
from .library import check, library

SPLIT_MAX_PARTS = 16
SPLIT_BELOW_TOKENS = 64     # steps of fewer tokens cut windows finely: their few rows must fill the GPU
SPLIT_LONG_KEYS = 512       # longer steps cut the keys of a row into pieces of about this many, so that rows deep in a prompt
SPLIT_MAX_ROW_PARTS = 8192  # do not run much longer than the others; at most this many (token, part) pairs
_scratch: dict[tuple, torch.Tensor] = {}  # (device index, floats per token and part, pairs) -> the partial sums of cut windows


def _partial_sums(device, heads: int, dv: int, pairs: int = 0) -> torch.Tensor:
    """Room for the partial sums of ``pairs`` (token, part) pairs, in sizes that are made once and never replaced
    (captured steps point at them): the finest cut of a short step, or the next power of two."""
    per = heads * dv + 2 * heads
    capacity = SPLIT_BELOW_TOKENS * SPLIT_MAX_PARTS
    while capacity < pairs:
        capacity *= 2
    key = (torch.device(device).index or 0, per, capacity)
    have = _scratch.get(key)
    if have is None:
        have = _scratch[key] = torch.empty(capacity * per, dtype=torch.float32, device=device)
    return have


def set_tensor_cores(on: bool) -> None:
    """Whether bfloat16 calls may run the tensor-core form of the attention kernel (the default) or always the CUDA-core one."""
    library().cw_window_attention_set_mma(1 if on else 0)


def store_rows(src: torch.Tensor, col0: int, width: int, cache_rows: torch.Tensor, slots: torch.Tensor, status: torch.Tensor) -> None:
    """``cache_rows[slots[n]] = src[n, col0 : col0 + width]`` for every token n with a slot (< 0: none)."""
    if src.dim() != 2 or src.stride(1) != 1:
        raise ValueError("src must be [N, C] with unit column stride")
    _need(cache_rows, src.dtype, "cache")
    _need(slots, torch.int32, "slots", 1)
    n = src.shape[0]
    total = cache_rows.numel() // width
    check(library().cw_store_rows(_ptr(src), src.stride(0) if n > 1 else max(src.stride(0), src.shape[1]), col0, width, _ptr(cache_rows),
                                  _ptr(slots), n, total, dtype_code(src.dtype), _ptr(status), _stream()), "store_rows")


def rotate_store(src: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor, slots: torch.Tensor | None, inv_freq: torch.Tensor | None,
                 heads: int, kv_heads: int, dk: int, dv: int, rot: int, cache_rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """From the float32 product rows ``src`` [N, >= heads*dk + kv_heads*(dk + dv)] (queries, then ``[key | value]`` per
    key/value head): the first ``rot`` entries of every query and key head turned by the token's position (entry i with
    entry i + rot/2 by ``position * inv_freq[i]``, float32 angles); returns the queries [N, heads*dk] in the cache's dtype
    and stores the rows ``[key | value]`` where ``slots`` says (None: nothing is stored)."""
    if src.dtype != torch.float32 or src.dim() != 2 or src.stride(1) != 1:
        raise ValueError("src must be float32 [N, C] with unit column stride")
    _need(cache_rows, None, "cache", 4)
    if tuple(cache_rows.shape[2:]) != (kv_heads, dk + dv):
        raise ValueError(f"cache rows {tuple(cache_rows.shape)} are not [pages, page_size, {kv_heads}, {dk + dv}]")
    if rot:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rot:
            raise ValueError(f"inv_freq has {inv_freq.shape[0]} entries for {rot} rotated dimensions")
    n = src.shape[0]
    q = torch.empty((n, heads * dk), dtype=cache_rows.dtype, device=src.device)
    total = cache_rows.shape[0] * cache_rows.shape[1]
    check(library().cw_rotate_store(_ptr(src), src.stride(0) if n > 1 else max(src.stride(0), src.shape[1]), _ptr(positions), _ptr(tok_seq),
                                    _ptr(slots), _ptr(inv_freq) if rot else None, n, heads, kv_heads, dk, dv, rot, _ptr(q), _ptr(cache_rows),
                                    total, dtype_code(cache_rows.dtype), _ptr(status), _stream()), "rotate_store")
    return q


NO_WINDOW = 1 << 30  # a window that never closes: every earlier position is seen


def pool_rows(cache_rows: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor,
              pool_slots: torch.Tensor, pool_cache: torch.Tensor, pool: int, status: torch.Tensor) -> None:
    """For every token whose position ends a block of ``pool`` positions ((position + 1) % pool == 0): the mean of the block's
    rows of ``cache_rows`` [pages, page_size, kv_heads, width] (through the request's ``block_tables`` row) is written to row
    ``pool_slots[n]`` of ``pool_cache`` [pages', page_size, kv_heads, width].  The sum is float32, in position order."""
    _need(cache_rows, None, "cache", 4)
    _need(pool_cache, cache_rows.dtype, "pool cache", 4)
    if tuple(pool_cache.shape[1:]) != tuple(cache_rows.shape[1:]):
        raise ValueError(f"pool cache rows {tuple(pool_cache.shape)} do not match cache rows {tuple(cache_rows.shape)}")
    _need(block_tables, torch.int32, "block_tables", 2)
    _need(pool_slots, torch.int32, "pool_slots", 1)
    n = positions.shape[0]
    width = cache_rows.shape[2] * cache_rows.shape[3]
    check(library().cw_pool_rows(_ptr(cache_rows), _ptr(block_tables), block_tables.shape[1], cache_rows.shape[1], cache_rows.shape[0],
                                 _ptr(positions), _ptr(tok_seq), _ptr(pool_slots), _ptr(pool_cache), pool_cache.shape[0] * pool_cache.shape[1],
                                 width, int(pool), n, dtype_code(cache_rows.dtype), _ptr(status), _stream()), "pool_rows")


def window_parts(num_tokens: int, window: int, dtype: torch.dtype, longest_context: int | None = None) -> int:
    """In how many pieces the keys of a row are cut (the pieces are added up by a second kernel).  float32 runs never
    cut: their results do not depend on the step's size to the last bit.  bfloat16: finely when a step has so few
    tokens that whole windows per thread block would leave most of the GPU idle; coarsely in longer steps over long
    windows, where the last rows of a prompt would otherwise run several times as long as the first.
    ``longest_context``: a bound on the step's longest context, for windows that never close."""
    if dtype != torch.bfloat16 or window <= 256:
        return 1
    if num_tokens < SPLIT_BELOW_TOKENS:
        return max(1, min(SPLIT_MAX_PARTS, window // 128, 128 // max(1, num_tokens)))
    longest = min(window, num_tokens + window // 2)  # (keys that a row of this step may see: a guess, contexts are not known here)
    if window >= NO_WINDOW and longest_context is not None:
        longest = max(num_tokens, longest_context)
    return max(1, min(longest // SPLIT_LONG_KEYS, SPLIT_MAX_ROW_PARTS // num_tokens, SPLIT_MAX_PARTS))


def reserve_window_scratch(device, heads: int, dv: int) -> None:
    _partial_sums(device, heads, dv)


def window_attention(q: torch.Tensor, cache_rows: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor,
                     tok_seq: torch.Tensor, q_start: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, window: int, scale: float,
                     head_scale: torch.Tensor | None, talk: torch.Tensor | None, head_bias: torch.Tensor | None,
                     sigmoid_weights: bool, status: torch.Tensor, parts: int = 1, blocked: bool = False,
                     sink: torch.Tensor | None = None, softcap: float = 0.0, slopes: torch.Tensor | None = None,
                     temperature: tuple | None = None, gate: torch.Tensor | None = None, pool: int = 0,
                     pool_rows_cache: torch.Tensor | None = None, pool_tables: torch.Tensor | None = None) -> torch.Tensor:
    """[N, heads*dv] in ``q``'s dtype.  ``q`` [N, >= heads*dk] (queries in the leading columns, unit column stride);
    ``cache_rows`` [pages, page_size, kv_heads, dk + dv]; the step's tokens are already stored there.  ``blocked``:
    positions are cut into blocks of ``window`` and a token sees its own block up to itself, instead of the last
    ``window`` positions.  ``sink`` [heads]: a logit per head that enters the softmax's denominator once.  ``softcap``:
    the score becomes ``softcap tanh(score / softcap)``; ``slopes`` [heads]: ``slopes[h] * (distance to the key)`` is taken
    off the (capped) score; ``temperature`` = (coef, every): the scores of a query at position p are first multiplied by
    ``1 + coef ln(floor((p + 1) / every) + 1)``; ``gate`` float32 [N, >= heads] (unit column stride): head h's output is
    multiplied by ``sigmoid(gate[n, h])``; ``pool``: every block of ``pool`` positions that ends at or before p - window is
    seen as one more key and value, row b of the request in ``pool_rows_cache`` (through ``pool_tables``)."""
    if q.dim() != 2 or q.stride(1) != 1 or q.shape[1] < heads * dk:
        raise ValueError("q must be [N, >= heads*dk] with unit column stride")
    _need(cache_rows, q.dtype, "cache", 4)
    if tuple(cache_rows.shape[2:]) != (kv_heads, dk + dv):
        raise ValueError(f"cache rows {tuple(cache_rows.shape)} are not [pages, page_size, {kv_heads}, {dk + dv}]")
    _need(block_tables, torch.int32, "block_tables", 2)
    _need(q_start, torch.int32, "q_start", 1)
    if sink is not None and sigmoid_weights:
        raise ValueError("a sink belongs to softmax weights")
    for name, t, size in (("head_scale", head_scale, heads), ("talk", talk, heads * heads), ("head_bias", head_bias, heads),
                          ("sink", sink, heads)):
        if t is not None:
            _need(t, torch.float32, name)
            if t.numel() != size:
                raise ValueError(f"{name} has {t.numel()} numbers, {size} expected")
    n = q.shape[0]
    if slopes is not None:
        _need(slopes, torch.float32, "slopes", 1)
        if slopes.shape[0] != heads:
            raise ValueError(f"slopes has {slopes.shape[0]} numbers for {heads} heads")
    if gate is not None and (gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[1] < heads or gate.shape[0] != n):
        raise ValueError("gate must be float32 [N, >= heads] with unit column stride")
    if pool:
        _need(pool_rows_cache, q.dtype, "pool cache", 4)
        _need(pool_tables, torch.int32, "pool_tables", 2)
        if tuple(pool_rows_cache.shape[1:]) != tuple(cache_rows.shape[1:]) or pool_tables.shape[0] != block_tables.shape[0]:
            raise ValueError("the pooled rows' cache and tables must match the cache's rows and the step's requests")
    coef, every = temperature if temperature is not None else (0.0, 0)
    out = torch.empty((n, heads * dv), dtype=q.dtype, device=q.device)
    partial = None
    if parts > 1:
        if parts > SPLIT_MAX_PARTS:
            raise ValueError(f"windows are cut in at most {SPLIT_MAX_PARTS} parts")
        partial = _partial_sums(q.device, heads, dv, n * parts)
    check(library().cw_window_attention(
        _ptr(q), q.stride(0) if n > 1 else max(q.stride(0), q.shape[1]), _ptr(cache_rows), _ptr(block_tables), block_tables.shape[1],
        cache_rows.shape[1], cache_rows.shape[0], _ptr(positions), _ptr(tok_seq), n, heads, kv_heads, dk, dv, int(window), float(scale),
        _ptr(head_scale), _ptr(talk), _ptr(head_bias), 1 if sigmoid_weights else 0, 1 if blocked else 0, _ptr(sink), _ptr(out), parts,
        _ptr(partial),
        _ptr(q_start), q_start.shape[0] - 1, dtype_code(q.dtype), _ptr(status),
        float(softcap), _ptr(slopes), float(coef), int(every), _ptr(gate), (gate.stride(0) if n > 1 else max(gate.stride(0), gate.shape[1])) if gate is not None else 0,
        int(pool), _ptr(pool_rows_cache) if pool else None, _ptr(pool_tables) if pool else None, pool_tables.shape[1] if pool else 0,
        pool_rows_cache.shape[0] if pool else 0, _stream()), "window_attention")
    return out
