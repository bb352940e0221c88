"""Python faces of the products in groups and of the mixture-of-experts kernels (``csrc/grouped_gemm.cu``)."""

from __future__ import annotations

import torch

from . import _need, _ptr, _stream, dtype_code
from .library import check, library

EPI_STORE, EPI_STORE_F32, EPI_SILU_MUL, EPI_SIGMOID_GATE = 0, 1, 2, 3


def set_tensor_cores(on: bool) -> None:
    """bfloat16 products in groups run on the tensor cores when their sizes allow (the default); ``False`` keeps them
    on the CUDA-core kernel that float32 runs use (for comparisons)."""
    library().cw_grouped_gemm_set_mma(1 if on else 0)


def per_head_product(a: torch.Tensor, a_head_width: int, w: torch.Tensor, out: torch.Tensor, out_head_width: int,
                     gate: torch.Tensor | None = None) -> torch.Tensor:
    """For every head h: ``out[:, h*out_head_width : +n] = a[:, h*a_head_width : +k] @ w[h].T`` with ``w`` [H, n, k];
    with ``gate`` (same layout as ``out``) the result is multiplied by sigmoid(gate)."""
    _need(a, None, "a", 2)
    _need(w, a.dtype, "w", 3)
    _need(out, a.dtype, "out", 2)
    heads, n, k = w.shape
    rows = a.shape[0]
    if gate is not None:
        _need(gate, a.dtype, "gate", 2)
    check(library().cw_grouped_gemm(_ptr(a), a.shape[1], a_head_width, _ptr(w), None, n * k, _ptr(out), out.shape[1], out_head_width,
                                    None, None, 1, None, _ptr(gate), gate.shape[1] if gate is not None else 0, rows, n, k, heads,
                                    EPI_SIGMOID_GATE if gate is not None else EPI_STORE, 0.0, dtype_code(a.dtype), _stream()),
          "per_head_product")
    return out


SCORE_CHOSEN, SCORE_ALL, SCORE_SIGMOID = 0, 1, 2


def moe_choose(logits: torch.Tensor, bias: torch.Tensor | None, tok_seq: torch.Tensor, top: int, scoring: int = SCORE_CHOSEN,
               groups: int = 1, keep: int = 1, correction: torch.Tensor | None = None, weight_scale: float = 1.0,
               group_rank: int = 1):
    """(chosen experts int32 [N, top], their weights float32 [N, top]) from float32 router logits [N, E] (+ bias): the
    ``top`` largest, weighted by the softmax over the chosen ones (``SCORE_CHOSEN``) or by their shares of the softmax
    over all experts, not renormalised (``SCORE_ALL``); ``SCORE_SIGMOID``: an expert's score is the sigmoid of its logit,
    experts are ranked by score + ``correction`` [E] and weighted by the score alone.  With ``groups`` > 1 only experts of
    the ``keep`` best of ``groups`` equal runs of neighbours can be chosen (a run counts as the sum of its ``group_rank``
    largest entries).  Every weight is multiplied by ``weight_scale``.  Padding rows choose -1."""
    _need(logits, torch.float32, "logits", 2)
    n, e = logits.shape
    if correction is not None:
        _need(correction, torch.float32, "correction", 1)
        if correction.shape[0] != e or scoring != SCORE_SIGMOID:
            raise ValueError("a correction per expert goes with sigmoid scores")
    sel = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(library().cw_moe_choose(_ptr(logits), _ptr(bias), _ptr(tok_seq), _ptr(sel), _ptr(wt), n, e, top, int(scoring), int(groups), int(keep),
                                  _ptr(correction), float(weight_scale), int(group_rank), _stream()), "moe_choose")
    return sel, wt


def moe_group(sel: torch.Tensor, experts: int):
    """(offsets int32 [experts+1], order int32 [pairs]): the (token, choice) pairs sorted by expert."""
    pairs = sel.numel()
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=sel.device)
    order = torch.empty(pairs, dtype=torch.int32, device=sel.device)
    rank = torch.empty(pairs, dtype=torch.int32, device=sel.device)
    check(library().cw_moe_group(_ptr(sel), _ptr(offsets), _ptr(order), _ptr(rank), pairs, experts, _stream()), "moe_group")
    return offsets, order


def expert_gate_up(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, offsets: torch.Tensor | None, order: torch.Tensor | None,
                   top: int, limit: float = 0.0) -> torch.Tensor:
    """silu(x Wg_e^T) * (x Wu_e^T) for every pair, rows in sorted order; weights [E, ff, W].  With a positive ``limit`` the
    clamped form ``a sigmoid(1.702 a) (b + 1)``, ``a = min(x Wg^T, limit)``, ``b = clamp(x Wu^T, -limit, limit)``.
    ``offsets`` and ``order`` None: every row of ``x`` through every one of the E matrices (one: a dense layer)."""
    experts, ff, w = w_gate.shape
    pairs = order.numel() if order is not None else x.shape[0]
    act = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
    check(library().cw_grouped_gemm(_ptr(x), x.shape[1], 0, _ptr(w_gate), _ptr(w_up), ff * w, _ptr(act), ff, 0, _ptr(offsets),
                                    _ptr(order), top, None, None, 0, pairs, ff, w, experts, EPI_SILU_MUL, float(limit), dtype_code(x.dtype),
                                    _stream()), "expert_gate_up")
    return act


def expert_down(act: torch.Tensor, w_down: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    """float32 [pairs, W] in pair order (token * top + choice); weights [E, W, ff]."""
    experts, w, ff = w_down.shape
    pairs = order.numel()
    y = torch.empty((pairs, w), dtype=torch.float32, device=act.device)
    check(library().cw_grouped_gemm(_ptr(act), ff, 0, _ptr(w_down), None, w * ff, _ptr(y), w, 0, _ptr(offsets), None, 1, _ptr(order),
                                    None, 0, pairs, w, ff, experts, EPI_STORE_F32, 0.0, dtype_code(act.dtype), _stream()), "expert_down")
    return y


def moe_combine(residual: torch.Tensor, y: torch.Tensor, sel: torch.Tensor, wt: torch.Tensor, assign: bool = False) -> None:
    """residual[n] += sum over the choices, in order, of weight * y[n*top + choice]; ``assign``: the sum replaces
    residual[n] (zeros in rows that chose nothing)."""
    _need(residual, torch.float32, "residual", 2)
    n, w = residual.shape
    check(library().cw_moe_combine(_ptr(residual), _ptr(y), _ptr(sel), _ptr(wt), n, w, sel.shape[1], 1 if assign else 0, _stream()),
          "moe_combine")
