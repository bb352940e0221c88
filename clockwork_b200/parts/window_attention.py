"""Grouped-query attention over a sliding window, for layers whose keys and values have different sizes and
whose scores are not just a scaled dot product.

Parameters: ``hidden_size, heads, kv_heads, dim`` (query/key size per head), ``vdim`` (value size per head),
``window`` (position t sees positions j with 0 <= t - j < window; None: every j <= t), ``scale``, and the switches

* ``bias``: q, k, v and the output product have biases (tensors ``q.b, k.b, v.b, o.b``); ``out_bias`` (by default the same
  as ``bias``) says it for the output product alone;
* ``head_scale``: the score of head h is multiplied by ``temp[h]``;
* ``talk``: the heads' scores are mixed before they become weights, ``s_h <- sum_g talk[h, g] s_g``;
* ``head_bias``: ``pb[h]`` is added to the (mixed) score;
* ``weights``: ``"softmax"`` over the visible keys, or ``"sigmoid"`` of each score on its own (not normalised);
* ``mask``: ``"window"`` (the default: the last ``window`` positions) or ``"block"``: positions are cut into blocks of
  ``window`` counted from the start of the sequence, and position t sees the positions j <= t of its own block;
* ``sink``: the softmax's denominator also holds ``exp(sink[h])``, a learned logit per head without key or value
  (tensor ``sink`` [heads]); ``"zero"``: the logit is 0 for every head and there is no tensor (one is added to the denominator);
* ``pool``: beside the window, every block of ``pool`` positions (counted from the start of the sequence) that ends at or
  before t - window is seen as one key and one value, the means of the block's cached keys and values; tokens that have
  left the window and whose block is not yet seen are not seen at all.  A second cache keeps one row per block;
* ``softcap``: the scaled score s becomes ``softcap tanh(s / softcap)``;
* ``distance_bias``: ``{"halvings": c}``: ``2^(-c (h + 1) / heads) * (t - j)`` is taken off head h's (capped) score;
* ``query_temperature``: ``{"coef", "every"}``: the query at position t is multiplied by ``1 + coef ln(floor((t + 1) / every) + 1)``;
* ``gate``: head h's output is multiplied by ``sigmoid(W_g x)_h`` before the output product (tensor ``g`` [heads, hidden]);
* ``rotary``: ``{"dims", "base"}``: the first ``dims`` entries of every query and key head are rotated by the token's
  position before the key is cached, entry i with entry i + dims/2 by the angle ``t * base^(-2i/dims)`` (float32).

Without ``rotary`` positions do not enter the scores.  Tensors: ``q`` [heads*dim, hidden], ``k`` [kv_heads*dim, hidden], ``v``
[kv_heads*vdim, hidden], ``o`` [hidden, heads*vdim], and those the switches name.

The cache keeps one row ``[key | value]`` per token and key/value head (``PagedKVNeed(planes=1)`` with rows of
``dim + vdim``), in a page group that gives pages back behind the window (with ``pool``: behind the window or the last ``pool`` positions,
whichever reaches farther back, since a block's mean is taken from the cached rows when its last token arrives; the blocks'
rows live in a page group of one row per ``pool`` positions, ``PagedKVNeed(every=pool)``).  At load the rows of k and v are
interleaved head by head behind q, so that one product yields ``[q | k_0 v_0 | k_1 v_1 ..]`` per token and the
cache write is a copy of the row's tail (with ``rotary`` the product's output is float32 and one kernel rotates,
rounds once and stores).  A blocked layer's page group gives back the pages of blocks that have passed.
Scores, weights and weighted sums are float32 in either run precision.
"""

from __future__ import annotations

import torch

from ..ops import window as window_ops
from ..weights.decl import TensorDecl
from .base import Mixer, PagedKVNeed, PagedView, ResidualStream, StepContext
from .linear import Linear
from .registry import register_mixer


class WindowAttention(Mixer):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.window = window_ops.NO_WINDOW if p.get("window") is None else int(p["window"])
        self.scale = float(p["scale"])
        self.bias = bool(p.get("bias", False))
        self.out_bias = bool(p.get("out_bias", self.bias))
        self.has_head_scale, self.has_talk, self.has_head_bias = (bool(p.get(k, False)) for k in ("head_scale", "talk", "head_bias"))
        self.weights = str(p.get("weights", "softmax"))
        if self.weights not in ("softmax", "sigmoid"):
            raise ValueError(f"weights must be 'softmax' or 'sigmoid', got {self.weights!r}")
        self.mask = str(p.get("mask", "window"))
        if self.mask not in ("window", "block"):
            raise ValueError(f"mask must be 'window' or 'block', got {self.mask!r}")
        self.has_sink = bool(p.get("sink", False))
        self.zero_sink = p.get("sink") == "zero"
        if self.has_sink and self.weights != "softmax":
            raise ValueError("a sink belongs to softmax weights")
        self.pool = int(p.get("pool") or 0)
        if self.pool < 0 or (self.pool and (self.mask != "window" or self.window >= window_ops.NO_WINDOW)):
            raise ValueError("pooled blocks lie before a sliding window of finite size")
        self.softcap = float(p.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError("softcap must be positive")
        bias = p.get("distance_bias")
        self.halvings = float(bias["halvings"]) if bias else 0.0
        if bias and self.pool:
            raise ValueError("a pooled block has no distance: distance_bias and pool exclude each other")
        temp = p.get("query_temperature")
        self.temperature = (float(temp["coef"]), int(temp["every"])) if temp else None
        if temp and self.temperature[1] < 1:
            raise ValueError("query_temperature.every must be at least 1")
        self.has_gate = bool(p.get("gate", False))
        self.slopes = None
        rotary = p.get("rotary")
        self.rot_dims = int(rotary["dims"]) if rotary else 0
        self.rot_base = float(rotary["base"]) if rotary else 0.0
        if rotary and (self.rot_dims <= 0 or self.rot_dims % 2 or self.rot_dims > int(p["dim"]) or self.rot_base <= 0):
            raise ValueError(f"rotary dims {self.rot_dims} must be even, positive and at most dim {p['dim']}, the base positive")
        self.inv_freq = self.sink = None
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} not a multiple of kv_heads {self.kv_heads}")
        if min(self.dim, self.vdim, self.window) <= 0:
            raise ValueError("dim, vdim and window must be positive")
        self.row = self.dim + self.vdim
        self.qkv: Linear | None = None
        self.o: Linear | None = None
        self.head_scale = self.talk = self.head_bias = None

    def cache_need(self):
        if self.mask == "block":
            return PagedKVNeed(self.kv_heads, self.row, None, planes=1, block=self.window)
        if self.window >= window_ops.NO_WINDOW:
            return PagedKVNeed(self.kv_heads, self.row, None, planes=1)
        if self.pool:
            # (a block's mean is read from the cached rows when its last token arrives: the last `pool` positions stay too)
            return (PagedKVNeed(self.kv_heads, self.row, max(self.window, self.pool), planes=1),
                    PagedKVNeed(self.kv_heads, self.row, None, planes=1, every=self.pool))
        return PagedKVNeed(self.kv_heads, self.row, self.window, planes=1)

    def reserve_for_steps(self, max_seqs: int, max_ctx: int) -> None:
        if self.device.type == "cuda":
            window_ops.reserve_window_scratch(self.device, self.heads, self.vdim)

    def tensor_decls(self):
        h = self.hidden_size
        for name, out in (("q", self.heads * self.dim), ("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)):
            yield TensorDecl(self.name(name), (out, h), "matrix", "linear")
            if self.bias:
                yield TensorDecl(self.name(f"{name}.b"), (out,), "vector", "bias")
        if self.has_head_scale:
            yield TensorDecl(self.name("temp"), (self.heads,), "vector", "norm")
        if self.has_talk:
            yield TensorDecl(self.name("talk"), (self.heads, self.heads), "vector", "norm")
        if self.has_head_bias:
            yield TensorDecl(self.name("pb"), (self.heads,), "vector", "bias")
        if self.has_sink and not self.zero_sink:
            yield TensorDecl(self.name("sink"), (self.heads,), "vector", "bias")
        if self.has_gate:
            yield TensorDecl(self.name("g"), (self.heads, h), "matrix", "linear")
        yield TensorDecl(self.name("o"), (h, self.heads * self.vdim), "matrix", "linear")
        if self.out_bias:
            yield TensorDecl(self.name("o.b"), (h,), "vector", "bias")

    def _rows_by_kv_head(self, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """k [G*dim, ..] and v [G*vdim, ..] as [G*(dim + vdim), ..]: head by head, the key's rows before the value's."""
        g = self.kv_heads
        tail = k.shape[1:]
        return torch.cat([k.reshape(g, self.dim, *tail), v.reshape(g, self.vdim, *tail)], dim=1).reshape(g * self.row, *tail)

    def load_weights(self, fetch) -> None:
        q, k, v = (fetch(self.name(n)) for n in ("q", "k", "v"))
        # (with a gate its rows come last: one product yields [q | k_0 v_0 | .. | gate logits])
        gate = [fetch(self.name("g"))] if self.has_gate else []
        w = torch.cat([q, self._rows_by_kv_head(k, v), *gate], dim=0).contiguous()
        b = None
        if self.bias:
            qb, kb, vb = (fetch(self.name(f"{n}.b")) for n in ("q", "k", "v"))
            b = torch.cat([qb, self._rows_by_kv_head(kb, vb), *([torch.zeros_like(qb[: self.heads])] if self.has_gate else [])],
                          dim=0).contiguous()
        self.qkv = Linear(w, b)
        self.o = Linear(fetch(self.name("o")), fetch(self.name("o.b")) if self.out_bias else None)
        if self.has_head_scale:
            self.head_scale = fetch(self.name("temp")).contiguous()
        if self.has_talk:
            self.talk = fetch(self.name("talk")).contiguous()
        if self.has_head_bias:
            self.head_bias = fetch(self.name("pb")).contiguous()
        if self.has_sink:
            self.sink = torch.zeros(self.heads, dtype=torch.float32, device=w.device) if self.zero_sink else fetch(self.name("sink")).contiguous()
        if self.halvings:
            h = torch.arange(1, self.heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -self.halvings * h / self.heads).to(torch.float32).to(w.device)
        if self.rot_dims:
            # base^(-2i/dims) worked out in float64 and rounded once
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.inv_freq = (self.rot_base ** (-2.0 * i / self.rot_dims)).to(torch.float32).to(self.qkv.weight.device)

    def _attend(self, ctx: StepContext, x: torch.Tensor, view) -> torch.Tensor:
        view, pooled = view if self.pool else (view, None)
        rows = view.k_cache  # [pages, page_size, kv_heads, dim + vdim]
        gate = None
        if self.rot_dims or self.has_gate:
            # the product in float32, so that rotated queries and keys are rounded to the run's precision once (and the
            # gate's logits not at all)
            proj = self.qkv.to_float32(x)
            q = window_ops.rotate_store(proj, ctx.positions, ctx.tok_seq, view.slots if view.write else None,
                                        self.inv_freq, self.heads, self.kv_heads, self.dim, self.vdim, self.rot_dims, rows, ctx.status)
            if self.has_gate:
                gate = proj[:, self.heads * self.dim + self.kv_heads * self.row :]
        else:
            q = self.qkv(x)  # [N, heads*dim | kv_heads*(dim + vdim)]
            if view.write:
                window_ops.store_rows(q, self.heads * self.dim, self.kv_heads * self.row, rows, view.slots, ctx.status)
        if self.pool and view.write:
            window_ops.pool_rows(rows, view.block_tables, ctx.positions, ctx.tok_seq, pooled.slots, pooled.k_cache, self.pool, ctx.status)
        parts = window_ops.window_parts(ctx.num_tokens, self.window, self.dtype, ctx.max_ctx_len)
        return window_ops.window_attention(q, rows, view.block_tables, ctx.positions, ctx.tok_seq, ctx.q_start, self.heads, self.kv_heads,
                                           self.dim, self.vdim, self.window, self.scale, self.head_scale, self.talk,
                                           self.head_bias, self.weights == "sigmoid", ctx.status, parts,
                                           blocked=self.mask == "block", sink=self.sink, softcap=self.softcap, slopes=self.slopes,
                                           temperature=self.temperature, gate=gate, pool=self.pool,
                                           pool_rows_cache=pooled.k_cache if self.pool else None,
                                           pool_tables=pooled.block_tables if self.pool else None)

    def mix(self, ctx: StepContext, x: torch.Tensor, view: PagedView) -> torch.Tensor:
        return self.o.to_float32(self._attend(ctx, x, view))

    def forward(self, ctx: StepContext, x: torch.Tensor, view: PagedView, stream: ResidualStream):
        return self.o.add_or_defer(self._attend(ctx, x, view), stream)


register_mixer("window_attention", WindowAttention, replace=True)
