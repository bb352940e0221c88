"""Mixers that carry a state of fixed size per request instead of a cache of keys.

``mamba2`` (state-space duality form).  Parameters: ``hidden_size, heads, vdim, state, groups, conv,
norm_groups, eps``.  With inner = heads*vdim, the input product yields ``[z | x | B | C | dt]`` (widths
inner, inner, groups*state, groups*state, heads).  x, B and C pass a causal per-channel convolution of
``conv`` taps (tensor ``conv`` [channels, taps], the current token's tap last, bias ``conv.b``) and
SiLU.  ``dt = softplus(dt + dt_bias)``; per head (its B and C are those of group head // (heads/groups)):
``S <- exp(-exp(A_log) dt) S + dt B x^T`` (S is state x vdim), ``y = S^T C + D x``.  Then ``y silu(z)``
is RMS-normed in ``norm_groups`` equal parts, times ``norm``, and goes through ``o``.  Per request the
state slot holds S of every head and the last conv-1 inputs of the convolution.

``wkv`` (time mixing in the manner of RWKV).  Parameters: ``hidden_size, heads, dim, eps``; the inner size of the decay's
two products is whatever the checkpoint's ``w1`` has (``decay_rank`` only sizes random weights).  With x' the
previous token's input (zeros before the first), each of r, k, v, g, w reads ``x + (x' - x) mu_s``;
``r, k, v`` are products of their mixes, ``gate = silu(g product)``, ``w = exp(-exp(w2 tanh(w1 mix_w) + w0))``
per head and key channel.  Per head ``o = (S + diag(u) k v^T)^T r`` and then ``S <- diag(w) S + k v^T``.
Each head's o is divided by its root mean square, times ``norm``, times the gate, and goes through ``o``.
The state slot holds S of every head and the previous token's input.

``gated_linear`` (linear attention with a decay per key channel that the input chooses).  Parameters:
``hidden_size, heads, dim, vdim, tau, eps``; the inner size of the decay's two products is whatever the
checkpoint's ``a1`` has (``decay_rank`` only sizes random weights).  ``q = (W_q x) dim^(-1/2)``, ``k, v`` plain
products, ``a = sigmoid(W_a2 (W_a1 x) + b)^(1/tau)`` per head and key channel; per head ``S <- diag(a) S + k v^T``,
``o = S^T q`` (after the update).  Each head's o is divided by its root mean square over vdim, times ``norm`` (one
weight of vdim entries for all heads), times ``silu(W_g x)``, and goes through ``o``.  The state slot holds S.

``decay_linear`` (linear attention with one constant decay per head).  Parameters: ``hidden_size, heads, dim,
vdim, decay`` (a number per head), ``eps``.  ``q, k, v = silu(W_q x), silu(W_k x), silu(W_v x)``; per head
``S <- decay_h S + k v^T``, ``o = S^T q``.  The heads' outputs together are divided by their root mean square, times
``norm``, times ``sigmoid(W_g x)``, and go through ``o``.  The state slot holds S.

``channel_delta`` (gated delta rule with a decay per key channel).  Parameters: ``hidden_size, heads, kv_heads, dim, vdim,
conv, eps``; the inner sizes of the decay's and the gate's two products are whatever the checkpoint's ``a1`` and ``g1``
have.  ``q, k`` (kv_heads x dim) and ``v`` (heads x vdim) are products of the input that pass a causal per-channel
convolution of ``conv`` taps (tensors ``q.conv, k.conv, v.conv`` [channels, taps], the current token's tap last, no bias)
and SiLU; q and k are then divided per head by ``sqrt(sum of squares + 1e-6)``, q also by ``sqrt(dim)``; head h reads
q/k head ``h // (heads / kv_heads)``.  ``beta = sigmoid(W_b x)`` per head, ``a = exp(-exp(A_log[h]) softplus(W_a2 W_a1 x +
dt_bias))`` per head and key channel.  Per head ``S <- diag(a) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.  Each
head's o is divided by its root mean square, times ``norm`` (vdim entries, shared), times ``sigmoid(W_g2 W_g1 x)``, and goes
through ``o``.  The state slot holds S of every head and the last conv-1 inputs of the convolution.

``matrix_memory`` (a matrix memory with exponential gates kept stable by a running maximum).  Parameters: ``hidden_size,
heads, dim, vdim, gate_cap, eps``.  ``q = W_q x / sqrt(dim)``, ``k, v`` plain products; per head ``li = cap tanh((W_i x +
b_i)/cap)``, ``lf = log sigmoid(cap tanh((W_f x + b_f)/cap))``, ``m_t = max(lf + m_(t-1), li)`` (m is 0 before the first
token), ``S <- exp(lf + m_(t-1) - m_t) S + exp(li - m_t) k v^T`` and the same for ``n`` with k alone, ``o = S^T q /
(max(|n . q|, exp(-m_t)) + 1e-6)``.  Each head's o is divided by its root mean square, times ``norm`` (all heads' width),
times ``sigmoid(W_g x)``, and goes through ``o``.  The state slot holds S with n as one more value column, and m.

``hgrn2`` (linear attention whose forget gate also decides what is written).  Parameters: ``hidden_size, heads, dim, vdim,
eps``.  ``q = silu(W_q x)``, ``v = W_v x``, ``f = l + (1 - l) sigmoid(W_f x + b_f)`` per head and key channel with the lower
bound ``l`` (tensor ``lower`` [heads*dim]); per head ``S <- diag(f) S + (1 - f) v^T``, ``o = S^T q`` (after the update; there is
no key and no other scale).  Each head's o is divided by its root mean square over vdim, times ``norm`` (vdim entries, shared
by the heads), and goes through ``o``.  The state slot holds S.

All run the recurrence itself, the decays, step sizes and norms in float32 in either run precision;
the products that feed them write float32.  ``mix`` returns the output product as float32 for a mixer that
stands beside another (``side_by_side``).
"""

from __future__ import annotations

import torch

from ..ops import gemm as gemm_ops
from ..ops import recurrence as rec_ops
from ..weights.decl import TensorDecl
from .base import Mixer, ResidualStream, SlotStateNeed, StateView, StepContext
from .linear import Linear
from .registry import register_mixer


class Mamba2Mixer(Mixer):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.vdim, self.state_size = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["conv"]), int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        if self.heads % self.groups:
            raise ValueError(f"heads {self.heads} not a multiple of groups {self.groups}")
        if self.inner % self.norm_groups:
            raise ValueError(f"inner size {self.inner} not a multiple of norm_groups {self.norm_groups}")
        if self.taps < 1:
            raise ValueError("conv must be at least 1")
        self.channels = self.inner + 2 * self.groups * self.state_size
        self.proj_width = 2 * self.inner + 2 * self.groups * self.state_size + self.heads
        # the layout of a request's state row
        self.scan_offset = 0
        self.conv_offset = self.heads * self.state_size * self.vdim

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.conv_offset + (self.taps - 1) * self.channels,))

    def tensor_decls(self):
        yield TensorDecl(self.name("in"), (self.proj_width, self.hidden_size), "matrix", "linear")
        yield TensorDecl(self.name("conv"), (self.channels, self.taps), "vector", "norm")
        yield TensorDecl(self.name("conv.b"), (self.channels,), "vector", "bias")
        yield TensorDecl(self.name("dt_bias"), (self.heads,), "vector", "bias")
        yield TensorDecl(self.name("A_log"), (self.heads,), "vector", "bias")
        yield TensorDecl(self.name("D"), (self.heads,), "vector", "norm")
        yield TensorDecl(self.name("norm"), (self.inner,), "vector", "norm")
        yield TensorDecl(self.name("o"), (self.hidden_size, self.inner), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.w_in = Linear(fetch(self.name("in")))
        self.conv_w, self.conv_b = fetch(self.name("conv")), fetch(self.name("conv.b"))
        self.dt_bias, self.a_log, self.skip = fetch(self.name("dt_bias")), fetch(self.name("A_log")), fetch(self.name("D"))
        self.norm_w = fetch(self.name("norm"))
        self.o = Linear(fetch(self.name("o")))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        inner, gn = self.inner, self.groups * self.state_size
        proj = self.w_in.to_float32(x)  # [N, z | x | B | C | dt], float32
        xbc_raw = proj[:, inner : inner + self.channels]
        xbc = rec_ops.causal_conv(xbc_raw, self.conv_w, self.conv_b, view, self.conv_offset, ctx)
        rec_ops.carry_rows(xbc_raw, self.taps - 1, view, self.conv_offset, ctx)  # after the convolution has read the old rows
        y = rec_ops.recurrence_scan(
            rec_ops.FORM_STEP_SIZE, q=xbc[:, inner + gn :], k=xbc[:, inner : inner + gn], v=xbc[:, :inner],
            pre=proj[:, inner + self.channels :], p0=self.dt_bias, p1=self.a_log, p2=self.skip, view=view,
            offset=self.scan_offset, ctx=ctx, heads=self.heads, dk=self.state_size, dv=self.vdim,
            heads_per_group=self.heads // self.groups)
        out = rec_ops.gated_group_norm(y, proj[:, :inner], self.norm_w, self.norm_groups, self.eps, True, self.dtype)
        return self.o.add_or_defer(out, stream)


class WkvMixer(Mixer):
    graph_safe = True
    graph_safe_portions = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.decay_rank = int(p["heads"]), int(p["dim"]), int(p.get("decay_rank") or 32)
        self.eps = float(p["eps"])
        self.inner = self.heads * self.dim
        self.scan_offset = 0
        self.shift_offset = self.heads * self.dim * self.dim

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.shift_offset + self.hidden_size,))

    def tensor_decls(self):
        h, a = self.hidden_size, self.inner
        for s in self.MIXES:
            yield TensorDecl(self.name(f"mu.{s}"), (h,), "vector", "bias")
        for s in ("r", "k", "v", "g"):
            yield TensorDecl(self.name(s), (a, h), "matrix", "linear")
        yield TensorDecl(self.name("w1"), (self.decay_rank, h), "matrix", "linear", free_dims=(0,))
        yield TensorDecl(self.name("w2"), (a, self.decay_rank), "matrix", "linear", free_dims=(1,))
        yield TensorDecl(self.name("w0"), (a,), "vector", "bias")
        yield TensorDecl(self.name("u"), (self.heads, self.dim), "vector", "bias")
        yield TensorDecl(self.name("norm"), (a,), "vector", "norm")
        yield TensorDecl(self.name("o"), (h, a), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.mu = torch.stack([fetch(self.name(f"mu.{s}")) for s in self.MIXES]).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (Linear(fetch(self.name(s))) for s in ("r", "k", "v", "g"))
        self.w1, self.w2 = Linear(fetch(self.name("w1"))), Linear(fetch(self.name("w2")))
        if self.w1.out_features != self.w2.in_features:
            raise ValueError(f"{self.name('w1')} has {self.w1.out_features} rows, {self.name('w2')} {self.w2.in_features} columns")
        self.w0 = fetch(self.name("w0"))
        self.bonus = fetch(self.name("u")).reshape(-1).contiguous()
        self.norm_w = fetch(self.name("norm"))
        self.o = Linear(fetch(self.name("o")))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        mixes = rec_ops.shift_mix(x, self.mu, view, self.shift_offset, ctx)  # [5, N, H]
        rec_ops.carry_rows(x, 1, view, self.shift_offset, ctx)  # after the mixes have read the old row
        r, k, v, g = (w.to_float32(mixes[i]) for i, w in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)))
        pre = self.w2.to_float32(rec_ops.activation_(self.w1(mixes[4]), rec_ops.ACT_TANH))
        o = rec_ops.recurrence_scan(rec_ops.FORM_CHANNEL_DECAY, q=r, k=k, v=v, pre=pre, p0=self.w0, p1=self.bonus, p2=None,
                                    view=view, offset=self.scan_offset, ctx=ctx, heads=self.heads, dk=self.dim, dv=self.dim)
        out = rec_ops.gated_group_norm(o, g, self.norm_w, self.heads, self.eps, False, self.dtype)
        return self.o.add_or_defer(out, stream)


class _LinearAttention(Mixer):
    """What the two linear-attention mixers share: one product for ``[q | k | v | gate]`` with float32 output, the
    state of heads*dim*vdim numbers, and the output product."""

    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        if min(self.heads, self.dim, self.vdim) <= 0:
            raise ValueError("heads, dim and vdim must be positive")
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.heads * self.dim * self.vdim,))

    def _projection_decls(self):
        h = self.hidden_size
        for s, out in (("q", self.qk), ("k", self.qk), ("v", self.inner), ("g", self.inner)):
            yield TensorDecl(self.name(s), (out, h), "matrix", "linear")
        yield TensorDecl(self.name("o"), (h, self.inner), "matrix", "linear")

    def _load_projections(self, fetch) -> None:
        self.w_in = Linear(torch.cat([fetch(self.name(s)) for s in ("q", "k", "v", "g")], dim=0).contiguous())
        self.o = Linear(fetch(self.name("o")))

    def _split(self, proj):
        qk, inner = self.qk, self.inner
        return proj[:, :qk], proj[:, qk : 2 * qk], proj[:, 2 * qk : 2 * qk + inner], proj[:, 2 * qk + inner :]

    def mix(self, ctx: StepContext, x, view: StateView):
        return self.o.to_float32(self._gated_output(ctx, x, view))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        return self.o.add_or_defer(self._gated_output(ctx, x, view), stream)


class GatedLinearMixer(_LinearAttention):
    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.tau = float(spec["tau"])
        self.decay_rank = int(spec.get("decay_rank") or 16)
        if self.tau <= 0:
            raise ValueError("tau must be positive")

    def tensor_decls(self):
        yield from self._projection_decls()
        yield TensorDecl(self.name("a1"), (self.decay_rank, self.hidden_size), "matrix", "linear", free_dims=(0,))
        yield TensorDecl(self.name("a2"), (self.qk, self.decay_rank), "matrix", "linear", free_dims=(1,))
        yield TensorDecl(self.name("a2.b"), (self.qk,), "vector", "bias")
        yield TensorDecl(self.name("norm"), (self.vdim,), "vector", "norm")

    def load_weights(self, fetch) -> None:
        self._load_projections(fetch)
        self.a1 = Linear(fetch(self.name("a1")))
        self.a2 = Linear(fetch(self.name("a2")), fetch(self.name("a2.b")))
        if self.a1.out_features != self.a2.in_features:
            raise ValueError(f"{self.name('a1')} has {self.a1.out_features} rows, {self.name('a2')} {self.a2.in_features} columns")
        self.norm_w = fetch(self.name("norm")).contiguous()

    def _gated_output(self, ctx: StepContext, x, view: StateView):
        q, k, v, g = self._split(self.w_in.to_float32(x))
        decay = rec_ops.sigmoid_power_decay_(self.a2.to_float32(self.a1(x)), self.tau)
        o = rec_ops.recurrence_scan(rec_ops.FORM_CHANNEL_DECAY_AFTER, q=q, k=k, v=v, pre=decay, p0=None, p1=None, p2=None, view=view,
                                    offset=0, ctx=ctx, heads=self.heads, dk=self.dim, dv=self.vdim, q_scale=self.dim ** -0.5)
        return rec_ops.gated_group_norm(o, g, self.norm_w, self.heads, self.eps, False, self.dtype, gate=rec_ops.GATE_SILU,
                                        shared_weight=True)


class DecayLinearMixer(_LinearAttention):
    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        decay = [float(d) for d in spec["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"decay has {len(decay)} numbers for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32).to(device)

    def tensor_decls(self):
        yield from self._projection_decls()
        yield TensorDecl(self.name("norm"), (self.inner,), "vector", "norm")

    def load_weights(self, fetch) -> None:
        self._load_projections(fetch)
        self.norm_w = fetch(self.name("norm")).contiguous()

    def _gated_output(self, ctx: StepContext, x, view: StateView):
        proj = rec_ops.activation_cols_(self.w_in.to_float32(x), 2 * self.qk + self.inner, rec_ops.ACT_SILU)  # q, k, v; not the gate
        q, k, v, g = self._split(proj)
        o = rec_ops.recurrence_scan(rec_ops.FORM_HEAD_DECAY, q=q, k=k, v=v, pre=None, p0=self.decay, p1=None, p2=None, view=view,
                                    offset=0, ctx=ctx, heads=self.heads, dk=self.dim, dv=self.vdim)
        return rec_ops.gated_group_norm(o, g, self.norm_w, 1, self.eps, False, self.dtype, gate=rec_ops.GATE_SIGMOID)


class BoundedForgetMixer(Mixer):
    """``hgrn2``: see the module's text.  One product for ``[q | f | v]`` with float32 output; one kernel makes silu(q), the
    gates f and 1 - f; the scan is the one of ``gated_linear`` with 1 - f in the key's place."""

    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        if min(self.heads, self.dim, self.vdim) <= 0:
            raise ValueError("heads, dim and vdim must be positive")
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.heads * self.dim * self.vdim,))

    def tensor_decls(self):
        h = self.hidden_size
        yield TensorDecl(self.name("q"), (self.qk, h), "matrix", "linear")
        yield TensorDecl(self.name("f"), (self.qk, h), "matrix", "linear")
        yield TensorDecl(self.name("f.b"), (self.qk,), "vector", "bias")
        yield TensorDecl(self.name("lower"), (self.qk,), "vector", "unit_interval")
        yield TensorDecl(self.name("v"), (self.inner, h), "matrix", "linear")
        yield TensorDecl(self.name("norm"), (self.vdim,), "vector", "norm")
        yield TensorDecl(self.name("o"), (h, self.inner), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.w_in = Linear(torch.cat([fetch(self.name(s)) for s in ("q", "f", "v")], dim=0).contiguous())
        self.f_bias = fetch(self.name("f.b")).contiguous()
        self.lower = fetch(self.name("lower")).contiguous()
        self.norm_w = fetch(self.name("norm")).contiguous()
        self.o = Linear(fetch(self.name("o")))

    def _normed_output(self, ctx: StepContext, x, view: StateView):
        qk = self.qk
        proj = self.w_in.to_float32(x)  # [N, q | f | v], float32
        take = rec_ops.bounded_forget_(proj, qk, self.f_bias, self.lower)  # q <- silu(q), f in place, 1 - f
        o = rec_ops.recurrence_scan(rec_ops.FORM_CHANNEL_DECAY_AFTER, q=proj[:, :qk], k=take, v=proj[:, 2 * qk :], pre=proj[:, qk : 2 * qk],
                                    p0=None, p1=None, p2=None, view=view, offset=0, ctx=ctx, heads=self.heads, dk=self.dim, dv=self.vdim)
        return rec_ops.gated_group_norm(o, None, self.norm_w, self.heads, self.eps, False, self.dtype, gate=rec_ops.GATE_NONE,
                                        shared_weight=True)

    def mix(self, ctx: StepContext, x, view: StateView):
        return self.o.to_float32(self._normed_output(ctx, x, view))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        return self.o.add_or_defer(self._normed_output(ctx, x, view), stream)


class ChannelDeltaMixer(Mixer):
    graph_safe = True
    graph_safe_portions = True
    UNIT_EPS = 1e-6  # inside the root of the unit vectors' lengths

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps = float(p["eps"])
        self.decay_rank, self.gate_rank = int(p.get("decay_rank") or 16), int(p.get("gate_rank") or 16)
        if min(self.heads, self.kv_heads, self.dim, self.vdim, self.taps) <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a positive multiple of kv_heads {self.kv_heads}; dim, vdim, conv positive")
        self.qk, self.inner = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk + self.inner       # what passes the convolution: q, k, v
        self.decays = self.heads * self.dim
        self.scan_offset = 0
        self.conv_offset = self.heads * self.dim * self.vdim

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.conv_offset + (self.taps - 1) * self.channels,))

    def tensor_decls(self):
        h = self.hidden_size
        for s, out in (("q", self.qk), ("k", self.qk), ("v", self.inner)):
            yield TensorDecl(self.name(s), (out, h), "matrix", "linear")
            yield TensorDecl(self.name(f"{s}.conv"), (out, self.taps), "vector", "norm")
        yield TensorDecl(self.name("b"), (self.heads, h), "matrix", "linear")
        yield TensorDecl(self.name("A_log"), (self.heads,), "vector", "bias")
        yield TensorDecl(self.name("norm"), (self.vdim,), "vector", "norm")
        yield TensorDecl(self.name("a1"), (self.decay_rank, h), "matrix", "linear", free_dims=(0,))
        yield TensorDecl(self.name("a2"), (self.decays, self.decay_rank), "matrix", "linear", free_dims=(1,))
        yield TensorDecl(self.name("dt_bias"), (self.decays,), "vector", "bias")
        yield TensorDecl(self.name("g1"), (self.gate_rank, h), "matrix", "linear", free_dims=(0,))
        yield TensorDecl(self.name("g2"), (self.inner, self.gate_rank), "matrix", "linear", free_dims=(1,))
        yield TensorDecl(self.name("o"), (h, self.inner), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.w_in = Linear(torch.cat([fetch(self.name(s)) for s in ("q", "k", "v", "b")], dim=0).contiguous())
        self.conv_w = torch.cat([fetch(self.name(f"{s}.conv")) for s in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = fetch(self.name("A_log")).contiguous(), fetch(self.name("dt_bias")).contiguous()
        self.norm_w = fetch(self.name("norm")).contiguous()
        self.a1, self.a2 = Linear(fetch(self.name("a1"))), Linear(fetch(self.name("a2")))
        self.g1, self.g2 = Linear(fetch(self.name("g1"))), Linear(fetch(self.name("g2")))
        for first, second in ((self.a1, self.a2), (self.g1, self.g2)):
            if first.out_features != second.in_features:
                raise ValueError(f"{self.prefix}: a product of {first.out_features} rows feeds one of {second.in_features} columns")
        self.o = Linear(fetch(self.name("o")))

    def _gated_output(self, ctx: StepContext, x, view: StateView):
        qk, c = self.qk, self.channels
        proj = self.w_in.to_float32(x)  # [N, q | k | v | beta], float32
        raw = proj[:, :c]
        qkv = rec_ops.causal_conv(raw, self.conv_w, None, view, self.conv_offset, ctx)
        rec_ops.carry_rows(raw, self.taps - 1, view, self.conv_offset, ctx)  # after the convolution has read the old rows
        rec_ops.unit_heads_(qkv, 2 * self.kv_heads, self.dim, self.UNIT_EPS, self.kv_heads, self.dim ** -0.5)
        pre = self.a2.to_float32(self.a1(x))
        o = rec_ops.delta_scan(q=qkv[:, :qk], k=qkv[:, qk : 2 * qk], v=qkv[:, 2 * qk :], pre=pre, beta=proj[:, c:],
                               dt_bias=self.dt_bias, a_log=self.a_log, view=view, offset=self.scan_offset, ctx=ctx, heads=self.heads,
                               dk=self.dim, dv=self.vdim, heads_per_group=self.heads // self.kv_heads)
        gate = self.g2.to_float32(self.g1(x))
        return rec_ops.gated_group_norm(o, gate, self.norm_w, self.heads, self.eps, False, self.dtype, gate=rec_ops.GATE_SIGMOID,
                                        shared_weight=True)

    def mix(self, ctx: StepContext, x, view: StateView):
        return self.o.to_float32(self._gated_output(ctx, x, view))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        return self.o.add_or_defer(self._gated_output(ctx, x, view), stream)


class MatrixMemoryMixer(Mixer):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        if min(self.heads, self.dim, self.vdim) <= 0 or not self.cap > 0:
            raise ValueError("heads, dim, vdim and gate_cap must be positive")
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.scan_offset = 0
        self.max_offset = self.heads * (self.vdim + 1) * self.dim  # behind S and n: the running maximum of every head

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((self.max_offset + self.heads,))

    def tensor_decls(self):
        h = self.hidden_size
        for s, out in (("q", self.qk), ("k", self.qk), ("v", self.inner), ("g", self.inner), ("i", self.heads), ("f", self.heads)):
            yield TensorDecl(self.name(s), (out, h), "matrix", "linear")
        yield TensorDecl(self.name("i.b"), (self.heads,), "vector", "bias")
        yield TensorDecl(self.name("f.b"), (self.heads,), "vector", "bias")
        yield TensorDecl(self.name("norm"), (self.inner,), "vector", "norm")
        yield TensorDecl(self.name("o"), (h, self.inner), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.w_in = Linear(torch.cat([fetch(self.name(s)) for s in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous())
        self.bias_i, self.bias_f = fetch(self.name("i.b")).contiguous(), fetch(self.name("f.b")).contiguous()
        self.norm_w = fetch(self.name("norm")).contiguous()
        self.o = Linear(fetch(self.name("o")))

    def _gated_output(self, ctx: StepContext, x, view: StateView):
        qk, inner, h = self.qk, self.inner, self.heads
        proj = self.w_in.to_float32(x)  # [N, q | k | v | gate | input gate | forget gate], float32
        at = 2 * qk + 2 * inner
        coef = rec_ops.gate_scan(proj[:, at : at + h], proj[:, at + h :], self.bias_i, self.bias_f, self.cap, view, self.max_offset, ctx, h)
        y = rec_ops.recurrence_scan(rec_ops.FORM_GATED_WITH_KEY_SUM, q=proj[:, :qk], k=proj[:, qk : 2 * qk], v=proj[:, 2 * qk : 2 * qk + inner],
                                    pre=coef, p0=None, p1=None, p2=None, view=view, offset=self.scan_offset, ctx=ctx, heads=h, dk=self.dim,
                                    dv=self.vdim + 1, q_scale=self.dim ** -0.5)
        return rec_ops.memory_norm(y, coef[:, 2 * h :], proj[:, 2 * qk + inner : at], self.norm_w, h, self.vdim, self.eps, self.dtype)

    def mix(self, ctx: StepContext, x, view: StateView):
        return self.o.to_float32(self._gated_output(ctx, x, view))

    def forward(self, ctx: StepContext, x, view: StateView, stream: ResidualStream):
        return self.o.add_or_defer(self._gated_output(ctx, x, view), stream)


register_mixer("hgrn2", BoundedForgetMixer, replace=True)
register_mixer("channel_delta", ChannelDeltaMixer, replace=True)
register_mixer("matrix_memory", MatrixMemoryMixer, replace=True)
register_mixer("gated_linear", GatedLinearMixer, replace=True)
register_mixer("decay_linear", DecayLinearMixer, replace=True)
register_mixer("mamba2", Mamba2Mixer, replace=True)
register_mixer("wkv", WkvMixer, replace=True)
