"""Python faces of the kernels for layers that carry a state of fixed size from token to token
(``csrc/recurrence.cu``): token shift, short causal convolution, the rows kept for the next step,
the recurrence itself in its two forms, the gated norm in parts, and in-place activations.

A request's state is one float32 row of the cache manager's slot tensor (``StateView``); a part
lays several pieces out in that row and names each by its offset."""

from __future__ import annotations

import torch

from . import _need, _ptr, _stream, dtype_code
from .library import check, library

FORM_CHANNEL_DECAY, FORM_STEP_SIZE, FORM_CHANNEL_DECAY_AFTER, FORM_HEAD_DECAY, FORM_GATED_WITH_KEY_SUM = 0, 1, 2, 3, 4
ACT_GELU_TANH, ACT_TANH, ACT_SILU, ACT_SIGMOID = 0, 1, 2, 3
GATE_SILU, GATE_SIGMOID, GATE_NONE = 0, 1, 2


def _state_args(view) -> tuple:
    state = view.state
    _need(state, torch.float32, "state", 2)
    _need(view.slots, torch.int64, "state slots", 1)
    return state.data_ptr(), state.stride(0), view.slots.data_ptr()


def shift_mix(x: torch.Tensor, mu: torch.Tensor, view, offset: int, ctx) -> torch.Tensor:
    """[mixes, N, W]: ``x + (x_prev - x) * mu[s]``; the row before a portion's first comes from the state."""
    _need(x, None, "x", 2)
    _need(mu, torch.float32, "mu", 2)
    n, w = x.shape
    if mu.shape[1] != w:
        raise ValueError("mu must be [mixes, width]")
    out = torch.empty((mu.shape[0], n, w), dtype=x.dtype, device=x.device)
    state, stride, slots = _state_args(view)
    check(library().cw_shift_mix(_ptr(x), _ptr(mu), state, stride, offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start),
                                 _ptr(out), n, w, mu.shape[0], dtype_code(x.dtype), _stream()), "shift_mix")
    return out


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, view, offset: int, ctx) -> torch.Tensor:
    """silu(conv(x) + bias) per channel; ``x`` float32 [N, C] (may be a column slice), ``weight`` [C, taps]."""
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be float32 [N, C] with unit column stride")
    _need(weight, torch.float32, "weight", 2)
    n, c = x.shape
    if weight.shape[0] != c:
        raise ValueError("conv weight must be [channels, taps]")
    out = torch.empty((n, c), dtype=torch.float32, device=x.device)
    state, stride, slots = _state_args(view)
    check(library().cw_causal_conv(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), c), _ptr(weight), _ptr(bias), state, stride,
                                   offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start), _ptr(out), n, c, weight.shape[1],
                                   _stream()), "causal_conv")
    return out


def carry_rows(x: torch.Tensor, rows: int, view, offset: int, ctx) -> None:
    """Keeps the last ``rows`` rows of every request's portion of ``x`` [N, C] in its state (older kept rows shift)."""
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [N, C] with unit column stride")
    n, c = x.shape
    state, stride, slots = _state_args(view)
    check(library().cw_carry_rows(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), c), state, stride, offset, slots,
                                  _ptr(ctx.tok_seq), _ptr(ctx.q_start), ctx.num_seqs, c, rows, dtype_code(x.dtype), _stream()),
          "carry_rows")


def recurrence_scan(form: int, q, k, v, pre, p0, p1, p2, view, offset: int, ctx, heads: int, dk: int, dv: int,
                    heads_per_group: int = 1, q_scale: float = 1.0) -> torch.Tensor:
    """float32 [N, heads*dv].  ``q``, ``k`` [N, groups*dk], ``v`` [N, heads*dv], ``pre`` [N, heads*dk] (forms 0 and 2) or
    [N, heads] (form 1) or None (form 3): float32, unit column stride, any row stride.  The state piece at ``offset``
    holds heads*dk*dv numbers.  Form 0 turns ``pre`` into the decays in place (it is a product's output that nothing
    else reads); form 2 takes ``pre`` as the decays themselves (``sigmoid_power_decay``); form 3 takes a constant
    decay per head in ``p0``.  ``q_scale`` multiplies the outputs of forms 2 and 3."""
    for name, t in (("q", q), ("k", k), ("v", v), ("pre", pre)):
        if t is None and name == "pre" and form == FORM_HEAD_DECAY:
            continue
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be float32 [N, *] with unit column stride")
    n = v.shape[0]
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=v.device)
    state, stride, slots = _state_args(view)

    def ld(t):
        return t.stride(0) if n > 1 else max(t.stride(0), t.shape[1])

    # decays and step sizes once per token, ahead of the scan
    if form == FORM_CHANNEL_DECAY:
        check(library().cw_recurrence_coefficients(form, _ptr(pre), ld(pre), _ptr(p0), None, None, n, heads * dk, _stream()),
              "recurrence_coefficients")
    elif form == FORM_STEP_SIZE:
        coef = torch.empty((n, 2 * heads), dtype=torch.float32, device=v.device)
        check(library().cw_recurrence_coefficients(form, _ptr(pre), ld(pre), _ptr(p0), _ptr(p1), _ptr(coef), n, heads, _stream()),
              "recurrence_coefficients")
        pre = coef
    check(library().cw_recurrence_scan(form, _ptr(q), ld(q), _ptr(k), ld(k), _ptr(v), ld(v), _ptr(pre), 0 if pre is None else ld(pre),
                                       _ptr(p0), _ptr(p1), _ptr(p2), state, stride, offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start),
                                       ctx.num_seqs, heads, dk, dv, heads_per_group, _ptr(out), heads * dv, float(q_scale), _stream()),
          "recurrence_scan")
    return out


def unit_heads_(x: torch.Tensor, heads: int, dim: int, eps: float, leading: int, leading_scale: float, scale: float = 1.0) -> torch.Tensor:
    """In place on the first ``heads*dim`` columns of float32 ``x`` [N, C]: every head divided by ``sqrt(sum of squares + eps)``,
    the first ``leading`` heads then times ``leading_scale``, the others times ``scale``."""
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] < heads * dim:
        raise ValueError("x must be float32 [N, >= heads*dim] with unit column stride")
    n = x.shape[0]
    check(library().cw_unit_heads(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), x.shape[1]), n, heads, dim, float(eps), int(leading),
                                  float(leading_scale), float(scale), _stream()), "unit_heads")
    return x


def delta_scan(q, k, v, pre, beta, dt_bias, a_log, view, offset: int, ctx, heads: int, dk: int, dv: int,
               heads_per_group: int = 1) -> torch.Tensor:
    """float32 [N, heads*dv]: the gated delta rule ``S <- diag(a) S; u = beta (v - S^T k); S <- S + k u^T; y = S^T q`` per
    head, with ``a = exp(-exp(a_log[h]) softplus(pre + dt_bias))`` and ``beta = sigmoid(beta)``, both made in place from the
    products' outputs (nothing else reads them).  ``q``, ``k`` [N, groups*dk], ``v`` [N, heads*dv], ``pre`` [N, heads*dk],
    ``beta`` [N, heads]: float32, unit column stride, any row stride.  The state piece at ``offset`` holds heads*dk*dv numbers."""
    for name, t in (("q", q), ("k", k), ("v", v), ("pre", pre), ("beta", beta)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be float32 [N, *] with unit column stride")
    _need(dt_bias, torch.float32, "dt_bias", 1)
    _need(a_log, torch.float32, "a_log", 1)
    if dt_bias.shape[0] != heads * dk or a_log.shape[0] != heads:
        raise ValueError("dt_bias must have heads*dk entries and a_log heads")
    n = v.shape[0]
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=v.device)
    state, stride, slots = _state_args(view)

    def ld(t):
        return t.stride(0) if n > 1 else max(t.stride(0), t.shape[1])

    check(library().cw_delta_coefficients(_ptr(pre), ld(pre), _ptr(dt_bias), _ptr(a_log), _ptr(beta), ld(beta), n, heads, dk, _stream()),
          "delta_coefficients")
    check(library().cw_delta_scan(_ptr(q), ld(q), _ptr(k), ld(k), _ptr(v), ld(v), _ptr(pre), ld(pre), _ptr(beta), ld(beta), state, stride,
                                  offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start), ctx.num_seqs, heads, dk, dv, heads_per_group,
                                  _ptr(out), heads * dv, _stream()), "delta_scan")
    return out


def gate_scan(zi: torch.Tensor, zf: torch.Tensor, bias_i: torch.Tensor | None, bias_f: torch.Tensor | None, cap: float, view,
              offset: int, ctx, heads: int) -> torch.Tensor:
    """float32 [N, 3*heads] = ``[keep | take | floor]`` per token and head from the pre-activations of an input gate and a
    forget gate (``zi``, ``zf`` [N, heads], float32, any row stride): ``li = cap tanh((zi + bias_i)/cap)``,
    ``lf = log sigmoid(cap tanh((zf + bias_f)/cap))``, ``m_t = max(lf + m_(t-1), li)``, ``keep = exp(lf + m_(t-1) - m_t)``,
    ``take = exp(li - m_t)``, ``floor = exp(-m_t)``.  The running maximum of every head is one float of the request's state
    at ``offset`` (0 when a request starts)."""
    for name, t in (("zi", zi), ("zf", zf)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != heads:
            raise ValueError(f"{name} must be float32 [N, heads] with unit column stride")
    n = zi.shape[0]
    coef = torch.empty((n, 3 * heads), dtype=torch.float32, device=zi.device)
    state, stride, slots = _state_args(view)
    check(library().cw_gate_scan(_ptr(zi), zi.stride(0) if n > 1 else max(zi.stride(0), heads), _ptr(zf),
                                 zf.stride(0) if n > 1 else max(zf.stride(0), heads), _ptr(bias_i), _ptr(bias_f), float(cap), state, stride,
                                 offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start), ctx.num_seqs, heads, n, _ptr(coef), _stream()), "gate_scan")
    return coef


def memory_norm(y: torch.Tensor, floor: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, heads: int, dv: int, eps: float,
                out_dtype: torch.dtype) -> torch.Tensor:
    """[N, heads*dv]: ``y`` [N, heads*(dv+1)] holds per head ``[S^T q | n . q]``; every head's first dv entries are divided
    by ``max(|n . q|, floor) + 1e-6``, then by their root mean square, times ``weight`` [heads*dv], times ``sigmoid(z)``.
    ``floor`` [N, heads] and ``z`` [N, heads*dv]: float32, any row stride."""
    _need(y, torch.float32, "y", 2)
    _need(weight, torch.float32, "weight", 1)
    for name, t in (("floor", floor), ("z", z)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be float32 [N, *] with unit column stride")
    n = y.shape[0]
    if y.shape[1] != heads * (dv + 1) or weight.shape[0] != heads * dv:
        raise ValueError("y must be [N, heads*(dv+1)] and weight [heads*dv]")
    out = torch.empty((n, heads * dv), dtype=out_dtype, device=y.device)
    check(library().cw_memory_norm(_ptr(y), _ptr(floor), floor.stride(0) if n > 1 else max(floor.stride(0), heads), _ptr(z),
                                   z.stride(0) if n > 1 else max(z.stride(0), heads * dv), _ptr(weight), _ptr(out), n, heads, dv, float(eps),
                                   dtype_code(out_dtype), _stream()), "memory_norm")
    return out


def sigmoid_power_decay_(pre: torch.Tensor, tau: float) -> torch.Tensor:
    """In place: ``sigmoid(pre)^(1/tau)``, the decays of a gated linear-attention layer.  float32 [N, C], any row stride."""
    if pre.dtype != torch.float32 or pre.dim() != 2 or pre.stride(1) != 1:
        raise ValueError("pre must be float32 [N, C] with unit column stride")
    n, c = pre.shape
    check(library().cw_sigmoid_power_decay(_ptr(pre), pre.stride(0) if n > 1 else max(pre.stride(0), c), n, c, 1.0 / float(tau),
                                           _stream()), "sigmoid_power_decay")
    return pre


def bounded_forget_(proj: torch.Tensor, channels: int, bias: torch.Tensor | None, lower: torch.Tensor) -> torch.Tensor:
    """In place on float32 ``proj`` [N, >= 2*channels] = ``[q | z | ..]``: ``q <- silu(q)`` and ``z <- f = lower + (1 - lower)
    sigmoid(z + bias)``, forget gates that never fall below ``lower`` [channels]; returns ``1 - f`` as float32 [N, channels]
    (what a channel of the state takes of the new value)."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < 2 * channels:
        raise ValueError("proj must be float32 [N, >= 2*channels] with unit column stride")
    _need(lower, torch.float32, "lower", 1)
    if lower.shape[0] != channels or (bias is not None and bias.shape[0] != channels):
        raise ValueError(f"lower and bias must have {channels} entries")
    n = proj.shape[0]
    take = torch.empty((n, channels), dtype=torch.float32, device=proj.device)
    check(library().cw_bounded_forget(_ptr(proj), proj.stride(0) if n > 1 else max(proj.stride(0), proj.shape[1]), _ptr(bias), _ptr(lower),
                                      _ptr(take), n, channels, _stream()), "bounded_forget")
    return take


def activation_cols_(x: torch.Tensor, cols: int, kind: int) -> torch.Tensor:
    """In place on the first ``cols`` columns of every row of ``x`` [N, C] (unit column stride)."""
    if x.dim() != 2 or x.stride(1) != 1 or not 0 <= cols <= x.shape[1]:
        raise ValueError("x must be [N, C] with unit column stride and cols within C")
    n = x.shape[0]
    check(library().cw_activation_cols(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), x.shape[1]), n, cols, kind,
                                       dtype_code(x.dtype), _stream()), "activation_cols")
    return x


def gated_group_norm(y: torch.Tensor, z: torch.Tensor | None, weight: torch.Tensor, parts: int, eps: float, gate_first: bool,
                     out_dtype: torch.dtype, gate: int = GATE_SILU, shared_weight: bool = False) -> torch.Tensor:
    """``gate_first``: norm_parts(y * gate(z)) * weight; else norm_parts(y) * weight * gate(z).  y, z float32.
    ``gate``: silu or sigmoid, or ``GATE_NONE`` (``z`` None: norm_parts(y) * weight).  ``shared_weight``: ``weight`` has one
    part's width and every part uses it."""
    _need(y, torch.float32, "y", 2)
    if (z is None) != (gate == GATE_NONE):
        raise ValueError("GATE_NONE goes with z = None")
    if z is not None and (z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1):
        raise ValueError("z must be float32 [N, C] with unit column stride")
    _need(weight, torch.float32, "weight", 1)
    n, c = y.shape
    if weight.shape[0] != (c // parts if shared_weight else c):
        raise ValueError(f"weight of {weight.shape[0]} for {parts} parts of {c} columns")
    out = torch.empty((n, c), dtype=out_dtype, device=y.device)
    mode = (1 if gate_first else 0) | (2 if gate == GATE_SIGMOID else 0) | (4 if shared_weight else 0) | (8 if z is None else 0)
    ldz = 0 if z is None else (z.stride(0) if n > 1 else max(z.stride(0), c))
    check(library().cw_gated_group_norm(_ptr(y), _ptr(z), ldz, _ptr(weight), _ptr(out), n, c,
                                        parts, float(eps), mode, dtype_code(out_dtype), _stream()),
          "gated_group_norm")
    return out


def activation_(x: torch.Tensor, kind: int) -> torch.Tensor:
    """In place: gelu in its tanh form, or tanh."""
    _need(x, None, "x")
    check(library().cw_activation(_ptr(x), x.numel(), kind, dtype_code(x.dtype), _stream()), "activation")
    return x
