"""A plain, slow forward pass of the Kapolorn design: whole sequences, no cache, one function per
mechanism, float32 or float64 torch on the CPU.  It is the yardstick of the tests and shares no
code with ``clockwork_b200``.

The design in this file's notation (x: residual row, W: a stored [out, in] matrix, t: position in the
sequence from 0, n(y) = y / sqrt(mean(y^2) + eps), sg = logistic sigmoid):

* input:    x_t = E[token] s_e
* order:    layers 0 .. a-1 once, layers a .. b-1 `times` times over (same weights, every pass a cache or
            state of its own), layers b .. once
* layer:    x <- x + n(mixer(n(x) g1)) g1b;  x <- x + n(ff(n(x) g2)) g2b   (a layer may have no ff)
* `channel_delta` mixer (gated delta rule, a decay per key channel):
            q, k, v = silu(conv(W h)) with a causal per-channel convolution over the last `taps` inputs;
            q, k per head divided by sqrt(|.|^2 + 1e-6), q also by sqrt(dk);  beta = sg(W_b h) per head;
            a = exp(-exp(A_head) softplus(W_a2 W_a1 h + dt)) per head and key channel;
            S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
            out = W_o concat_heads(n(o_head) g sg(W_g2 W_g1 h)_head)       (g of size dv, shared by the heads)
* `parallel` mixer: c_l left(h) + c_r right(h)
  - left:   attention of H query heads on G key/value heads; the first `dims` entries of every query and key head
            are rotated (entry i with entry i + dims/2 by the angle t b^(-2i/dims)); position t sees j <= t of its
            own block of `size` positions (t // size == j // size); weights = softmax over the visible keys and one
            more logit per head (`sink`) that has no value
  - right:  a matrix memory with stabilised exponential gates: q = W_q h / sqrt(dk);
            li = cap tanh((W_i h + b_i)/cap);  lf = log sg(cap tanh((W_f h + b_f)/cap));
            m_t = max(lf + m_(t-1), li) with m before the first token 0;
            S <- exp(lf + m_(t-1) - m_t) S + exp(li - m_t) k v^T, and the same for n with k alone;
            o = S^T q / (max(|n . q|, exp(-m_t)) + 1e-6);
            out = W_o (concat_heads(n(o_head)) g sg(W_g h))                 (g over all heads)
* ff:       a mixture of experts: p = softmax(W_r h) over all experts; experts lie in `count` equal groups of
            neighbours, a group counts as its best expert, only the `keep` best groups may be chosen from; the `top`
            allowed experts with the largest p are used with weight p (not renormalised); a shared expert always runs.
            expert(h) = W_down (a sg(1.702 a) (b + 1)),  a = min(W_gate h, lim),  b = clamp(W_up h, -lim, lim)
* output:   z = E (n(x) g_final);  logits = c tanh(z / c)
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def exact(x):
    return x


def to_bfloat16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scaled_norm(x, g, eps):
    return unit_rms(x, eps) * g


def run_order(config):
    """The indices of the layers in the order they run, and for every run which pass of its layer it is."""
    count = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, 0) for i in range(a)]
    for p in range(times):
        order += [(i, p) for i in range(a, b)]
    order += [(i, 0) for i in range(b, count)]
    return order


# ---- attention in blocks of positions, with rotation and a sink ---------------------------------------
def rotate_leading(x, positions, dims, base):
    """x [T, heads, d]: entries i and i + dims/2 (i < dims/2) of every head turn by positions * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    lo, hi, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin, rest], dim=-1)


def block_mask(count, size, first=0):
    t = torch.arange(first, first + count)
    return (t[None, :] <= t[:, None]) & ((t[:, None] // size) == (t[None, :] // size))


def blocked_sink_attention(h, w, p, m, rnd=exact, first=0):
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    positions = torch.arange(first, first + t)
    q = (h @ w[f"{p}.q"].T).reshape(t, heads, dk)
    k = (h @ w[f"{p}.k"].T).reshape(t, groups, dk)
    v = rnd(h @ w[f"{p}.v"].T).reshape(t, groups, dv)
    q = rnd(rotate_leading(rnd(q), positions, m["rot"]["dims"], m["rot"]["base"]))
    k = rnd(rotate_leading(rnd(k), positions, m["rot"]["dims"], m["rot"]["base"]))
    per = heads // groups
    scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(per, dim=1)) * m["scale"]
    scores = scores.masked_fill(~block_mask(t, m["mask"]["size"], first), float("-inf"))
    sink = w[f"{p}.sink"].to(h.dtype)[:, None, None].expand(heads, t, 1)
    weights = torch.softmax(torch.cat([scores, sink], dim=-1), dim=-1)[..., :-1]
    o = torch.einsum("hts,shd->thd", weights, v.repeat_interleave(per, dim=1)).reshape(t, heads * dv)
    return rnd(o) @ w[f"{p}.o"].T


# ---- the matrix memory with stabilised exponential gates ------------------------------------------------
def capped(z, cap):
    return cap * torch.tanh(z / cap)


def matrix_memory_scan(q, k, v, log_in, log_forget):
    """q, k [T, H, dk], v [T, H, dv], log gates [T, H] -> [T, H, dv]."""
    t, heads, dk = q.shape
    state = torch.zeros(heads, dk, v.shape[-1], dtype=q.dtype)
    norm = torch.zeros(heads, dk, dtype=q.dtype)
    m = torch.zeros(heads, dtype=q.dtype)
    out = []
    for i in range(t):
        m_new = torch.maximum(log_forget[i] + m, log_in[i])
        keep, take = torch.exp(log_forget[i] + m - m_new), torch.exp(log_in[i] - m_new)
        state = keep[:, None, None] * state + take[:, None, None] * k[i][:, :, None] * v[i][:, None, :]
        norm = keep[:, None] * norm + take[:, None] * k[i]
        m = m_new
        top = torch.einsum("hkv,hk->hv", state, q[i])
        bottom = torch.maximum((norm * q[i]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out.append(top / bottom[:, None])
    return torch.stack(out)


def matrix_memory_mixer(h, w, p, m, eps, rnd=exact):
    heads, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    t = h.shape[0]
    q = (h @ w[f"{p}.q"].T).reshape(t, heads, dk) * dk ** -0.5
    k = (h @ w[f"{p}.k"].T).reshape(t, heads, dk)
    v = (h @ w[f"{p}.v"].T).reshape(t, heads, dv)
    log_in = capped(h @ w[f"{p}.i"].T + w[f"{p}.i.b"], cap)
    log_forget = F.logsigmoid(capped(h @ w[f"{p}.f"].T + w[f"{p}.f.b"], cap))
    o = unit_rms(matrix_memory_scan(q, k, v, log_in, log_forget), eps).reshape(t, heads * dv)
    return rnd(o * w[f"{p}.norm"] * torch.sigmoid(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def side_by_side(h, w, p, m, eps, rnd=exact):
    left = blocked_sink_attention(h, w, f"{p}.left", m["left"], rnd)
    right = matrix_memory_mixer(h, w, f"{p}.right", m["right"], eps, rnd)
    return m["left_scale"] * left + m["right_scale"] * right


# ---- the gated delta rule with a decay per key channel ----------------------------------------------------
def short_convolution(x, taps_weight):
    """x [T, C], taps_weight [C, taps] (the last column is the current token's): zeros before the first row."""
    taps = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j : j + x.shape[0]] * taps_weight[:, j]
    return out


def unit_length(x):
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_rule_scan(q, k, v, decay, beta):
    """q, k, decay [T, H, dk], v [T, H, dv], beta [T, H] -> [T, H, dv]; the read-out sees the token's own write."""
    t, heads, dk = q.shape
    state = torch.zeros(heads, dk, v.shape[-1], dtype=q.dtype)
    out = []
    for i in range(t):
        state = decay[i][:, :, None] * state
        u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", state, k[i]))
        state = state + k[i][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", state, q[i]))
    return torch.stack(out)


def channel_delta_mixer(h, w, p, m, eps, rnd=exact):
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = F.silu(short_convolution(h @ w[f"{p}.q"].T, w[f"{p}.q.conv"])).reshape(t, groups, dk)
    k = F.silu(short_convolution(h @ w[f"{p}.k"].T, w[f"{p}.k.conv"])).reshape(t, groups, dk)
    v = F.silu(short_convolution(h @ w[f"{p}.v"].T, w[f"{p}.v.conv"])).reshape(t, heads, dv)
    per = heads // groups
    q = (unit_length(q) * dk ** -0.5).repeat_interleave(per, dim=1)
    k = unit_length(k).repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ w[f"{p}.b"].T)
    step = F.softplus(rnd(h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.dt_bias"]).reshape(t, heads, dk)
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"])[None, :, None] * step)
    o = delta_rule_scan(q, k, v, decay, beta)
    gate = torch.sigmoid(rnd(h @ w[f"{p}.g1"].T) @ w[f"{p}.g2"].T).reshape(t, heads, dv)
    o = (scaled_norm(o, w[f"{p}.norm"], eps) * gate).reshape(t, heads * dv)
    return rnd(o) @ w[f"{p}.o"].T


# ---- the mixture of experts ------------------------------------------------------------------------------
def clamped_expert(h, w, p, limit, rnd=exact):
    a = torch.clamp(h @ w[f"{p}.gate"].T, max=limit)
    b = torch.clamp(h @ w[f"{p}.up"].T, min=-limit, max=limit)
    return rnd(a * torch.sigmoid(1.702 * a) * (b + 1.0)) @ w[f"{p}.down"].T


def route(h, w, p, r):
    """(chosen experts [T, top], their weights [T, top], how far every token's choice is from another one [T]: the
    smallest gap, in router logits, between something taken and the best thing left out, among groups and among the
    allowed experts; infinite where nothing is left out)."""
    experts, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    scores = torch.softmax(h @ w[f"{p}.router"].T, dim=-1)
    best = scores.reshape(-1, count, experts // count).max(-1).values
    kept = torch.zeros_like(best, dtype=torch.bool).scatter(-1, best.topk(keep, dim=-1).indices, True)
    allowed = kept.repeat_interleave(experts // count, dim=-1)
    ranked = scores.masked_fill(~allowed, -1.0)
    chosen = ranked.topk(top, dim=-1).indices
    margin = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    if keep < count:
        order = best.sort(dim=-1, descending=True).values
        margin = torch.minimum(margin, torch.log(order[:, keep - 1] / order[:, keep]))
    if top < keep * (experts // count):
        order = ranked.sort(dim=-1, descending=True).values
        margin = torch.minimum(margin, torch.log(order[:, top - 1] / order[:, top]))
    return chosen, scores.gather(-1, chosen), margin


def mixture_of_experts(h, w, p, m, rnd=exact, forced=None, log=None):
    """``forced``: the experts to use (the weights are still this run's scores of them); ``log``: a list that receives
    (chosen, margin) of this call."""
    chosen, weights, margin = route(h, w, p, m["router"])
    if log is not None:
        log.append((chosen, margin))
    if forced is not None:
        chosen = forced
        weights = torch.softmax(h @ w[f"{p}.router"].T, dim=-1).gather(-1, chosen)
    if m.get("shared") is not None:
        out = clamped_expert(h, w, f"{p}.shared", m["shared"]["limit"], rnd)
    else:
        out = torch.zeros_like(h)
    for e in range(m["router"]["experts"]):
        share = (weights * (chosen == e)).sum(-1, keepdim=True)
        rows = (chosen == e).any(-1)
        if rows.any():
            out[rows] = out[rows] + share[rows] * clamped_expert(h[rows], w, f"{p}.e{e}", m["expert"]["limit"], rnd)
    return out


# ---- the model -------------------------------------------------------------------------------------------
def mixer_of(layer, h, w, p, eps, rnd=exact):
    if layer["type"] == "parallel":
        return side_by_side(h, w, p, layer["mixer"], eps, rnd)
    if layer["type"] == "channel_delta":
        return channel_delta_mixer(h, w, p, layer["mixer"], eps, rnd)
    raise ValueError(layer["type"])


def forward(config, weights, tokens, dtype=torch.float64, rnd=exact, keep_layers=False, routes=None, log=None):
    """Logits [T, vocab] of one whole sequence (and, with ``keep_layers``, the residual after every layer run).
    ``log``: a list that receives (chosen experts, margin) of every feed-forward run, in run order; ``routes``: such a
    list of an earlier call, whose choices this call then uses instead of its own (the yardstick of a rounded run that
    must not count a choice that rounding flipped)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    kept, ff_run = [], 0
    for i, _ in run_order(config):
        layer = config["layers"][i]
        h = rnd(scaled_norm(x, w[f"l{i}.norm1"], eps))
        x = x + scaled_norm(mixer_of(layer, h, w, f"l{i}.mix", eps, rnd), w[f"l{i}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rnd(scaled_norm(x, w[f"l{i}.norm2"], eps))
            forced = routes[ff_run][0] if routes is not None else None
            x = x + scaled_norm(mixture_of_experts(h, w, f"l{i}.mlp", layer["mlp"], rnd, forced, log), w[f"l{i}.norm2b"], eps)
            ff_run += 1
        kept.append(x)
    z = rnd(scaled_norm(x, w["final.norm"], eps)) @ w["embed"].T
    cap = config.get("logit_softcap")
    logits = z if cap is None else cap * torch.tanh(z / cap)
    return (logits, torch.stack(kept)) if keep_layers else logits


def first_position_margin(config, weights, token, dtype=torch.float64):
    """At position 0 a head of the matrix memory and of the delta rule puts out (k . q) times a positive number times v,
    and its norm makes sign(k . q) n(v) of that: the smallest |cos(q, k)| over those heads, in every layer run, says how
    far the first token is from a sign that rounding could flip."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor([token], dtype=torch.long)] * config["embedding"]["scale"]
    margin = 1.0

    def cosine(q, k):
        return float(((q * k).sum(-1) / (q.norm(dim=-1) * k.norm(dim=-1))).abs().min())

    for i, _ in run_order(config):
        layer, p = config["layers"][i], f"l{i}.mix"
        h = scaled_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "parallel":
            m = layer["mixer"]["right"]
            q, k = ((h @ w[f"{p}.right.{s}"].T).reshape(m["heads"], m["dim"]) for s in "qk")
        else:
            m = layer["mixer"]  # one row: the convolution leaves the current token's tap
            q, k = (F.silu((h @ w[f"{p}.{s}"].T) * w[f"{p}.{s}.conv"][:, -1]).reshape(m["kv_heads"], m["dim"]) for s in "qk")
        margin = min(margin, cosine(q, k))
        x = x + scaled_norm(mixer_of(layer, h, w, p, eps), w[f"l{i}.norm1b"], eps)
        if layer.get("mlp") is not None:
            h = scaled_norm(x, w[f"l{i}.norm2"], eps)
            x = x + scaled_norm(mixture_of_experts(h, w, f"l{i}.mlp", layer["mlp"]), w[f"l{i}.norm2b"], eps)
    return margin


def steady_first_token(config, weights, candidates=range(40)):
    """The candidate whose answer at position 0 is farthest from such a flip."""
    return max(candidates, key=lambda token: first_position_margin(config, weights, token))


def greedy_generate(config, weights, prompt, count, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, weights, tokens, dtype=dtype)[-1].argmax()))
    return tokens[len(prompt):]
