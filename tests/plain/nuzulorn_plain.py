"""A plain, slow forward pass of the Nuzulorn design: whole sequences, no cache, one function per
mechanism, float32 or float64 torch on the CPU.  It is the yardstick of the tests and shares no
code with ``clockwork_b200``.

The design in this file's notation (x: residual row, W: a stored [out, in] matrix, t: position in the
sequence from 0, n(y) = y / sqrt(mean(y^2) + eps), sg = logistic sigmoid, m = residual_mult):

* input:    x_t = E[token_t] + B[(token_(t-1) a + token_t b) mod buckets];  the first token reads row `buckets` of B
* layer i:  y = x + m mixer(n(x) g1);  y <- y + m ff(n(y) g2)  (a layer may have no ff);  X_(i+1) = y;
            what the next layer (or the output) reads is sum_(j <= i+1) c_i[j] X_j, with X_0 the input rows
* `attention`:   H query heads on G key/value heads, q/k/v with biases; the first `dims` entries of every query and key
            head are rotated (entry r with entry r + dims/2 by the angle t base^(-2r/dims)); position t sees the
            positions j with 0 <= t - j < size and, for every block b of P positions that ends at or before t - size,
            one key and one value that are the block's means; weights = exp(s) / (1 + sum exp(s)) over all of these;
            head h's output times sg(W_g x)_h; then W_o with a bias
* `attention_2`: the same heads without rotation: q_t times 1 + coef ln(floor((t + 1) / every) + 1);
            s = cap tanh(scale q.k / cap) - 2^(-8 (h + 1) / H) (t - j) over all j <= t;
            weights = exp(s) / (exp(sink_h) + sum exp(s)); then W_o without a bias
* `hgrn2`:  q = silu(W_q x), f = l + (1 - l) sg(W_f x + b_f) per head and channel, v = W_v x;
            S <- diag(f) S + (1 - f) v^T;  o = S^T q;  out = W_o concat_heads(n(o_head) g)  (g of size dv, shared)
* ff:       s = sg(W_r x); c = s + correction; experts lie in `count` equal groups of neighbours, a group counts as the
            sum of its two largest c, only the `keep` best groups may be chosen from; the `top` allowed experts with the
            largest c are used with weight s * router_scale;  expert(x) = W_down (silu(W_gate x) (W_up x))
* output:   logits = E (n(x) g_final)
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F


def exact(x):
    return x


def to_bfloat16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ---- input rows ----------------------------------------------------------------------------------
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """The row of the pair table that every token reads: a hash of (previous token, token); the first token the last row."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return torch.tensor(rows, dtype=torch.long)


def input_rows(tokens, embed, pair_table, pair):
    return embed[torch.tensor(tokens, dtype=torch.long)] + pair_table[pair_rows(tokens, pair["buckets"], pair["mul_prev"], pair["mul_cur"])]


# ---- rotation ------------------------------------------------------------------------------------
def rotate_leading(x, positions, dims, base):
    """x [T, heads, d]: entries r and r + dims/2 (r < dims/2) of every head turn by positions * base^(-2r/dims)."""
    half = dims // 2
    r = torch.arange(half, dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * base ** (-2.0 * r / dims)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    lo, hi, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin, rest], dim=-1)


# ---- the two attentions --------------------------------------------------------------------------
def visible_blocks(t, size, pool):
    """How many blocks of `pool` positions lie wholly before the window of position t."""
    return max(0, (t - size + 1) // pool) if t - size + 1 >= 0 else 0


def window_pool_attention(h, w, m, first_position=0, store=exact):
    """h [T, width] -> [T, width].  ``w``: q, q.b, k, k.b, v, v.b, g, o, o.b.  ``store``: what the cache does to a key or
    value (rounding in a bfloat16 run)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, pool = m["mask"]["size"], m["mask"]["pool"]
    pos = torch.arange(first_position, first_position + T)
    q = (h @ w["q"].T + w["q.b"]).view(T, H, dk)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, dk)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q = rotate_leading(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = store(rotate_leading(k, pos, m["rot"]["dims"], m["rot"]["base"]))
    v = store(v)
    gate = torch.sigmoid(h @ w["g"].T)  # [T, H]
    blocks = T // pool
    kb = store(k[: blocks * pool].view(blocks, pool, G, dk).mean(1)) if blocks else k[:0]
    vb = store(v[: blocks * pool].view(blocks, pool, G, dv).mean(1)) if blocks else v[:0]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        lo = max(0, t - size + 1)
        nb = visible_blocks(t, size, pool)
        for hd in range(H):
            g = hd // (H // G)
            keys = torch.cat([kb[:nb, g], k[lo : t + 1, g]])
            vals = torch.cat([vb[:nb, g], v[lo : t + 1, g]])
            s = (keys @ q[t, hd]) * m["scale"]
            mx = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - mx)
            p = e / (torch.exp(-mx) + e.sum())
            out[t, hd] = (p[:, None] * vals).sum(0) * gate[t, hd]
    return out.reshape(T, H * dv) @ w["o"].T + w["o.b"]


def query_temperature(t, coef, every):
    return 1.0 + coef * math.log((t + 1) // every + 1)


def distance_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def capped_sink_attention(h, w, m, store=exact):
    """h [T, width] -> [T, width].  ``w``: q, q.b, k, k.b, v, v.b, sink, o."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    cap = m["softcap"]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, dk)
    k = store((h @ w["k"].T + w["k.b"]).view(T, G, dk))
    v = store((h @ w["v"].T + w["v.b"]).view(T, G, dv))
    slopes = distance_slopes(H)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        temp = query_temperature(t, m["q_temp"]["coef"], m["q_temp"]["every"])
        dist = torch.arange(t, -1, -1, dtype=h.dtype)  # t - j for j = 0 .. t
        for hd in range(H):
            g = hd // (H // G)
            s = (k[: t + 1, g] @ (q[t, hd] * temp)) * m["scale"]
            s = cap * torch.tanh(s / cap) - slopes[hd] * dist
            sink = w["sink"][hd]
            mx = torch.maximum(s.max(), sink)
            e = torch.exp(s - mx)
            p = e / (torch.exp(sink - mx) + e.sum())
            out[t, hd] = (p[:, None] * v[: t + 1, g]).sum(0)
    return out.reshape(T, H * dv) @ w["o"].T


# ---- the recurrent mixer -------------------------------------------------------------------------
def bounded_forget_recurrence(h, w, m, eps, state=None):
    """h [T, width] -> ([T, width], the state after the last token [heads, dk, dv]).  ``w``: q, f, f.b, lower, v, norm, o."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = F.silu(h @ w["q"].T).view(T, H, dk)
    lower = w["lower"].view(H, dk)
    f = lower + (1.0 - lower) * torch.sigmoid(h @ w["f"].T + w["f.b"]).view(T, H, dk)
    v = (h @ w["v"].T).view(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    out = unit_rms(out, eps) * w["norm"]
    return out.reshape(T, H * dv) @ w["o"].T, S


# ---- experts ---------------------------------------------------------------------------------------
def route(logits, correction, top, count, keep):
    """logits [T, E] -> (chosen experts [T, top], their sigmoid scores [T, top], margins [T]: how far, in the scores that
    rank them, the last kept group is from the first dropped one and the last chosen expert from the first one left out)."""
    T, E = logits.shape
    s = torch.sigmoid(logits)
    c = s + correction
    margin = torch.full((T,), math.inf, dtype=logits.dtype)
    if count > 1:
        per = E // count
        grouped = c.view(T, count, per)
        rank = grouped.topk(min(2, per), dim=-1).values.sum(-1)  # [T, count]
        ordered = rank.sort(dim=-1, descending=True)
        kept = ordered.indices[:, :keep]
        if keep < count:
            margin = torch.minimum(margin, ordered.values[:, keep - 1] - ordered.values[:, keep])
        allowed = torch.zeros(T, count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        c = torch.where(allowed[:, :, None].expand(T, count, per).reshape(T, E), c, torch.full_like(c, -math.inf))
    ordered = c.sort(dim=-1, descending=True)
    chosen = ordered.indices[:, :top]
    if top < E:
        margin = torch.minimum(margin, ordered.values[:, top - 1] - ordered.values[:, top])  # (inf when no allowed expert is left out)
    return chosen, s.gather(1, chosen), margin


def experts(h, w, f, log=None, routes=None):
    """h [T, width] -> [T, width].  ``w``: router, correction, e<j>.gate|up|down.  ``log``: a list that receives (chosen,
    margins); ``routes``: choices to use instead of this run's own (those of a run that does not round), the scores this run's."""
    r = f["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    logits = h @ w["router"].T
    chosen, score, margin = route(logits, w["correction"], r["top"], groups["count"], groups["keep"])
    if log is not None:
        log.append((chosen, margin))
    if routes is not None:
        chosen = routes
        score = torch.sigmoid(logits).gather(1, chosen)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), score[t]):
            a = F.silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += s * r["scale"] * (w[f"e{e}.down"] @ a)
    return out


# ---- the model -------------------------------------------------------------------------------------
def sub(weights, prefix):
    return {k[len(prefix) + 1 :]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def mixer(kind, h, w, m, eps, store=exact):
    if kind == "attention":
        return window_pool_attention(h, w, m, store=store)
    if kind == "attention_2":
        return capped_sink_attention(h, w, m, store=store)
    if kind == "hgrn2":
        return bounded_forget_recurrence(h, w, m, eps)[0]
    raise ValueError(f"unknown layer type {kind!r}")


def forward(config, weights, tokens, dtype=torch.float64, act=exact, store=exact, return_layers=False, log=None, routes=None):
    """Logits [T, vocab] of one sequence (and, if asked, the residual rows behind every layer after and before the average
    over the depth).  ``act``: applied to what a bfloat16 run keeps in bfloat16 between kernels (normed rows); ``store``: to
    what the cache keeps.  ``log``: receives every feed-forward's (chosen experts, margins), in layer order; ``routes``: such
    a log of another run, whose choices this run uses."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = input_rows(tokens, w["embed"], w["bigram"], config["embedding"]["bigram"])
    history, layer_out, averaged = [x], [], []
    routes = list(routes) if routes is not None else None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        y = x + mult * mixer(layer["type"], act(unit_rms(x, eps) * w[f"{p}.norm1"]), sub(w, f"{p}.mix"), layer["mixer"], eps, store)
        if layer.get("mlp") is not None:
            y = y + mult * experts(act(unit_rms(y, eps) * w[f"{p}.norm2"]), sub(w, f"{p}.mlp"), layer["mlp"], log,
                                   routes.pop(0)[0] if routes is not None else None)
        layer_out.append(y)
        history.append(y)
        x = sum(c * X for c, X in zip(w[f"{p}.dwa"], history))
        averaged.append(x)
    logits = act(unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, torch.stack(averaged), torch.stack(layer_out)) if return_layers else logits


def greedy(config, weights, prompt, new_tokens, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(config, weights, tokens, dtype)[-1].argmax()))
    return tokens[len(prompt):]


def read_model_dir(folder, dtype=torch.float32):
    """(config, {name: tensor}) of a folder with config.json and model.safetensors, read with nothing but the file format:
    an 8-byte little-endian header length, a JSON header, raw little-endian data."""
    import struct

    import numpy as np

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    blob = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + n])
    data = blob[8 + n :]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        if meta["dtype"] == "BF16":
            t = torch.from_numpy(raw.copy()).view(torch.bfloat16)
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(raw.copy()).view(torch.float32)
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(raw.copy()).view(torch.int32)
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        t = t.reshape(meta["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return config, out
