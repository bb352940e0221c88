"""Small Kapolorn configurations of the tests and random weights for them, drawn here (tensor names and shapes are
written out from the configuration by this file's own rules, not asked of the package).

The four differ in every size, in the order of layers, in what is looped and in the values that a model may happen to
make equal or 1: one key/value head for all query heads and as many as query heads; values narrower and wider than keys;
all of a head rotated and only its first entries; blocks of 1 position (a token sees itself and the sink), shorter than a
page, no multiple of a page, and longer than the prompts; a delta-rule layer with one q/k head for all heads, and with
one tap (no convolution state); a single memory head; a layer without feed-forward; one group of experts (or none
named), as many groups as experts, every expert chosen, a single chosen expert; no shared expert; no loop, a loop of one
layer three times, a loop over the whole model; scales of 1; widths that are no power of two; inner sizes of the
low-rank products that are no multiple of 8."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _pair(heads, kv_heads, dim, vdim, block, scale, rot, base, r_heads, r_dim, r_vdim, cap, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": block},
                 "rot": {"dims": rot, "base": base}},
        "left_scale": left_scale,
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": cap},
        "right_scale": right_scale}}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _moe(ff, limit, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def _model(vocab, width, eps, scale, cap, loop, layers):
    out = {"architecture": "Kapolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "logit_softcap": cap, "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIG_A = _model(96, 64, 1e-5, 2.0, 12.0, (1, 2, 3), [
    (_pair(4, 2, 24, 12, 21, 0.3, 8, 1000.0, 3, 20, 12, 8.0, 0.7, 1.3), _moe(40, 1.5, 6, 3, (3, 2), (56, 2.5))),
    (_delta(4, 2, 12, 20, 3), _moe(24, 1.0, 4, 1, (2, 1), (16, 1.0))),
    (_pair(3, 1, 16, 40, 7, 0.25, 16, 50000.0, 1, 24, 8, 15.0, 1.0, 1.0), None),
])
CONFIG_B = _model(80, 48, 1e-6, 1.0, 30.0, None, [
    (_delta(3, 3, 8, 8, 1), _moe(32, 2.0, 3, 3, None, None)),
    (_pair(2, 2, 12, 20, 200, 0.3, 12, 100.0, 4, 8, 16, 5.0, 1.5, 0.5), _moe(20, 0.5, 5, 2, (1, 1), (24, 3.0))),
    (_pair(6, 2, 8, 8, 1, 0.4, 2, 10000.0, 2, 16, 24, 20.0, 0.9, 1.1), _moe(16, 1.0, 4, 2, (4, 2), None)),
])
CONFIG_C = _model(120, 72, 1e-5, 0.5, 8.0, (0, 3, 2), [
    (_pair(6, 1, 8, 24, 16, 0.35, 4, 300.0, 2, 40, 16, 12.0, 1.1, 0.8), _moe(28, 1.2, 8, 3, (4, 2), (36, 1.8))),
    (_delta(2, 1, 40, 8, 4), None),
    (_delta(5, 5, 8, 24, 2), _moe(48, 3.0, 2, 1, (2, 2), (8, 0.7))),
])
CONFIG_D = _model(1000, 320, 1e-6, 1.5, 25.0, (1, 3, 2), [  # sizes that the tensor-core kernels take
    (_pair(8, 2, 32, 64, 100, 32 ** -0.5, 32, 10000.0, 3, 24, 40, 15.0, 1.2, 0.9), _moe(128, 2.0, 8, 2, (4, 2), (192, 2.5))),
    (_pair(12, 3, 48, 80, 60, 48 ** -0.5, 16, 500000.0, 2, 32, 64, 10.0, 0.8, 1.1), _moe(96, 1.0, 16, 4, (2, 1), (64, 1.5))),
    (_delta(4, 2, 64, 48, 4), _moe(64, 1.5, 6, 2, (3, 1), (256, 1.0))),
    (_pair(4, 4, 80, 200, 30, 80 ** -0.5, 80, 1000.0, 4, 64, 32, 20.0, 1.0, 1.0), None),
])
CONFIGS = {"A": (CONFIG_A, 4, 5), "B": (CONFIG_B, 8, 8), "C": (CONFIG_C, 16, 3), "D": (CONFIG_D, 16, 24)}  # name -> (config, page size, low rank)


def tensor_shapes(config: dict, rank: int) -> dict[str, tuple]:
    w = config["width"]
    out = {"embed": (config["vocab"], w), "final.norm": (w,)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        out.update({f"l{i}.norm1": (w,), f"l{i}.norm1b": (w,)})
        if layer["type"] == "parallel":
            left, right = m["left"], m["right"]
            h, g, dk, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            out.update({f"{p}.left.q": (h * dk, w), f"{p}.left.k": (g * dk, w), f"{p}.left.v": (g * dv, w), f"{p}.left.o": (w, h * dv),
                        f"{p}.left.sink": (h,)})
            rh, rk, rv = right["heads"], right["dim"], right["vdim"]
            out.update({f"{p}.right.q": (rh * rk, w), f"{p}.right.k": (rh * rk, w), f"{p}.right.v": (rh * rv, w),
                        f"{p}.right.g": (rh * rv, w), f"{p}.right.o": (w, rh * rv), f"{p}.right.norm": (rh * rv,),
                        f"{p}.right.i": (rh, w), f"{p}.right.i.b": (rh,), f"{p}.right.f": (rh, w), f"{p}.right.f.b": (rh,)})
        else:
            h, g, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({f"{p}.q": (g * dk, w), f"{p}.k": (g * dk, w), f"{p}.v": (h * dv, w), f"{p}.q.conv": (g * dk, taps),
                        f"{p}.k.conv": (g * dk, taps), f"{p}.v.conv": (h * dv, taps), f"{p}.b": (h, w), f"{p}.A_log": (h,),
                        f"{p}.dt_bias": (h * dk,), f"{p}.a1": (rank, w), f"{p}.a2": (h * dk, rank), f"{p}.g1": (rank + 1, w),
                        f"{p}.g2": (h * dv, rank + 1), f"{p}.norm": (dv,), f"{p}.o": (w, h * dv)})
        mlp = layer["mlp"]
        if mlp is not None:
            ff = mlp["expert"]["ff"]
            out.update({f"l{i}.norm2": (w,), f"l{i}.norm2b": (w,), f"l{i}.mlp.router": (mlp["router"]["experts"], w)})
            for e in range(mlp["router"]["experts"]):
                out.update({f"l{i}.mlp.e{e}.gate": (ff, w), f"l{i}.mlp.e{e}.up": (ff, w), f"l{i}.mlp.e{e}.down": (w, ff)})
            if mlp.get("shared") is not None:
                sf = mlp["shared"]["ff"]
                out.update({f"l{i}.mlp.shared.gate": (sf, w), f"l{i}.mlp.shared.up": (sf, w), f"l{i}.mlp.shared.down": (w, sf)})
    return out


def draw_weights(config: dict, rank: int, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, 1/in) so that activations keep their size; attention peaked (query and key
    sides scaled up) so that a key that is missed or seen wrongly moves the logits; sinks near the scores' size so
    that a sink left out shows; decays close to one and forget gates open, so that a state remembers dozens of tokens
    and a lost or stale state shows; routers wide enough that choices are rarely close calls."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, rank).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        n = lambda scale=1.0: torch.randn(shape, generator=gen) * scale  # noqa: E731
        if leaf == "embed":
            t = n(0.7)
        elif leaf in ("norm1", "norm2", "final.norm", "mix.right.norm", "mix.norm"):
            t = 1.0 + n(0.2)
        elif leaf in ("norm1b", "norm2b"):
            t = 0.5 + n(0.1)
        elif leaf in ("mix.left.q", "mix.left.k"):
            t = n(2.5 / math.sqrt(shape[-1]))
        elif leaf == "mix.left.sink":
            t = 1.0 + n(1.0)
        elif leaf == "mix.right.f.b":
            t = 3.0 + n(1.0)
        elif leaf == "mix.right.i.b":
            t = n(1.0)
        elif leaf == "mix.A_log":
            t = -1.5 + n(0.5)
        elif leaf == "mix.dt_bias":
            t = -2.0 + n(1.0)
        elif leaf.endswith(".conv"):
            t = n(0.5) + (torch.arange(shape[1]) == shape[1] - 1).float()
        elif leaf == "mlp.router":
            t = n(3.0 / math.sqrt(shape[-1]))
        else:
            t = n(1.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


ROUTING_CLASSES = 8


def steady_routing(config: dict, weights: dict[str, torch.Tensor], seed: int = 0, step: float = 0.5) -> dict[str, torch.Tensor]:
    """Router choices that rounding cannot flip, for runs in bfloat16 that are compared with a run that rounds
    elsewhere.  The first ``ROUTING_CLASSES`` coordinates of the residual become a one-hot code of token mod classes (4
    after the embedding's scale) that no layer writes to (the output norms' weights are 0 there), and every router
    reads, for each class, a permutation of the levels 0, step, 2 step .. from that class's coordinate, besides a
    thirtieth of its drawn weights on the others.  Router logits are then (4 / rms(x)) times distinct levels plus a
    small part that depends on the context: the order, among groups and among experts, is the class's permutation, and
    the scores still fall off slowly enough that every chosen expert counts."""
    c = ROUTING_CLASSES
    gen = torch.Generator().manual_seed(1000 + seed)
    out = dict(weights)
    embed = weights["embed"].float().clone()
    embed[:, :c] = 0.0
    rows = torch.arange(embed.shape[0])
    embed[rows, rows % c] = 4.0 / config["embedding"]["scale"]
    out["embed"] = embed.to(torch.bfloat16)
    for i, layer in enumerate(config["layers"]):
        for name in (f"l{i}.norm1b", f"l{i}.norm2b"):
            if name in weights:
                t = weights[name].clone()
                t[:c] = 0.0
                out[name] = t
        if layer["mlp"] is not None:
            norm = weights[f"l{i}.norm2"].clone()
            norm[:c] = 1.0
            out[f"l{i}.norm2"] = norm
            router = weights[f"l{i}.mlp.router"].float() / 30.0
            experts = router.shape[0]
            for k in range(c):
                router[:, k] = step * torch.randperm(experts, generator=gen).float()
            out[f"l{i}.mlp.router"] = router.to(torch.bfloat16)
    return out


def write_model(folder, name: str, seed: int = 0, steady: bool = False) -> Path:
    from clockwork_b200.weights import save_safetensors

    config, _, rank = CONFIGS[name]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    weights = draw_weights(config, rank, seed)
    save_safetensors(folder / "model.safetensors", steady_routing(config, weights, seed) if steady else weights)
    return folder


def tokens_for(config: dict, length: int, salt: int = 0) -> list[int]:
    state = (7919 * salt + 32452843 * length + 313) & 0x7FFFFFFF
    out = []
    for _ in range(length):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % config["vocab"])
    return out
