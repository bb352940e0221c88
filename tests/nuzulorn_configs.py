"""Small Nuzulorn configurations of the tests and random weights for them, drawn here (tensor names and shapes are
written out from the configuration by this file's own rules, not asked of the package).

The four differ in every size, in the order of layers and in the values that a model may happen to make equal or 1: one
key/value head for all query heads and as many as query heads; values narrower and wider than keys; all of a head rotated
and only its first entries; windows of 1 position (a token sees itself, the pooled blocks and the sink), shorter than a page
and than a block, no multiple of a page or of a block, and longer than the prompts (no block is ever seen); blocks of 1
position (every token that left the window is seen again at once), blocks that are no divisor of the page size, blocks longer
than the window; a query temperature that changes every 3 positions and one that never changes within a prompt; a cap far
above the scores and one that bends them; one recurrent head; a layer without feed-forward; one group of experts (or none
named), as many groups as experts (a group of one expert counts as that expert), every expert chosen, a single chosen
expert; a residual multiplier of 1; pair tables of 1 bucket and of more buckets than the vocabulary; widths that are no
power of two."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _window(heads, kv_heads, dim, vdim, scale, size, pool, rot, base):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": size, "pool": pool}, "rot": {"dims": rot, "base": base}}}


def _capped(heads, kv_heads, dim, vdim, scale, cap, coef, every):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "softcap": cap, "q_temp": {"coef": coef, "every": every}}}


def _recurrent(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def _moe(ff, experts, top, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _model(vocab, width, eps, mult, pair, layers):
    return {"architecture": "Nuzulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"bigram": {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}},
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


CONFIG_A = _model(96, 64, 1e-5, 0.6, (53, 31, 7), [
    (_window(4, 2, 24, 12, 0.3, 21, 5, 8, 1000.0), _moe(40, 6, 3, 1.5, (3, 2))),
    (_recurrent(3, 12, 20), _moe(24, 4, 1, 2.0, (2, 1))),
    (_capped(4, 2, 16, 24, 0.25, 4.0, 0.4, 3), None),
    (_window(3, 1, 16, 40, 0.25, 7, 9, 16, 50000.0), _moe(16, 4, 2, 0.8, (4, 2))),
])
CONFIG_B = _model(80, 48, 1e-6, 1.0, (1, 3, 5), [
    (_capped(3, 3, 8, 8, 0.5, 50.0, 1.5, 1000), _moe(32, 3, 3, 1.0, None)),
    (_window(2, 2, 12, 20, 0.3, 200, 6, 12, 100.0), _moe(20, 5, 2, 1.2, (1, 1))),
    (_window(6, 2, 8, 8, 0.4, 1, 1, 2, 10000.0), None),
    (_recurrent(1, 16, 8), _moe(16, 4, 2, 2.5, (2, 2))),
])
CONFIG_C = _model(120, 72, 1e-5, 0.3, (211, 5, 11), [
    (_recurrent(5, 8, 24), None),
    (_window(6, 1, 8, 24, 0.35, 16, 4, 4, 300.0), _moe(28, 8, 3, 2.5, (4, 2))),
    (_capped(6, 1, 8, 24, 0.35, 8.0, 0.5, 16), _moe(48, 2, 1, 0.5, (2, 1))),
    (_window(2, 2, 40, 8, 0.15, 5, 11, 40, 200000.0), _moe(12, 6, 6, 1.0, (3, 3))),
])
CONFIG_D = _model(1000, 320, 1e-6, 0.5, (1201, 97, 29), [  # sizes that the tensor-core kernels take
    (_capped(8, 2, 32, 64, 32 ** -0.5, 15.0, 0.7, 32), _moe(128, 8, 2, 1.7, (4, 2))),
    (_window(12, 3, 48, 80, 48 ** -0.5, 60, 7, 16, 500000.0), _moe(96, 16, 4, 1.5, (2, 1))),
    (_recurrent(4, 64, 48), _moe(64, 6, 2, 1.0, (3, 1))),
    (_window(4, 4, 80, 200, 80 ** -0.5, 100, 16, 80, 1000.0), None),
    (_window(8, 8, 64, 64, 0.125, 33, 10, 32, 20000.0), _moe(64, 8, 2, 2.0, (2, 1))),
])
CONFIGS = {"A": (CONFIG_A, 4), "B": (CONFIG_B, 8), "C": (CONFIG_C, 16), "D": (CONFIG_D, 16)}  # name -> (config, page size)


def tensor_shapes(config: dict) -> dict[str, tuple]:
    w = config["width"]
    out = {"embed": (config["vocab"], w), "bigram": (config["embedding"]["bigram"]["buckets"] + 1, w), "final.norm": (w,)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        out.update({f"l{i}.norm1": (w,), f"l{i}.dwa": (i + 2,)})
        if layer["type"] == "hgrn2":
            h, dk, dv = m["heads"], m["dim"], m["vdim"]
            out.update({f"{p}.q": (h * dk, w), f"{p}.f": (h * dk, w), f"{p}.f.b": (h * dk,), f"{p}.lower": (h * dk,),
                        f"{p}.v": (h * dv, w), f"{p}.norm": (dv,), f"{p}.o": (w, h * dv)})
        else:
            h, g, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({f"{p}.q": (h * dk, w), f"{p}.q.b": (h * dk,), f"{p}.k": (g * dk, w), f"{p}.k.b": (g * dk,),
                        f"{p}.v": (g * dv, w), f"{p}.v.b": (g * dv,), f"{p}.o": (w, h * dv)})
            if layer["type"] == "attention":
                out.update({f"{p}.g": (h, w), f"{p}.o.b": (w,)})
            else:
                out[f"{p}.sink"] = (h,)
        mlp = layer["mlp"]
        if mlp is not None:
            ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
            out.update({f"l{i}.norm2": (w,), f"l{i}.mlp.router": (experts, w), f"l{i}.mlp.correction": (experts,)})
            for e in range(experts):
                out.update({f"l{i}.mlp.e{e}.gate": (ff, w), f"l{i}.mlp.e{e}.up": (ff, w), f"l{i}.mlp.e{e}.down": (w, ff)})
    return out


def draw_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, 1/in) so that activations keep their size; attention peaked (query and key sides
    scaled up) so that a key that is missed or seen wrongly moves the logits; sinks near the scores' size so that a sink
    left out shows; forget gates mostly open with lower bounds spread over (0, 1), so that a state remembers dozens of
    tokens and a lost or stale state shows; the weights over the depth near an average with some of them negative."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        n = lambda scale=1.0: torch.randn(shape, generator=gen) * scale  # noqa: E731
        if leaf in ("embed", "bigram"):
            t = n(0.7)
        elif leaf in ("norm1", "norm2", "final.norm", "mix.norm"):
            t = 1.0 + n(0.2)
        elif leaf in ("mix.q", "mix.k"):
            t = n(2.5 / math.sqrt(shape[-1]))
        elif leaf in ("mix.q.b", "mix.k.b", "mix.v.b", "mix.o.b"):
            t = n(0.3)
        elif leaf == "mix.sink":
            t = 1.0 + n(1.0)
        elif leaf == "mix.g":
            t = n(1.5 / math.sqrt(shape[-1]))
        elif leaf == "mix.f.b":
            t = 2.0 + n(1.0)
        elif leaf == "mix.lower":
            t = torch.rand(shape, generator=gen) * 0.9
        elif leaf == "dwa":
            t = (1.0 + n(0.5)) / shape[0]
        elif leaf == "mlp.router":
            t = n(3.0 / math.sqrt(shape[-1]))
        elif leaf == "mlp.correction":
            t = n(0.1)
        else:
            t = n(1.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


ROUTING_CLASSES = 8


def steady_routing(config: dict, weights: dict[str, torch.Tensor], seed: int = 0, spread: float = 3.0) -> dict[str, torch.Tensor]:
    """Router choices that rounding cannot flip, for runs in bfloat16 that are compared with a run that rounds elsewhere.
    The first ``ROUTING_CLASSES`` coordinates of the input rows become a one-hot code of token mod classes that no layer
    writes to (the rows of every output product, output bias and expert's down product are 0 there; the pair table too), and
    every router reads, for each class, evenly spaced levels between -spread/2 and spread/2 from that class's coordinate,
    besides a hundredth of its drawn weights on the others: the groups in an order drawn per class, each group a run of
    neighbouring levels (so that no two groups' sums of their best entries come close), the experts of a group in a drawn
    order too.  The average over the depth only rescales the code.  Whether the
    margins between chosen and not chosen (groups and experts) are wide enough for a given prompt is for the caller to check
    with the plain implementation's log."""
    c = ROUTING_CLASSES
    gen = torch.Generator().manual_seed(1000 + seed)
    out = dict(weights)
    for name in ("embed", "bigram"):
        t = weights[name].float().clone()
        t[:, :c] = 0.0
        if name == "embed":
            rows = torch.arange(t.shape[0])
            t[rows, rows % c] = 2.0
        out[name] = t.to(torch.bfloat16)
    for i, layer in enumerate(config["layers"]):
        names = [f"l{i}.mix.o", f"l{i}.mix.o.b"]
        if layer["mlp"] is not None:
            names += [f"l{i}.mlp.e{e}.down" for e in range(layer["mlp"]["router"]["experts"])]
        for name in names:
            if name in weights:
                t = weights[name].clone()
                t[:c] = 0.0
                out[name] = t
        dwa = weights[f"l{i}.dwa"].float().abs() + 0.05  # (positive: the code keeps its sign)
        out[f"l{i}.dwa"] = dwa.to(torch.bfloat16)
        if layer["mlp"] is not None:
            norm = weights[f"l{i}.norm2"].clone()
            norm[:c] = 1.0
            out[f"l{i}.norm2"] = norm
            router = weights[f"l{i}.mlp.router"].float() / 100.0
            experts = router.shape[0]
            groups = (layer["mlp"]["router"].get("groups") or {"count": 1})["count"]
            per = experts // groups
            for k in range(c):
                order = torch.randperm(groups, generator=gen)
                level = torch.cat([order[g] * per + torch.randperm(per, generator=gen) for g in range(groups)]).float()
                router[:, k] = spread * (level / max(1, experts - 1) - 0.5)
            out[f"l{i}.mlp.router"] = router.to(torch.bfloat16)
            out[f"l{i}.mlp.correction"] = (weights[f"l{i}.mlp.correction"].float() * 0.02).to(torch.bfloat16)
    return out


def write_model(folder, name: str, seed: int = 0, steady: bool = False) -> Path:
    from clockwork_b200.weights import save_safetensors

    config, _ = CONFIGS[name]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    weights = draw_weights(config, seed)
    save_safetensors(folder / "model.safetensors", steady_routing(config, weights, seed) if steady else weights)
    return folder


def tokens_for(config: dict, length: int, salt: int = 0) -> list[int]:
    state = (7919 * salt + 32452843 * length + 313) & 0x7FFFFFFF
    out = []
    for _ in range(length):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % config["vocab"])
    return out
