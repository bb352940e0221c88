"""Kapolorn: a decoder whose layers are listed one by one in ``config.json``; a run of them may be looped.

``config.json`` keys: ``architecture`` ("Kapolorn"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``logit_softcap`` (absent or null: none), ``loop`` (``{"start", "stop", "times"}``: layers start .. stop-1 run ``times``
times in a row with the same weights, every pass with a cache and state of its own; absent: no loop) and ``layers``, a
list of ``{"type", "mixer", "mlp"}``.  ``type`` names the mixer:

* ``parallel``: two mixers side by side on the same input, summed as ``left_scale * left + right_scale * right``.
  ``left`` (``heads, kv_heads, dim, vdim, scale, mask.size, rot.dims, rot.base``) is softmax attention with rotary
  positions on the leading ``rot.dims`` entries of every query and key head (rotate-half pairing), over blocks of
  ``mask.size`` positions counted from the start of the sequence, with a learned logit per head (``sink``) in the
  denominator.  ``right`` (``heads, dim, vdim, gate_cap``) is a matrix memory with capped exponential gates.
* ``channel_delta`` (``heads, kv_heads, dim, vdim, conv``): the gated delta rule with a decay per key channel, short
  causal convolutions on q, k and v.

``mlp`` is ``null`` or ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "groups": {"count",
"keep"}}, "shared": {"ff", "limit"}}``: routed experts with clamped gated activations, scores from the softmax over
all experts, experts chosen from the best groups only, a shared expert for every token (``groups`` and ``shared`` may be
absent).  Every layer norms the input and the output of each sublayer (``norm1, norm1b, norm2, norm2b``).  The embedding
rows are multiplied by ``embedding.scale``; the output head is the embedding table itself, and the logits are bent by
``cap tanh(logits / cap)``.  Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*`` (``left.*`` and
``right.*`` in a ``parallel`` layer), ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.router``, ``l<i>.mlp.shared.gate|up|down``,
``final.norm``.  Nothing here fixes a size.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec, looped_schedule
from ..config.registry import register_architecture
from .rapitar import _need

LAYER_TYPES = ("parallel", "channel_delta")


@dataclass(frozen=True)
class KapolornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: float | None
    loop: tuple  # (start, stop, times)
    layers: tuple  # of (mixer PartSpec, feed-forward PartSpec)
    raw: dict


def _layers_2k(repeats: int) -> list:
    """Layer sizes of a model of 2,048 width: attention of 16 heads of 128 on 4 key/value heads over blocks of 1,024
    positions beside a matrix memory of 16 heads of 64 x 128; a delta-rule layer of 16 heads of 128 x 128; 32 experts of
    1,408 in 4 groups, of which 4 of the best 2 groups, and a shared expert of 1,536 (a token goes through 7,168 rows)."""
    moe = {"kind": "moe", "expert": {"ff": 1408, "limit": 7.0},
           "router": {"experts": 32, "top": 4, "groups": {"count": 4, "keep": 2}}, "shared": {"ff": 1536, "limit": 7.0}}
    pair = {"type": "parallel", "mlp": moe, "mixer": {
        "left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024},
                 "rot": {"dims": 64, "base": 10000.0}},
        "left_scale": 1.0,
        "right": {"heads": 16, "dim": 64, "vdim": 128, "gate_cap": 15.0},
        "right_scale": 1.0}}
    delta = {"type": "channel_delta", "mlp": moe, "mixer": {"heads": 16, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4}}
    return [pair, pair, pair, delta] * repeats


class KapolornArchitecture:
    name = "Kapolorn"
    layer_count_key = None  # the layers are a list: a shape with fewer layers is another list
    named_shapes = {
        "kapolorn-2k": {"architecture": "Kapolorn", "vocab": 32768, "width": 2048, "norm": {"eps": 1e-6},
                        "embedding": {"scale": 1.0}, "logit_softcap": 30.0, "layers": _layers_2k(2)},
        "kapolorn-tiny": {"architecture": "Kapolorn", "vocab": 256, "width": 64, "norm": {"eps": 1e-5},
                          "embedding": {"scale": 2.0}, "logit_softcap": 20.0, "loop": {"start": 1, "stop": 2, "times": 2},
                          "layers": [
            {"type": "parallel", "mlp": {"kind": "moe", "expert": {"ff": 32, "limit": 2.0},
                                         "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}},
                                         "shared": {"ff": 48, "limit": 3.0}},
             "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 24},
                                "rot": {"dims": 8, "base": 1000.0}},
                       "left_scale": 0.8, "right": {"heads": 2, "dim": 8, "vdim": 16, "gate_cap": 10.0}, "right_scale": 1.1}},
            {"type": "channel_delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 3}}]},
    }

    @staticmethod
    def _mixer(kind: str, m: dict[str, Any], width: int, eps: float, where: str) -> PartSpec:
        if kind not in LAYER_TYPES:
            raise ValueError(f"config.json: {where}: unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        if kind == "channel_delta":
            return PartSpec("channel_delta", dict(hidden_size=width, heads=_need(m, "heads", where), kv_heads=_need(m, "kv_heads", where),
                                                  dim=_need(m, "dim", where), vdim=_need(m, "vdim", where), conv=_need(m, "conv", where),
                                                  eps=eps))
        left, right = m.get("left") or {}, m.get("right") or {}
        lw, rw = where + ".left", where + ".right"
        rot = left.get("rot") or {}
        attention = dict(hidden_size=width, heads=_need(left, "heads", lw), kv_heads=_need(left, "kv_heads", lw),
                         dim=_need(left, "dim", lw), vdim=_need(left, "vdim", lw), scale=_need(left, "scale", lw, float),
                         window=_need(left.get("mask") or {}, "size", lw + ".mask"), mask="block", sink=True, weights="softmax",
                         rotary={"dims": _need(rot, "dims", lw + ".rot"), "base": _need(rot, "base", lw + ".rot", float)})
        memory = dict(hidden_size=width, heads=_need(right, "heads", rw), dim=_need(right, "dim", rw), vdim=_need(right, "vdim", rw),
                      gate_cap=_need(right, "gate_cap", rw, float), eps=eps)
        return PartSpec("side_by_side", dict(hidden_size=width, normed=False, left_scale=_need(m, "left_scale", where, float),
                                             right_scale=_need(m, "right_scale", where, float),
                                             left=PartSpec("window_attention", attention), right=PartSpec("matrix_memory", memory)))

    @staticmethod
    def _ffn(f, width: int, where: str) -> PartSpec:
        if f is None:
            return PartSpec("none", {})
        if f.get("kind") != "moe":
            raise ValueError(f"config.json: {where}: unknown feed-forward kind {f.get('kind')!r}")
        expert, router = f.get("expert") or {}, f.get("router") or {}
        params = dict(hidden_size=width, expert_size=_need(expert, "ff", where + ".expert"),
                      limit=_need(expert, "limit", where + ".expert", float), experts=_need(router, "experts", where + ".router"),
                      top=_need(router, "top", where + ".router"), scoring="all", router_bias=False)
        groups = router.get("groups")
        if groups is not None:
            params.update(groups=_need(groups, "count", where + ".router.groups"), keep=_need(groups, "keep", where + ".router.groups"))
        shared = f.get("shared")
        if shared is not None:
            params["shared"] = {"size": _need(shared, "ff", where + ".shared"), "limit": _need(shared, "limit", where + ".shared", float)}
        return PartSpec("moe", params)

    def parse_config(self, raw: dict[str, Any]) -> KapolornConfig:
        width = _need(raw, "width", "the model")
        eps = _need(raw.get("norm") or {}, "eps", "norm", float)
        scale = _need(raw.get("embedding") or {}, "scale", "embedding", float)
        cap = raw.get("logit_softcap")
        if cap is not None:
            cap = _need(raw, "logit_softcap", "the model", float)
            if not cap > 0:
                raise ValueError(f"config.json: logit_softcap must be positive, got {cap!r}")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            layers.append((self._mixer(entry.get("type"), entry.get("mixer") or {}, width, eps, where + ".mixer"),
                           self._ffn(entry.get("mlp"), width, where + ".mlp")))
        loop = raw.get("loop")
        if loop is None:
            bounds = (0, 0, 1)
        else:
            start, stop = loop.get("start"), loop.get("stop")
            for key, value in (("start", start), ("stop", stop)):
                if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                    raise ValueError(f"config.json: loop.{key} must be a non-negative integer, got {value!r}")
            bounds = (start, stop, _need(loop, "times", "loop"))
            if not start <= stop <= len(layers):
                raise ValueError(f"config.json: a loop over layers {start} .. {stop - 1} does not fit {len(layers)} layers")
        return KapolornConfig(_need(raw, "vocab", "the model"), width, eps, scale, cap, bounds, tuple(layers), dict(raw))

    def model_spec(self, config: KapolornConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "weight_suffix": ""})
        layers = [LayerSpec(block="sandwich_residual", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, prefix=f"l{i}")
                  for i, (mixer, ffn) in enumerate(config.layers)]
        return ModelSpec(architecture=self.name, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                         schedule=looped_schedule(len(layers), *config.loop), final_norm=norm, embedding_name="embed",
                         final_norm_prefix="final.norm", head_name="head", tie_word_embeddings=True,
                         embedding_scale=config.embedding_scale, logit_softcap=config.logit_softcap, raw=config.raw)


register_architecture(KapolornArchitecture(), replace=True)
