"""Nuzulorn: a decoder whose layers are listed one by one in ``config.json``, with a second embedding table read by a hash
of (previous token, token), scaled residual contributions and a weighted average over the depth behind every layer.

``config.json`` keys: ``architecture`` ("Nuzulorn"), ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
``embedding.bigram`` (``buckets, mul_prev, mul_cur``) and ``layers``, a list of ``{"type", "mixer", "mlp"}``.  ``type`` names
the mixer:

* ``attention`` (``heads, kv_heads, dim, vdim, scale, mask.size, mask.pool, rot.dims, rot.base``): softmax attention over
  a sliding window of ``mask.size`` positions and, before it, one key and value per whole block of ``mask.pool`` positions
  (the block's means); rotary positions on the leading ``rot.dims`` entries of every query and key head (rotate-half
  pairing); one added to the softmax's denominator; an output gate per head; biases on q, k, v and the output product.
* ``attention_2`` (``heads, kv_heads, dim, vdim, scale, softcap, q_temp.coef, q_temp.every``): causal softmax attention
  without rotation: a query temperature that grows with the logarithm of the position, capped scores, a distance bias with
  slopes ``2^(-8 (h + 1) / heads)``, a learned logit per head in the denominator; biases on q, k, v.
* ``hgrn2`` (``heads, dim, vdim``): linear attention whose forget gate, bounded from below, also decides what is written.

``mlp`` is ``null`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count",
"keep"}}}``: routed experts with sigmoid scores, ranked with a correction per expert, chosen from the best groups of
neighbours (a group counts as the sum of its two best), weighted by score times ``router.scale``.  Tensor names: ``embed``,
``bigram``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.router|correction``, ``l<i>.dwa``,
``final.norm``.  The output head is the embedding table.  Nothing here fixes a size.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec, sequential_schedule
from ..config.registry import register_architecture
from .rapitar import _need

LAYER_TYPES = ("attention", "attention_2", "hgrn2")
DISTANCE_HALVINGS = 8.0  # head h's distance slope is 2^(-8 (h + 1) / heads)
GROUP_RANK = 2           # a group of experts counts as the sum of its two largest entries


@dataclass(frozen=True)
class NuzulornConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    pair: dict  # buckets, mul_prev, mul_cur
    layers: tuple  # of (mixer PartSpec, feed-forward PartSpec)
    raw: dict


def _layers_2k(repeats: int) -> list:
    """Layer sizes of a model of 2,048 width: capped causal attention of 16 heads of 128 on 4 key/value heads; windowed
    attention of 16 heads of 128 on 4 key/value heads over 1,024 positions with blocks of 64 pooled before them; a recurrent
    layer of 16 heads of 128 x 128; 32 experts of 1,792 in 4 groups, of which 4 of the best 2 groups (a token goes through
    7,168 rows)."""
    moe = {"kind": "moe", "expert": {"ff": 1792}, "router": {"experts": 32, "top": 4, "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
    capped = {"type": "attention_2", "mlp": moe, "mixer": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                          "softcap": 30.0, "q_temp": {"coef": 0.1, "every": 1024}}}
    windowed = {"type": "attention", "mlp": moe, "mixer": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                          "mask": {"size": 1024, "pool": 64}, "rot": {"dims": 64, "base": 10000.0}}}
    recurrent = {"type": "hgrn2", "mlp": moe, "mixer": {"heads": 16, "dim": 128, "vdim": 128}}
    return [capped, windowed, windowed, recurrent] * repeats


class NuzulornArchitecture:
    name = "Nuzulorn"
    layer_count_key = None  # the layers are a list: a shape with fewer layers is another list
    named_shapes = {
        "nuzulorn-2k": {"architecture": "Nuzulorn", "vocab": 32768, "width": 2048, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
                        "embedding": {"bigram": {"buckets": 65521, "mul_prev": 8191, "mul_cur": 131}}, "layers": _layers_2k(2)},
        "nuzulorn-tiny": {"architecture": "Nuzulorn", "vocab": 256, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
                          "embedding": {"bigram": {"buckets": 61, "mul_prev": 7, "mul_cur": 3}}, "layers": [
            {"type": "attention", "mlp": {"kind": "moe", "expert": {"ff": 32},
                                          "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}},
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 20, "pool": 5},
                       "rot": {"dims": 8, "base": 1000.0}}},
            {"type": "hgrn2", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 16}},
            {"type": "attention_2", "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 4, "top": 1, "scale": 2.0}},
             "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.25, "softcap": 5.0,
                       "q_temp": {"coef": 0.3, "every": 16}}}]},
    }

    @staticmethod
    def _mixer(kind: str, m: dict[str, Any], width: int, eps: float, where: str) -> PartSpec:
        if kind not in LAYER_TYPES:
            raise ValueError(f"config.json: {where}: unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        if kind == "hgrn2":
            return PartSpec("hgrn2", dict(hidden_size=width, heads=_need(m, "heads", where), dim=_need(m, "dim", where),
                                          vdim=_need(m, "vdim", where), eps=eps))
        common = dict(hidden_size=width, heads=_need(m, "heads", where), kv_heads=_need(m, "kv_heads", where), dim=_need(m, "dim", where),
                      vdim=_need(m, "vdim", where), scale=_need(m, "scale", where, float), weights="softmax", bias=True)
        if kind == "attention":
            mask, rot = m.get("mask") or {}, m.get("rot") or {}
            return PartSpec("window_attention", dict(
                common, window=_need(mask, "size", where + ".mask"), pool=_need(mask, "pool", where + ".mask"), sink="zero", gate=True,
                out_bias=True, rotary={"dims": _need(rot, "dims", where + ".rot"), "base": _need(rot, "base", where + ".rot", float)}))
        temp = m.get("q_temp") or {}
        return PartSpec("window_attention", dict(
            common, window=None, sink=True, out_bias=False, softcap=_need(m, "softcap", where, float),
            distance_bias={"halvings": DISTANCE_HALVINGS},
            query_temperature={"coef": _need(temp, "coef", where + ".q_temp", float), "every": _need(temp, "every", where + ".q_temp")}))

    @staticmethod
    def _ffn(f, width: int, where: str) -> PartSpec:
        if f is None:
            return PartSpec("none", {})
        if f.get("kind") != "moe":
            raise ValueError(f"config.json: {where}: unknown feed-forward kind {f.get('kind')!r}")
        expert, router = f.get("expert") or {}, f.get("router") or {}
        params = dict(hidden_size=width, expert_size=_need(expert, "ff", where + ".expert"), experts=_need(router, "experts", where + ".router"),
                      top=_need(router, "top", where + ".router"), scoring="sigmoid", correction=True, router_bias=False,
                      weight_scale=_need(router, "scale", where + ".router", float))
        groups = router.get("groups")
        if groups is not None:
            params.update(groups=_need(groups, "count", where + ".router.groups"), keep=_need(groups, "keep", where + ".router.groups"))
            params["group_rank"] = min(GROUP_RANK, params["experts"] // max(1, params["groups"]))
        return PartSpec("moe", params)

    def parse_config(self, raw: dict[str, Any]) -> NuzulornConfig:
        width = _need(raw, "width", "the model")
        eps = _need(raw.get("norm") or {}, "eps", "norm", float)
        mult = _need(raw, "residual_mult", "the model", float)
        pair = (raw.get("embedding") or {}).get("bigram") or {}
        pair = {key: _need(pair, key, "embedding.bigram") for key in ("buckets", "mul_prev", "mul_cur")}
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            layers.append((self._mixer(entry.get("type"), entry.get("mixer") or {}, width, eps, where + ".mixer"),
                           self._ffn(entry.get("mlp"), width, where + ".mlp")))
        return NuzulornConfig(_need(raw, "vocab", "the model"), width, eps, mult, pair, tuple(layers), dict(raw))

    def model_spec(self, config: NuzulornConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "weight_suffix": ""})
        layers = [LayerSpec(block="depth_averaged_residual", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, prefix=f"l{i}",
                            block_params={"residual_mult": config.residual_mult, "run": i})
                  for i, (mixer, ffn) in enumerate(config.layers)]
        pair = PartSpec("hashed_pair", dict(config.pair, size=config.width, name="bigram", vocab=config.vocab))
        return ModelSpec(architecture=self.name, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                         schedule=sequential_schedule(len(layers)), final_norm=norm, embedding_name="embed",
                         final_norm_prefix="final.norm", head_name="head", tie_word_embeddings=True,
                         pair_embedding=pair, keeps_layer_outputs=True, raw=config.raw)


register_architecture(NuzulornArchitecture(), replace=True)
