"""Pre-norm residual block: ``h += mixer(norm1(h)); h += ffn(norm2(h))``.

Reference: ``clockwork/engine/model.py:131-154``.  The block owns the arrangement only; its
mixer, feed-forward and norms are whatever the layer's spec names.  Tensor prefixes follow the
Hugging Face layout: ``<layer>.self_attn``, ``<layer>.mlp``, ``<layer>.input_layernorm``,
``<layer>.post_attention_layernorm``.
"""

from __future__ import annotations

from ..config.model_spec import LayerSpec
from .base import Block, ResidualStream, StepContext
from .registry import build_part, register_block


class PreNormResidualBlock(Block):
    NAMES = ("input_layernorm", "self_attn", "post_attention_layernorm", "mlp")  # first norm, mixer, second norm, feed-forward

    def __init__(self, layer: LayerSpec, dtype, device) -> None:
        self.layer = layer
        self.prefix = layer.prefix
        self.dtype, self.device = dtype, device
        norm1, mixer, norm2, ffn = self.NAMES
        self.mixer_norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.{norm1}", dtype, device)
        self.mixer = build_part("mixer", layer.mixer, f"{layer.prefix}.{mixer}", dtype, device)
        self.ffn_norm = self.ffn = None  # a layer without a feed-forward names the kind ``none``
        if layer.ffn.kind != "none":
            self.ffn_norm = build_part("norm", layer.ffn_norm, f"{layer.prefix}.{norm2}", dtype, device)
            self.ffn = build_part("ffn", layer.ffn, f"{layer.prefix}.{ffn}", dtype, device)

    def parts(self):
        return (self.mixer_norm, self.mixer) + (() if self.ffn is None else (self.ffn_norm, self.ffn))

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def tensor_decls(self):
        for part in self.parts():
            yield from part.tensor_decls()

    def load_weights(self, fetch) -> None:
        for part in self.parts():
            part.load_weights(fetch)

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _normed(norm, consumer, stream: ResidualStream, status):
        if getattr(consumer, "takes_half_normed", False) and hasattr(norm, "split_weight"):
            return norm.forward(stream, status, lazy=True)
        return norm.forward(stream, status)

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        x = self._normed(self.mixer_norm, self.mixer, stream, ctx.status)
        stream.next_norm = self.ffn_norm if self.ffn is not None else following_norm  # what the mixer's output product may begin
        stream.push(self.mixer.forward(ctx, x, view, stream))
        if self.ffn is None:
            stream.next_norm = None
            return
        x = self._normed(self.ffn_norm, self.ffn, stream, ctx.status)
        stream.next_norm = following_norm
        stream.push(self.ffn.forward(ctx, x, stream))
        stream.next_norm = None


class ShortNamePreNormBlock(PreNormResidualBlock):
    """The same arrangement with the tensor prefixes ``<layer>.norm1``, ``<layer>.mix``, ``<layer>.norm2``, ``<layer>.mlp``."""

    NAMES = ("norm1", "mix", "norm2", "mlp")


class SandwichResidualBlock(Block):
    """A norm before and after each sublayer: ``h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h)))``.

    The mixer and the feed-forward hand their outputs over as terms of a sum that is not yet formed
    (``Mixer.mix_terms``, ``FeedForward.output_terms``: float32 tensors with factors); one float32 kernel forms the sum,
    norms it over the width and adds it into the residual.  Tensor prefixes: ``<layer>.norm1``, ``.mix``, ``.norm2``,
    ``.mlp`` and the norms behind the sublayers ``.norm1b``, ``.norm2b`` (parts of the same kind as the norms in front).
    A layer may have no feed-forward (kind ``none``)."""

    NAMES = ("norm1", "mix", "norm2", "mlp", "norm1b", "norm2b")

    def __init__(self, layer: LayerSpec, dtype, device) -> None:
        self.layer = layer
        self.prefix = layer.prefix
        self.dtype, self.device = dtype, device
        norm1, mixer, norm2, ffn, norm1b, norm2b = self.NAMES
        self.mixer_norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.{norm1}", dtype, device)
        self.mixer = build_part("mixer", layer.mixer, f"{layer.prefix}.{mixer}", dtype, device)
        self.mixer_out_norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.{norm1b}", dtype, device)
        self.ffn_norm = self.ffn = self.ffn_out_norm = None
        if layer.ffn.kind != "none":
            self.ffn_norm = build_part("norm", layer.ffn_norm, f"{layer.prefix}.{norm2}", dtype, device)
            self.ffn = build_part("ffn", layer.ffn, f"{layer.prefix}.{ffn}", dtype, device)
            self.ffn_out_norm = build_part("norm", layer.ffn_norm, f"{layer.prefix}.{norm2b}", dtype, device)
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"norm kind {layer.mixer_norm.kind!r} cannot norm a sublayer's output (no add_normed)")

    def parts(self):
        first = (self.mixer_norm, self.mixer, self.mixer_out_norm)
        return first + (() if self.ffn is None else (self.ffn_norm, self.ffn, self.ffn_out_norm))

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def tensor_decls(self):
        for part in self.parts():
            yield from part.tensor_decls()

    def load_weights(self, fetch) -> None:
        for part in self.parts():
            part.load_weights(fetch)

    def first_norm(self):
        return self.mixer_norm

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        stream.next_norm = None  # (no product adds into the residual here: every output passes a norm first)
        x = self.mixer_norm.forward(stream, ctx.status)
        self.mixer_out_norm.add_normed(stream, self.mixer.mix_terms(ctx, x, view))
        if self.ffn is None:
            return
        x = self.ffn_norm.forward(stream, ctx.status)
        self.ffn_out_norm.add_normed(stream, self.ffn.output_terms(ctx, x))


register_block("sandwich_residual", SandwichResidualBlock, replace=True)
register_block("prenorm_residual", PreNormResidualBlock, replace=True)
register_block("prenorm_residual_short", ShortNamePreNormBlock, replace=True)
