"""A pre-norm residual block whose contributions are scaled, and whose output is a weighted average over the depth:

    y = x + m * mixer(norm1(x));   y <- y + m * ffn(norm2(y))        (a layer may have no feed-forward)
    X_(r+1) = y;   what the next layer reads: sum over j <= r + 1 of c[j] * X_j

with X_0 the model's input rows, X_(j+1) what layer run j left (before the average), m the block parameter
``residual_mult`` and c the layer's tensor ``<layer>.dwa`` (run r has r + 2 coefficients).  The model keeps the planes X_j
(``ModelSpec.keeps_layer_outputs``; ``ResidualStream.layer_outputs``).  Tensor prefixes: ``<layer>.norm1``, ``.mix``,
``.norm2``, ``.mlp``.

The mixer hands its output over as terms of a sum (``Mixer.mix_terms``: float32, added to nothing), the feed-forward
likewise (``FeedForward.output_terms``).  Two float32 kernels do the rest: one adds the scaled mixer output and runs the
second norm; one adds the scaled feed-forward output, stores the plane, forms the average and, when the next block's
first norm is known, runs that norm too.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.model_spec import LayerSpec
from ..weights.decl import TensorDecl
from .base import Block, ResidualStream, StepContext
from .registry import build_part, register_block


class DepthAveragedBlock(Block):
    NAMES = ("norm1", "mix", "norm2", "mlp", "dwa")

    def __init__(self, layer: LayerSpec, dtype, device) -> None:
        self.layer = layer
        self.prefix = layer.prefix
        self.dtype, self.device = dtype, device
        norm1, mixer, norm2, ffn, coef = self.NAMES
        self.mult = float(layer.block_params.get("residual_mult", 1.0))
        self.run = int(layer.block_params["run"])  # which layer run of the model this is: its plane is run + 1
        self.coef_name = f"{layer.prefix}.{coef}"
        self.coef: torch.Tensor | None = None
        self.mixer_norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.{norm1}", dtype, device)
        self.mixer = build_part("mixer", layer.mixer, f"{layer.prefix}.{mixer}", dtype, device)
        self.ffn_norm = self.ffn = None
        if layer.ffn.kind != "none":
            self.ffn_norm = build_part("norm", layer.ffn_norm, f"{layer.prefix}.{norm2}", dtype, device)
            self.ffn = build_part("ffn", layer.ffn, f"{layer.prefix}.{ffn}", dtype, device)
            if not hasattr(self.ffn_norm, "scaled_add"):
                raise ValueError(f"norm kind {layer.ffn_norm.kind!r} cannot follow a scaled contribution (no scaled_add)")

    def parts(self):
        return (self.mixer_norm, self.mixer) + (() if self.ffn is None else (self.ffn_norm, self.ffn))

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def tensor_decls(self):
        for part in self.parts():
            yield from part.tensor_decls()
        yield TensorDecl(self.coef_name, (self.run + 2,), "vector", "mean_weights")

    def load_weights(self, fetch) -> None:
        for part in self.parts():
            part.load_weights(fetch)
        self.coef = fetch(self.coef_name).contiguous()

    def first_norm(self):
        return self.mixer_norm

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        planes, run = stream.layer_outputs, stream.runs_done
        if planes is None:
            raise RuntimeError("this block needs the earlier layers' outputs (ModelSpec.keeps_layer_outputs)")
        if run != self.run:
            raise RuntimeError(f"layer run {run} reached the block of run {self.run}")
        stream.next_norm = None  # (no product adds into the residual here)
        x = self.mixer_norm.forward(stream, ctx.status)
        terms = [(t, f * self.mult) for t, f in self.mixer.mix_terms(ctx, x, view)]
        rows = stream.residual_after_flush()
        # where the average goes: over the rows just read, unless they are a plane that later layers read again
        if rows.data_ptr() == planes[0].data_ptr():
            if stream.spare is None:
                stream.spare = torch.empty_like(rows)
            into = stream.spare
        else:
            into = rows
        if self.ffn is not None:
            plane = planes[run + 1]
            x = self.ffn_norm.scaled_add(rows, terms, into=plane)
            terms = [(t, f * self.mult) for t, f in self.ffn.output_terms(ctx, x)]
            rows = plane
        weight, eps = following_norm.weight_and_eps() if hasattr(following_norm, "weight_and_eps") else (None, 0.0)
        normed = ops.depth_average(rows, terms, planes, run + 1, self.coef, into, weight, eps, self.dtype)
        stream.residual = into
        stream.runs_done = run + 1
        stream.normed = (following_norm, normed) if normed is not None else None


register_block("depth_averaged_residual", DepthAveragedBlock, replace=True)
