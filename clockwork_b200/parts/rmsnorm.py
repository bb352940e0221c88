"""RMSNorm over the float32 residual stream, fused with the pending residual add.

Reference: ``clockwork/engine/model.py:38-49`` (float32 statistics, ``x * rsqrt(mean(x^2) +
eps)``, then the weight) and ``:150``/``:154`` (the residual sums the norm kernel absorbs).
Parameters: ``size``, ``eps``; optional ``offset`` (added to the stored weight: with 1.0 the checkpoint holds the weight's
distance from one and the norm multiplies by ``1 + w``) and ``weight_suffix`` (the tensor's name
behind the prefix, ``weight`` by default; empty: the prefix itself is the name).  Tensor: [size], kept
in float32.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops.gemm import RowScaled
from ..weights.decl import TensorDecl
from .base import Norm, ResidualStream
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True
    graph_safe_portions = True
    takes_partial_sums = True  # ``forward`` hands whatever the stream holds to ``ops.add_rmsnorm``, slabs included

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.offset = float(spec.get("offset", 0.0))
        suffix = spec.get("weight_suffix", "weight")
        self.weight_name = self.name(suffix) if suffix else self.prefix
        self.weight: torch.Tensor | None = None

    def tensor_decls(self):
        yield TensorDecl(self.weight_name, (self.size,), role="vector", init="zeros" if self.offset else "norm")

    def load_weights(self, fetch) -> None:
        self.weight = fetch(self.weight_name)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()  # float32: exact for a weight stored in bfloat16

    def split_weight(self) -> torch.Tensor | None:
        """The weight a preceding product multiplies into the residual when it begins this norm."""
        return self.weight if self.dtype == torch.bfloat16 else None

    def forward(self, stream: ResidualStream, status: torch.Tensor, lazy: bool = False):
        ready, stream.normed = stream.normed, None
        if ready is not None and ready[0] is self and stream.pending is None:
            return ready[1]  # the block before already ran this norm on the residual as it stands
        half, stream.half_norm = stream.half_norm, None
        if lazy and half is not None and stream.pending is None and half[0] is self.weight:
            # the product that wrote the residual began this norm; the product that reads it finishes it
            residual, weight, eps, dtype = stream.residual, self.weight, self.eps, self.dtype
            return RowScaled(half[1], half[2], eps, self.size,
                             lambda: ops.add_rmsnorm(residual, None, weight, eps, dtype, status))
        delta, stream.pending = stream.pending, None
        return ops.add_rmsnorm(stream.residual, delta, self.weight, self.eps, self.dtype, status)

    def add_normed(self, stream: ResidualStream, terms) -> None:
        """``residual += norm(sum of factor * tensor over the terms) * weight``: this norm behind a sublayer, whose output
        comes as one or two pairs (float32 [N, size], factor).  Statistics, sum and residual are float32."""
        ops.sum_rmsnorm_add(stream.residual_after_flush(), terms, self.weight, self.eps)

    def scaled_add(self, x: torch.Tensor, terms, into: torch.Tensor | None = None) -> torch.Tensor:
        """``y = x + sum of factor * tensor over the terms`` (float32; one or two pairs) goes to ``into`` (``x`` itself when
        None); returns this norm of ``y``."""
        return ops.axpy_rmsnorm(x, terms, self.weight, self.eps, self.dtype, into)

    def weight_and_eps(self) -> tuple:
        """(weight, eps) for a kernel that runs this norm at the end of other work."""
        return self.weight, self.eps

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        stream.flush()
        return ops.rmsnorm_rows(stream.residual, rows, self.weight, self.eps, self.dtype, status)


register_norm("rmsnorm", RMSNorm, replace=True)
