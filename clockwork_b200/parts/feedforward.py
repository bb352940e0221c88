"""Feed-forwards besides SwiGLU: a dense two-matrix layer with GELU, and a mixture of experts.

``gelu_mlp``: ``down(gelu_tanh(up(x)))``, no biases.  Parameters: ``hidden_size, intermediate_size``;
tensors ``up`` [I, H], ``down`` [H, I].

``moe``: ``experts`` SwiGLU experts without biases (``e<i>.gate``, ``e<i>.up`` [F, H], ``e<i>.down``
[H, F]), a router ``router`` [E, H] with bias ``router.b``.  Router logits are a product with float32
accumulation and stay float32; each token takes
the ``top`` experts with the largest logits, weighted by the softmax over the chosen logits only; the
output is the weighted sum of the chosen experts' outputs, added into the float32 residual in the order
of the choices.  Tokens are grouped by expert on the device (no host round trip), so the part is safe
to capture in a CUDA graph.  Parameters: ``hidden_size, expert_size, experts, top``, and optionally

* ``scoring``: ``"chosen"`` (the default, as above), ``"all"``: the weights are the chosen experts' shares of the
  softmax over all experts, not renormalised, or ``"sigmoid"``: an expert's score is the sigmoid of its logit, and the
  weights are the chosen experts' scores, not renormalised;
* ``correction`` (with ``"sigmoid"``): experts are ranked, alone and in their runs, by score + ``correction[e]`` (tensor
  ``correction`` [E]); the weights do not contain it;
* ``weight_scale``: every weight is multiplied by it;
* ``groups, keep``: the experts lie in ``groups`` equal runs of neighbours and only experts of the ``keep`` best runs can
  be chosen; a run counts as the sum of its ``group_rank`` largest entries (1, the default: as its best expert);
* ``limit``: a positive number selects the clamped activation ``a sigmoid(1.702 a) (b + 1)`` with ``a = min(gate(x),
  limit)`` and ``b = clamp(up(x), -limit, limit)`` instead of ``silu(gate(x)) up(x)``;
* ``router_bias``: whether the router has a bias (tensor ``router.b``; the default) or not;
* ``shared``: ``{"size", "limit"}``: one more expert of the same form (tensors ``shared.gate|up|down``) that every token
  uses with weight one.

In a block that norms the feed-forward's output (``output_terms``) the sum of the experts' outputs is formed in a float32
buffer of its own instead of in the residual.
"""

from __future__ import annotations

import torch

from ..ops import gemm as gemm_ops
from ..ops import grouped as grouped_ops
from ..ops import recurrence as rec_ops
from ..weights.decl import TensorDecl
from .base import FeedForward, ResidualStream, StepContext
from .linear import Linear
from .registry import register_ffn


class GeluMLP(FeedForward):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.up: Linear | None = None
        self.down: Linear | None = None

    def tensor_decls(self):
        h, i = self.hidden_size, self.intermediate_size
        yield TensorDecl(self.name("up"), (i, h), "matrix", "linear")
        yield TensorDecl(self.name("down"), (h, i), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.up = Linear(fetch(self.name("up")))
        self.down = Linear(fetch(self.name("down")))

    def forward(self, ctx: StepContext, x, stream: ResidualStream):
        act = rec_ops.activation_(self.up(x), rec_ops.ACT_GELU_TANH)
        return self.down.add_or_defer(act, stream)


class MixtureOfExperts(FeedForward):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.hidden_size = int(spec["hidden_size"])
        self.expert_size = int(spec["expert_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        if not 0 < self.top <= self.experts:
            raise ValueError(f"top {self.top} must lie in 1..experts ({self.experts})")
        scoring = str(spec.get("scoring", "chosen"))
        modes = {"chosen": grouped_ops.SCORE_CHOSEN, "all": grouped_ops.SCORE_ALL, "sigmoid": grouped_ops.SCORE_SIGMOID}
        if scoring not in modes:
            raise ValueError(f"scoring must be one of {sorted(modes)}, got {scoring!r}")
        self.scoring = modes[scoring]
        self.has_correction = bool(spec.get("correction", False))
        if self.has_correction and scoring != "sigmoid":
            raise ValueError("a correction per expert goes with sigmoid scores")
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        self.groups, self.keep = int(spec.get("groups", 1)), int(spec.get("keep", 1))
        self.group_rank = int(spec.get("group_rank", 1))
        if not 1 <= self.group_rank <= min(4, max(1, int(spec["experts"]) // max(1, self.groups))):
            raise ValueError(f"group_rank {self.group_rank} must lie in 1..4 and within a run of experts")
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts do not lie in {self.groups} equal groups of which {self.keep} are kept")
        if self.keep * (self.experts // self.groups) < self.top:
            raise ValueError(f"the {self.keep} kept groups hold fewer than top = {self.top} experts")
        self.limit = float(spec.get("limit") or 0.0)
        self.has_router_bias = bool(spec.get("router_bias", True))
        shared = spec.get("shared")
        self.shared_size = int(shared["size"]) if shared else 0
        self.shared_limit = float(shared.get("limit") or 0.0) if shared else 0.0
        self.w_gate = self.w_up = self.w_down = self.router = self.router_bias = self.correction = None
        self.shared_gate = self.shared_up = self.shared_down = None

    def tensor_decls(self):
        h, f = self.hidden_size, self.expert_size
        for e in range(self.experts):
            yield TensorDecl(self.name(f"e{e}.gate"), (f, h), "matrix", "linear")
            yield TensorDecl(self.name(f"e{e}.up"), (f, h), "matrix", "linear")
            yield TensorDecl(self.name(f"e{e}.down"), (h, f), "matrix", "linear")
        yield TensorDecl(self.name("router"), (self.experts, h), "matrix", "linear")
        if self.has_router_bias:
            yield TensorDecl(self.name("router.b"), (self.experts,), "vector", "bias")
        if self.has_correction:
            yield TensorDecl(self.name("correction"), (self.experts,), "vector", "bias")
        if self.shared_size:
            yield TensorDecl(self.name("shared.gate"), (self.shared_size, h), "matrix", "linear")
            yield TensorDecl(self.name("shared.up"), (self.shared_size, h), "matrix", "linear")
            yield TensorDecl(self.name("shared.down"), (h, self.shared_size), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        stack = lambda what: torch.stack([fetch(self.name(f"e{e}.{what}")) for e in range(self.experts)]).contiguous()  # noqa: E731
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.router = Linear(fetch(self.name("router")))
        self.router_bias = fetch(self.name("router.b")) if self.has_router_bias else None
        self.correction = fetch(self.name("correction")).contiguous() if self.has_correction else None
        if self.shared_size:
            self.shared_gate = fetch(self.name("shared.gate")).unsqueeze(0).contiguous()  # one "expert" that every row goes through
            self.shared_up = fetch(self.name("shared.up")).unsqueeze(0).contiguous()
            self.shared_down = Linear(fetch(self.name("shared.down")))

    def _routed(self, ctx: StepContext, x):
        """(the chosen experts' outputs float32 [N*top, hidden] in choice order, the choices, their weights)."""
        sel, weights = grouped_ops.moe_choose(self.router.to_float32(x), self.router_bias, ctx.tok_seq, self.top, self.scoring,
                                              self.groups, self.keep, correction=self.correction, weight_scale=self.weight_scale,
                                              group_rank=self.group_rank)
        offsets, order = grouped_ops.moe_group(sel, self.experts)
        act = grouped_ops.expert_gate_up(x, self.w_gate, self.w_up, offsets, order, self.top, self.limit)
        return grouped_ops.expert_down(act, self.w_down, offsets, order), sel, weights

    def _shared_act(self, x):
        if self.shared_limit > 0.0:  # one dense gated product: the tensor-core kernel where it takes the sizes
            act = gemm_ops.clamped_gated_tc(x, self.shared_gate[0], self.shared_up[0], self.shared_limit)
            if act is not None:
                return act
        return grouped_ops.expert_gate_up(x, self.shared_gate, self.shared_up, None, None, 1, self.shared_limit)

    def forward(self, ctx: StepContext, x, stream: ResidualStream):
        y, sel, weights = self._routed(ctx, x)
        if self.shared_size:
            self.shared_down.add_into(self._shared_act(x), stream.residual_after_flush(), None)
        grouped_ops.moe_combine(stream.residual_after_flush(), y, sel, weights)
        return None

    def output_terms(self, ctx: StepContext, x):
        y, sel, weights = self._routed(ctx, x)
        if self.shared_size:
            out = self.shared_down.to_float32(self._shared_act(x))
            grouped_ops.moe_combine(out, y, sel, weights)  # (the rows of no request keep what the shared expert made of them)
        else:
            out = torch.empty((x.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
            grouped_ops.moe_combine(out, y, sel, weights, assign=True)
        return [(out, 1.0)]


register_ffn("gelu_mlp", GeluMLP, replace=True)
register_ffn("moe", MixtureOfExperts, replace=True)
