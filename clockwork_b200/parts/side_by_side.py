"""Two mixers side by side: both read the same input, each output is RMS-normed over the model's width
with a weight of its own, and the mixer's result is ``factor`` times their sum:

    out = factor * (n(left(h)) g_left + n(right(h)) g_right),   n(y) = y / sqrt(mean(y^2) + eps)

or, with ``normed = False``, the plain weighted sum ``left_scale * left(h) + right_scale * right(h)`` (no tensors of
its own; such a mixer stands in a block that norms the sum, and hands it over as two terms: ``mix_terms``).

Parameters: ``hidden_size, eps, factor`` (0.5: half the sum), ``left`` and ``right`` (the ``PartSpec`` of any
registered mixer that has ``mix``); or ``normed = False, left_scale, right_scale``.  Tensors: the mixers' own under
``<prefix>.left`` and ``<prefix>.right``, and (normed) the two weights ``left.out`` and ``right.out`` [hidden].  What the two keep per request is asked for as a tuple (pages
of the one, a state slot of the other); the norms and the sum into the residual are one float32 kernel.

The two mixers share nothing but their input, so the left one's kernels are launched on a second stream of the device
and meet the right one's at the kernel that adds both up (``SideBySide.concurrent = False``: one after the other on
the step's stream; the results are the same bits).  In a captured step the two chains become parallel branches of the
graph.  Every tensor the left mixer makes is made and last used inside that fork and join, so the allocator's
per-stream pools never hand memory on while the other stream still reads it.
"""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Mixer, PagedKVNeed, ResidualStream, SlotStateNeed, StepContext
from .registry import build_part, register_mixer


_side_streams: dict[int, "torch.cuda.Stream"] = {}  # one second stream per device, shared by every layer


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    index = device.index if device.index is not None else torch.cuda.current_device()
    stream = _side_streams.get(index)
    if stream is None:
        stream = _side_streams[index] = torch.cuda.Stream(device=index)
    return stream


class SideBySide(Mixer):
    concurrent = True  # the left mixer on a second stream beside the right one

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.normed = bool(p.get("normed", True))
        self.eps = float(p.get("eps", 0.0))
        self.factor = float(p.get("factor", 0.5))
        self.left_scale, self.right_scale = float(p.get("left_scale", 1.0)), float(p.get("right_scale", 1.0))
        self.left = build_part("mixer", p["left"], self.name("left"), dtype, device)
        self.right = build_part("mixer", p["right"], self.name("right"), dtype, device)
        self.graph_safe = bool(self.left.graph_safe and self.right.graph_safe)
        self.graph_safe_portions = bool(self.left.graph_safe_portions and self.right.graph_safe_portions)
        self.left_weight = self.right_weight = None
        needs = [m.cache_need() for m in (self.left, self.right)]
        if any(isinstance(n, tuple) for n in needs):
            raise ValueError("a mixer inside side_by_side must keep one thing per request at most")
        for kind in (PagedKVNeed, SlotStateNeed):
            if sum(isinstance(n, kind) for n in needs) > 1:
                raise ValueError(f"both mixers of {prefix!r} keep {kind.__name__}: one layer has one of each at most")
        self._needs = needs
        self._forked = self._joined = None  # events of the fork and the join (made at first use)

    def cache_need(self):
        kept = tuple(n for n in self._needs if n is not None)
        return kept or None

    def _views(self, view):
        """The views of the two mixers from the tuple that follows ``cache_need``'s order."""
        views = iter(view if isinstance(view, tuple) else (() if view is None else (view,)))
        return tuple(next(views) if n is not None else None for n in self._needs)

    # hooks of captured steps: whatever either mixer declares
    def step_scalars(self):
        return {**self.right.step_scalars(), **self.left.step_scalars()}

    def step_arrays(self, *args, **kwargs):
        return {**self.right.step_arrays(*args, **kwargs), **self.left.step_arrays(*args, **kwargs)}

    def reserve_for_steps(self, max_seqs: int, max_ctx: int) -> None:
        self.left.reserve_for_steps(max_seqs, max_ctx)
        self.right.reserve_for_steps(max_seqs, max_ctx)

    def tensor_decls(self):
        yield from self.left.tensor_decls()
        yield from self.right.tensor_decls()
        if not self.normed:
            return
        yield TensorDecl(self.name("left.out"), (self.hidden_size,), "vector", "norm")
        yield TensorDecl(self.name("right.out"), (self.hidden_size,), "vector", "norm")

    def load_weights(self, fetch) -> None:
        self.left.load_weights(fetch)
        self.right.load_weights(fetch)
        if not self.normed:
            return
        self.left_weight = fetch(self.name("left.out")).contiguous()
        self.right_weight = fetch(self.name("right.out")).contiguous()

    def mix_terms(self, ctx: StepContext, x, view):
        if self.normed:
            raise NotImplementedError("a side_by_side mixer that norms its two outputs adds them into the residual itself")
        a, b = self._both(ctx, x, view)
        return [(a, self.left_scale), (b, self.right_scale)]

    def forward(self, ctx: StepContext, x, view, stream: ResidualStream):
        if not self.normed:
            raise NotImplementedError("a side_by_side mixer without norms of its own stands in a block that norms its output")
        a, b = self._both(ctx, x, view)
        ops.pair_rmsnorm_add(stream.residual_after_flush(), a, b, self.left_weight, self.right_weight, self.eps, self.factor)
        return None

    def _both(self, ctx: StepContext, x, view):
        """The two mixers' outputs (float32 [N, hidden] each), the left one's kernels on the second stream."""
        left_view, right_view = self._views(view)
        if self.concurrent and x.is_cuda:
            if self._forked is None:
                self._forked, self._joined = torch.cuda.Event(), torch.cuda.Event()
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device)
            self._forked.record(main)
            side.wait_event(self._forked)  # x is ready (and everything the step's stream did before)
            with torch.cuda.stream(side):
                a = self.left.mix(ctx, x, left_view)
                self._joined.record(side)
            b = self.right.mix(ctx, x, right_view)
            main.wait_event(self._joined)
        else:
            a = self.left.mix(ctx, x, left_view)
            b = self.right.mix(ctx, x, right_view)
        return a, b


register_mixer("side_by_side", SideBySide, replace=True)
