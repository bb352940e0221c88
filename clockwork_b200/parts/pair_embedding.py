"""An embedding part that adds, to every token's embedding row, a row of a second table chosen by a hash of the pair
(previous token, token).

Parameters: ``size`` (the rows' width), ``buckets``, ``mul_prev``, ``mul_cur``, ``name`` (the tensor's name), optionally
``vocab`` (token ids at or above it are reported and skipped).  The table has
``buckets + 1`` rows: token t reads row ``(token_(t-1) * mul_prev + token_t * mul_cur) mod buckets``, a request's first token
the last row.  The previous token is part of a request's state: the part asks the cache manager for one int32 per request
(``SlotStateNeed``), where the last token of a prompt portion (or a decoded token) stays for the step that follows; inside a
portion the previous token is the row before.  Position 0 never reads the state, so a request that starts over needs no reset.
"""

from __future__ import annotations

import torch

from .. import ops
from ..weights.decl import TensorDecl
from .base import Part, SlotStateNeed, StateView, StepContext
from .registry import register_embedding


class HashedPairEmbedding(Part):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.size, self.buckets = int(p["size"]), int(p["buckets"])
        self.mul_prev, self.mul_cur = int(p["mul_prev"]), int(p["mul_cur"])
        self.table_name = str(p["name"])
        self.vocab = int(p.get("vocab") or (1 << 30))
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("buckets must be positive and the multipliers non-negative")
        self.table: torch.Tensor | None = None

    def cache_need(self) -> SlotStateNeed:
        return SlotStateNeed((1,), torch.int32)

    def tensor_decls(self):
        yield TensorDecl(self.table_name, (self.buckets + 1, self.size), "table", "embedding")

    def load_weights(self, fetch) -> None:
        self.table = fetch(self.table_name)

    def add_to_embedding(self, ctx: StepContext, x: torch.Tensor, token_ids: torch.Tensor, view: StateView) -> None:
        ops.pair_embed_add(x, self.table, token_ids, ctx, view, self.mul_prev, self.mul_cur, self.vocab)


register_embedding("hashed_pair", HashedPairEmbedding, replace=True)
