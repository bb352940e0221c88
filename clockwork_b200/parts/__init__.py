"""Parts: norms, position encodings, mixers, feed-forwards, blocks, and the model made of them.
Importing this package registers the built-in kinds."""

from . import (  # noqa: F401  (registration)
    attention, block, depth_block, feedforward, latent_attention, pair_embedding, parallel_block, rmsnorm, rotary, side_by_side,
    state_mixers, swiglu, window_attention,
)
from .base import (
    Block, FeedForward, Mixer, Norm, PagedKVNeed, PagedView, Part, PositionEncoding,
    ResidualStream, SlotStateNeed, StateView, StepContext,
)
from .linear import Linear
from .model import DecoderModel, build_model, tensor_decls_for_spec
from .registry import (
    build_block, build_part, register_block, register_embedding, register_ffn, register_mixer, register_norm,
    register_position, registered,
)

__all__ = [
    "Block", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "PagedView", "Part", "PositionEncoding",
    "ResidualStream", "SlotStateNeed", "StateView", "StepContext", "Linear", "DecoderModel",
    "build_model", "tensor_decls_for_spec", "build_block", "build_part", "register_block", "register_embedding",
    "register_ffn", "register_mixer", "register_norm", "register_position", "registered",
]
