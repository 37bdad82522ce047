from . import (  # noqa: F401 (register)
    attention, block, composite, delta_rule, embedding, feedforward, latent_attention, norm, position,
    recurrent, routed, sigmoid_attention, sink_attention, stream,
)
from .base import (
    Block,
    BuildEnv,
    CacheBinding,
    FeedForward,
    Mixer,
    Norm,
    PagedKVRequest,
    Part,
    PositionEncoding,
    StateRequest,
    WeightDecl,
)
from .registry import build_part, register_part, registered_kinds

__all__ = [
    "Block", "BuildEnv", "CacheBinding", "FeedForward", "Mixer", "Norm", "PagedKVRequest",
    "Part", "PositionEncoding", "StateRequest", "WeightDecl", "build_part", "register_part",
    "registered_kinds",
]
