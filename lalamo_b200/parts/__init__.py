"""The parts models are put together from.  Importing this package registers the built-in parts."""

from . import attention, feed_forward, norm, rope, short_conv  # noqa: F401  (registration)
from .base import (
    CacheNeed,
    CacheView,
    FeedForward,
    Mixer,
    Norm,
    PagedKVNeed,
    PagedKVView,
    Part,
    PositionEncoding,
    Runtime,
    SlotStateNeed,
    SlotStateView,
    StepInputs,
    TensorDecl,
    build_part,
    part_type,
    register_part,
)
from .block import Block, block_tensor_decls
from .model import DecoderModel, plan_tensor_decls

__all__ = [
    "Block",
    "CacheNeed",
    "CacheView",
    "DecoderModel",
    "FeedForward",
    "Mixer",
    "Norm",
    "PagedKVNeed",
    "PagedKVView",
    "Part",
    "PositionEncoding",
    "Runtime",
    "SlotStateNeed",
    "SlotStateView",
    "StepInputs",
    "TensorDecl",
    "block_tensor_decls",
    "build_part",
    "part_type",
    "plan_tensor_decls",
    "register_part",
]
