"""The parts models are put together from.  Importing this package registers the built-in parts."""

from . import attention, embedding, feed_forward, norm, rope, short_conv  # noqa: F401  (registration)
from .base import (
    CacheNeed,
    CacheView,
    FeedForward,
    HostSegments,
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
from .embedding import Embedding, Head
from .block import Block, PreNormBlock, block_tensor_decls, build_block, register_arrangement
from .model import DecoderModel, plan_tensor_decls

__all__ = [
    "Block",
    "CacheNeed",
    "CacheView",
    "DecoderModel",
    "Embedding",
    "FeedForward",
    "Head",
    "HostSegments",
    "Mixer",
    "Norm",
    "PagedKVNeed",
    "PagedKVView",
    "Part",
    "PositionEncoding",
    "PreNormBlock",
    "Runtime",
    "SlotStateNeed",
    "SlotStateView",
    "StepInputs",
    "TensorDecl",
    "block_tensor_decls",
    "build_block",
    "build_part",
    "part_type",
    "plan_tensor_decls",
    "register_arrangement",
    "register_part",
]
