"""Part specifications: the data from which a model is put together.

A model is described by a :class:`ModelPlan`: a tuple of :class:`BlockSpec` (each naming
its norm, mixer and feed-forward by a spec object) plus a *schedule*, the list that says
in which order blocks run.  Every size and constant lives in a spec; no part reads the
architecture's ``config.json`` and no part knows which model it is in.

The reference keeps the same information in a tree of ``*Config`` dataclasses
(``lalamo/modules/transformer_layer.py:164-207``, ``lalamo/modules/transformer.py:31-41``,
``lalamo/modules/decoder.py:158-207``).  Here the tree is flat, and the order of execution
is data as well.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar

__all__ = [
    "AttentionSpec",
    "BlockSpec",
    "EmbeddingSpec",
    "HeadSpec",
    "FeedForwardSpec",
    "GatedMLPSpec",
    "MixerSpec",
    "ModelPlan",
    "NormSpec",
    "PositionSpec",
    "RMSNormSpec",
    "RopeSpec",
    "ScheduleEntry",
    "ShortConvSpec",
]


@dataclass(frozen=True)
class NormSpec:
    """Base of all normalisation specs.  ``kind`` selects the part class."""

    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class RMSNormSpec(NormSpec):
    """Root-mean-square norm: ``x * rsqrt(mean(x^2) + eps) * (w + scale_offset)``.

    Mirrors ``NormalizationConfig`` with ``subtract_mean=False``
    (``lalamo/modules/normalization.py:49-76``).
    """

    kind: ClassVar[str] = "rms_norm"
    dim: int = 0
    eps: float = 1e-5
    scale_offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class RopeSpec(PositionSpec):
    """Unscaled rotary embedding over the first ``rotary_dim`` channels of a head,
    rotate-half (NeoX) pairing (``lalamo/modules/rope.py:58-102``)."""

    kind: ClassVar[str] = "rope"
    rotary_dim: int = 0
    theta: float = 10000.0


@dataclass(frozen=True)
class MixerSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query causal attention with optional per-head q/k norm, position encoding
    and sliding window (``lalamo/modules/token_mixers/attention.py:332-447``)."""

    kind: ClassVar[str] = "attention"
    model_dim: int = 0
    num_heads: int = 0
    num_groups: int = 0
    head_dim: int = 0
    qk_norm: NormSpec | None = None
    position: PositionSpec | None = None
    window: int | None = None
    scale: float | None = None  # None -> head_dim ** -0.5


@dataclass(frozen=True)
class ShortConvSpec(MixerSpec):
    """Gated depthwise causal convolution of ``kernel_size`` taps
    (``lalamo/modules/token_mixers/short_conv.py:51-157``)."""

    kind: ClassVar[str] = "short_conv"
    model_dim: int = 0
    kernel_size: int = 0
    has_bias: bool = False


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """``down(up(x) * act(gate(x)))`` (``lalamo/modules/mlp.py:233-262``)."""

    kind: ClassVar[str] = "gated_mlp"
    model_dim: int = 0
    hidden_dim: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class BlockSpec:
    """Pre-norm residual block: ``h = x + mixer(norm1(x)); y = h + ffn(norm2(h))``
    (``lalamo/modules/transformer_layer.py:220-377``)."""

    pre_mixer_norm: NormSpec
    mixer: MixerSpec
    pre_ffn_norm: NormSpec
    ffn: FeedForwardSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: a row of the table per token id, times ``scale``, into the residual stream
    (``lalamo/modules/embedding.py``)."""

    kind: ClassVar[str] = "token_embedding"
    vocab_size: int = 0
    model_dim: int = 0
    scale: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """The read-out: logits ``x @ W.T`` in 32-bit, with ``W`` the embedding table when ``tied``."""

    kind: ClassVar[str] = "lm_head"
    vocab_size: int = 0
    model_dim: int = 0
    tied: bool = True


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a block.

    ``layer`` indexes ``ModelPlan.layers`` (a layer may appear in several entries).
    ``cache_from`` names an earlier schedule entry whose cache this execution reads
    instead of owning one (the reference's ``kv_source_layer_index``,
    ``lalamo/modules/transformer.py:210-217``).
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelPlan:
    vocab_size: int
    model_dim: int
    layers: tuple[BlockSpec, ...]
    final_norm: NormSpec
    tie_embeddings: bool = True
    embedding_scale: float | None = None
    schedule: tuple[ScheduleEntry, ...] = field(default=())
    # The parts at the model's two ends.  Left ``None`` they are the plain token embedding and the
    # plain (tied or untied) read-out made from the fields above; an architecture with, say, scaled or
    # capped logits gives a specification of its own, for which a part is registered.
    embedding: EmbeddingSpec | None = None
    head: HeadSpec | None = None

    def __post_init__(self) -> None:
        if self.embedding is None:
            object.__setattr__(self, "embedding", EmbeddingSpec(self.vocab_size, self.model_dim, self.embedding_scale or 1.0))
        if self.head is None:
            object.__setattr__(self, "head", HeadSpec(self.vocab_size, self.model_dim, self.tie_embeddings))
        if not self.schedule:
            object.__setattr__(
                self, "schedule", tuple(ScheduleEntry(i) for i in range(len(self.layers)))
            )
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{position}] names layer {entry.layer}, but there are {len(self.layers)}")
            if entry.cache_from is not None and not 0 <= entry.cache_from < position:
                raise ValueError(
                    f"schedule[{position}].cache_from={entry.cache_from} must name an earlier schedule entry"
                )
