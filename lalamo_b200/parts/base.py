"""Interfaces of the parts a model is put together from, and the registry that maps a
specification class to the part class that runs it.

A part is built from ``(spec, tensors, runtime)`` and knows nothing else: not the model it is
in, not its layer index, not the architecture's tensor names.  The four families:

* :class:`Norm`           ``forward(x)`` and ``residual_forward(residual, delta)``
* :class:`PositionEncoding`  owns the tables a mixer needs to encode positions
* :class:`Mixer`          ``forward(x, step, cache)``; declares what cache it needs
* :class:`FeedForward`    ``forward(x, step)``

The reference's counterparts are ``TokenMixerBase`` (``lalamo/modules/token_mixer.py:120-145``),
``MLPBase`` (``lalamo/modules/mlp.py``), ``Normalization`` and ``RoPE``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar, Mapping

import numpy as np
import torch

from .. import ops

__all__ = [
    "REPLAY_MAX_TOKENS",
    "CacheNeed",
    "CacheView",
    "FeedForward",
    "HostSegments",
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
    "build_part",
    "part_type",
    "register_part",
]


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs.

    ``role``: ``"matrix"`` (stored and used in the compute type), ``"vector"`` (kept in 32-bit:
    norm scales, convolution taps, biases) or ``"table"`` (integers, int32).
    ``init`` tells the random-weights mode how to fill it: ``"normal"``, ``"ones"`` (one plus
    noise, for scales) or ``"zeros"``.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass
class Runtime:
    """What every part is given at build time: where and in which type it computes."""

    device: torch.device
    dtype: torch.dtype  # activation / matrix type: torch.bfloat16 or torch.float32
    status: torch.Tensor = field(default=None)  # type: ignore[assignment]  # int32[1], first kernel error

    def __post_init__(self) -> None:
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {self.dtype}")
        if self.status is None:
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def matrix(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape: int, dtype: torch.dtype | None = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


# ------------------------------------------------------------------------------- caches
@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache manager."""


@dataclass(frozen=True)
class PagedKVNeed(CacheNeed):
    """Keys and values of every past token (``window=None``) or of the last ``window`` tokens."""

    num_groups: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class SlotStateNeed(CacheNeed):
    """Per-request state of fixed size: one ``shape`` tensor per live request, zero at admission.
    ``dtype=None`` means the activation type."""

    shape: tuple[int, ...]
    dtype: torch.dtype | None = None


@dataclass
class CacheView:
    """A schedule entry's cache as its mixer sees it during one step."""

    owns: bool  # False when the entry reads another entry's cache and must not write it


@dataclass
class PagedKVView(CacheView):
    k_pages: torch.Tensor  # [pages, page_size, groups, head_dim]
    v_pages: torch.Tensor  # [pages, groups, head_dim, page_size] (transposed)
    block_table: torch.Tensor  # int32 [segments, max_blocks], -1 where no page is held


@dataclass
class SlotStateView(CacheView):
    state: torch.Tensor  # [slots, *shape]
    segment_slot: torch.Tensor  # int32 [segments]


@dataclass(frozen=True)
class HostSegments:
    """One step's portions as the host knows them, for parts that plan their work on the host
    (:meth:`Part.plan_step`): portion ``s`` covers rows ``start[s] : start[s] + length[s]`` of the
    step and its request holds ``context[s]`` tokens in the cache already."""

    start: tuple[int, ...]
    length: tuple[int, ...]
    context: tuple[int, ...]

    @property
    def tokens(self) -> int:
        return sum(self.length)


# Steps of more tokens than this are never replayed from a recording (the step function's rule): what a part
# decides for them may depend on the requests' contexts, what it decides for shorter steps may not.
REPLAY_MAX_TOKENS = 512


@dataclass
class StepInputs:
    """The device-side description of one step's ragged batch.

    ``segments`` request portions are laid out one after the other in ``tokens`` rows; portion
    ``s`` covers rows ``segment_start[s] : segment_start[s] + segment_length[s]`` and its first
    token has absolute position ``segment_context[s]`` (the number of tokens of that request
    already in the cache).
    """

    tokens: int
    segments: int
    token_ids: torch.Tensor  # int32 [tokens]
    positions: torch.Tensor  # int32 [tokens]
    token_segment: torch.Tensor  # int32 [tokens]
    segment_start: torch.Tensor  # int32 [segments]
    segment_length: torch.Tensor  # int32 [segments]
    segment_context: torch.Tensor  # int32 [segments]
    segment_slot: torch.Tensor  # int32 [segments]
    want_rows: torch.Tensor  # int32 [wanted]
    wanted: int
    max_segment_length: int
    max_context: int  # largest position + 1 over the batch
    host_segment_start: tuple[int, ...] = ()
    host_segment_length: tuple[int, ...] = ()
    host_segment_context: tuple[int, ...] = ()
    # What the parts planned for this step on the host (Part.plan_step), by plan key: the arrays on
    # the device (int32, uploaded with the rest of the description) and as the host made them.
    plans: dict[object, dict[str, torch.Tensor]] = field(default_factory=dict)
    host_plans: dict[object, dict[str, np.ndarray]] = field(default_factory=dict)

    def plan_of(self, part: "Part") -> tuple[dict[str, torch.Tensor], dict[str, np.ndarray]]:
        """The arrays ``part.plan_step`` made for this step: ``(on the device, on the host)``."""
        key = part.step_plan_key()
        if key not in self.plans:
            raise KeyError(f"this step carries no plan of {type(part).__name__}: the batch builder was not given it as a planner")
        return self.plans[key], self.host_plans[key]


# -------------------------------------------------------------------------------- parts
class Part:
    """Base of all parts."""

    spec_type: ClassVar[type]

    def __init__(self, spec: Any, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime

    @classmethod
    def tensor_decls(cls, spec: Any) -> dict[str, TensorDecl]:
        """The tensors this part needs, by local name."""
        return {}

    # ---- work a part plans on the host, step by step (tile lists, routing tables, chunk lists ...)
    # True if plan_step's arrays depend on the portions' contexts; if they depend on starts and
    # lengths only, a recorded step's copy of them is written once and never again.
    step_plan_uses_context: ClassVar[bool] = True

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray] | None:
        """Integer arrays this part's kernels need for the step, made on the host from the step's
        portions; ``None`` (the default) if it needs none.  The batch builder packs them into the
        step's one upload and hands them back through :meth:`StepInputs.plan_of`.  For a step that
        is replayed from a recording the arrays are made again and must keep their sizes while the
        portions' lengths stay the same."""
        return None

    def step_plan_key(self) -> object:
        """Parts whose plans are the same for every step (for instance all attention layers with one
        tiling) return the same key, and the plan is made and uploaded once."""
        return id(self)


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> torch.Tensor:
        """Normalises the rows of ``x`` (all, or those listed in ``rows``); activation type out."""
        raise NotImplementedError

    def residual_forward(
        self,
        residual: torch.Tensor,
        delta: torch.Tensor | None,
        rows: torch.Tensor | None = None,
        num_rows: int | None = None,
    ) -> torch.Tensor:
        """``residual += delta`` on the 32-bit residual stream, then the norm of the sum."""
        if delta is not None:
            ops.residual_add(residual, delta)
        return self.forward(residual, rows, num_rows)


class PositionEncoding(Part):
    pass


class Mixer(Part):
    # True if forward() only launches work on the current stream (no host synchronisation, no
    # host-side reads of device data): such a mixer's steps may be recorded in a CUDA graph.
    graph_safe = False

    def cache_need(self) -> CacheNeed | None:
        return None

    # True if forward() accepts ``residual=``: it may then add its output to the 32-bit residual
    # stream itself (in the epilogue of its last product) and return ``None`` instead of the output.
    can_accumulate = False

    def forward(self, x: torch.Tensor, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        raise NotImplementedError


class FeedForward(Part):
    can_accumulate = False  # as for Mixer

    def forward(self, x: torch.Tensor, step: StepInputs) -> torch.Tensor | None:
        raise NotImplementedError


_PART_TYPES: dict[type, type[Part]] = {}


def register_part(spec_type: type) -> Callable[[type[Part]], type[Part]]:
    """Class decorator: ``spec_type`` instances are run by the decorated part class."""

    def decorate(part_class: type[Part]) -> type[Part]:
        part_class.spec_type = spec_type
        _PART_TYPES[spec_type] = part_class
        return part_class

    return decorate


def part_type(spec: Any) -> type[Part]:
    for candidate in type(spec).__mro__:
        if candidate in _PART_TYPES:
            return _PART_TYPES[candidate]
    raise KeyError(f"no part is registered for specifications of type {type(spec).__name__}")


def build_part(spec: Any, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> Part:
    return part_type(spec)(spec, tensors, runtime)
