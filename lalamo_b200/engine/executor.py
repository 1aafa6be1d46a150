"""The step function: runs one ragged batch of request portions through the model.

A step is a list of :class:`StepEntry` (a request, its next tokens, and the places among them
whose logits are wanted).  Portions of prompts and single decoded tokens may stand side by side,
cut anywhere.  The step runs only the tokens it is given, from the cache that earlier steps
left, and returns 32-bit logits ``[wanted, vocab]`` in the order of the entries and of ``want``.

The reference's counterpart is ``Decoder.__call__`` on a rectangular padded batch that is either
all prefill or all decode (``lalamo/modules/decoder.py:220-317``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..parts.base import REPLAY_MAX_TOKENS, HostSegments, Part, Runtime, StepInputs
from ..parts.model import DecoderModel

__all__ = ["BatchBuilder", "BuiltStep", "Executor", "StepEntry", "StepError"]


class StepError(ValueError):
    """A step was malformed (unknown request, token outside the vocabulary, bad ``want``)."""


@dataclass
class StepEntry:
    """``token_source >= 0``: the portion's last token has not been to the host; it is row
    ``token_source`` of the token ids the step before sampled on the device (``previous_sampled`` of
    :meth:`Executor.step`), and the value given in ``tokens`` for that place is ignored."""

    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    token_source: int = -1


class _Staging:
    """Pinned host buffers, used in turn, each guarded by an event of its last copy."""

    def __init__(self, device: torch.device, depth: int = 2) -> None:
        self.device = device
        self.buffers: list[torch.Tensor | None] = [None] * depth
        self.events: list[torch.cuda.Event | None] = [None] * depth
        self.turn = 0

    def upload(self, values: np.ndarray, target: torch.Tensor | None = None) -> torch.Tensor:
        index = self.turn
        self.turn = (self.turn + 1) % len(self.buffers)
        event = self.events[index]
        if event is not None:
            event.synchronize()
        buffer = self.buffers[index]
        if buffer is None or buffer.numel() < values.size:
            capacity = max(4096, 1 << int(values.size - 1).bit_length())
            buffer = torch.empty(capacity, dtype=torch.int32, pin_memory=True)
            self.buffers[index] = buffer
        buffer[: values.size].numpy()[:] = values
        if target is None:
            on_device = torch.empty(values.size, dtype=torch.int32, device=self.device)
        else:
            if target.numel() != values.size:
                raise ValueError(f"the batch description has {values.size} words, the fixed buffer {target.numel()}")
            on_device = target
        on_device.copy_(buffer[: values.size], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[index] = event
        return on_device


@dataclass
class BuiltStep:
    """A step's description on the device, with what is needed to write it again in place."""

    inputs: StepInputs
    block_tables: list[torch.Tensor]  # one per cache group
    layout: dict[object, tuple[int, int]]  # section name -> (offset, size) in 32-bit words of the upload
    packed: np.ndarray  # the upload as the host made it
    buffer: torch.Tensor  # the upload on the device; every tensor of `inputs` and `block_tables` is a view of it


class BatchBuilder:
    """Turns a list of entries into the device-side description of the batch: reserves the pages
    the new tokens need and uploads token ids, positions, segment tables, the parts' own work lists
    (:meth:`~lalamo_b200.parts.base.Part.plan_step`) and block tables in one copy from pinned memory."""

    def __init__(self, cache: CacheManager, device: torch.device, vocab_size: int, planners: Sequence[Part] = ()) -> None:
        self.cache = cache
        self.vocab_size = vocab_size
        self._staging = _Staging(device)
        self.last_h2d_bytes = 0
        self.planners: dict[object, Part] = {}
        for part in planners:
            if type(part).plan_step is not Part.plan_step:
                self.planners.setdefault(part.step_plan_key(), part)

    def validate(self, entries: Sequence[StepEntry]) -> None:
        seen: set[object] = set()
        for entry in entries:
            if entry.request_id not in self.cache.requests:
                raise StepError(f"request {entry.request_id!r} is not live (admit it first)")
            if entry.request_id in seen:
                raise StepError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if len(entry.tokens) == 0:
                raise StepError(f"request {entry.request_id!r} brings no tokens")
            if len(entry.tokens) > 8:
                ids = np.asarray(entry.tokens, dtype=np.int64)
                bad = ids[(ids < 0) | (ids >= self.vocab_size)]
                if bad.size:
                    raise StepError(f"request {entry.request_id!r}: token {int(bad[0])} is outside the vocabulary of {self.vocab_size}")
            else:
                for token in entry.tokens:
                    if not 0 <= int(token) < self.vocab_size:
                        raise StepError(f"request {entry.request_id!r}: token {token} is outside the vocabulary of {self.vocab_size}")
            if entry.token_source < -1:
                raise StepError(f"request {entry.request_id!r}: token_source={entry.token_source}")
            for place in entry.want:
                if not 0 <= int(place) < len(entry.tokens):
                    raise StepError(f"request {entry.request_id!r}: want={place} is outside its {len(entry.tokens)} tokens")

    def pages_needed(self, entries: Sequence[StepEntry]) -> int:
        return sum(self.cache.pages_needed(e.request_id, self.cache.length(e.request_id) + len(e.tokens)) for e in entries)

    def plan_parts(self, segments: HostSegments, only_context_dependent: bool = False) -> dict[object, dict[str, np.ndarray]]:
        """What every planner makes of these portions: ``plan key -> {name: int32 array}``."""
        plans: dict[object, dict[str, np.ndarray]] = {}
        for key, part in self.planners.items():
            if only_context_dependent and not part.step_plan_uses_context:
                continue
            arrays = part.plan_step(segments) or {}
            plans[key] = {name: np.ascontiguousarray(array, dtype=np.int32).reshape(-1) for name, array in arrays.items()}
        return plans

    def build(
        self,
        entries: Sequence[StepEntry],
        table_width: int | None = None,
        target: torch.Tensor | None = None,
        max_context: int | None = None,
    ) -> BuiltStep:
        """Reserves pages and builds the device-side description of the batch (one block table per
        cache group).  ``table_width`` fixes the block tables' width, ``target`` is a device buffer
        to fill instead of a fresh one, ``max_context`` overrides the batch's longest context with a
        larger bound: together they make the description's addresses and shapes repeatable, which a
        recorded CUDA graph needs."""
        cache = self.cache
        if self.pages_needed(entries) > cache.free_pages():
            raise OutOfPages(self.pages_needed(entries), cache.free_pages())
        for entry in entries:
            cache.reserve(entry.request_id, cache.length(entry.request_id) + len(entry.tokens))

        lengths = [len(entry.tokens) for entry in entries]
        contexts = [cache.length(entry.request_id) for entry in entries]
        starts = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32) if entries else np.zeros(0, np.int32)
        tokens = int(sum(lengths))
        segments = len(entries)
        token_ids = np.concatenate([np.asarray(entry.tokens, dtype=np.int32) for entry in entries]) if entries else np.zeros(0, np.int32)
        token_segment = np.repeat(np.arange(segments, dtype=np.int32), lengths)
        positions = np.concatenate([np.arange(c, c + n, dtype=np.int32) for c, n in zip(contexts, lengths)]) if entries else np.zeros(0, np.int32)
        want_rows = np.asarray([start + int(place) for entry, start in zip(entries, starts) for place in entry.want], dtype=np.int32)
        slots = np.asarray([cache.requests[entry.request_id].slot for entry in entries], dtype=np.int32)
        sources = np.asarray([entry.token_source for entry in entries], dtype=np.int32)
        tables = cache.block_table_rows([entry.request_id for entry in entries], table_width)
        table_arrays = [np.asarray(rows, dtype=np.int32).reshape(segments, -1) for rows in tables]
        host_segments = HostSegments(tuple(int(s) for s in starts), tuple(lengths), tuple(contexts))
        host_plans = self.plan_parts(host_segments)

        sections: list[tuple[object, np.ndarray]] = [
            ("token_ids", token_ids), ("positions", positions), ("token_segment", token_segment), ("segment_start", starts),
            ("segment_length", np.asarray(lengths, np.int32)), ("segment_context", np.asarray(contexts, np.int32)),
            ("segment_slot", slots), ("want_rows", want_rows), ("token_source", sources),
        ]
        for key, arrays in host_plans.items():
            sections += [(("plan", key, name), array) for name, array in arrays.items()]
        sections += [(("block_table", group), table.reshape(-1)) for group, table in enumerate(table_arrays)]
        packed = np.concatenate([array for _, array in sections])
        if packed.size == 0:
            packed = np.zeros(1, np.int32)
        if target is not None and target.numel() != packed.size:
            target = None  # the caller sees from the layout that its buffer does not fit
        device_buffer = self._staging.upload(packed, target)
        self.last_h2d_bytes = packed.size * 4

        layout: dict[object, tuple[int, int]] = {}
        views: dict[object, torch.Tensor] = {}
        offset = 0
        for name, array in sections:
            layout[name] = (offset, array.size)
            views[name] = device_buffer[offset : offset + array.size]
            offset += array.size
        block_tables = [views[("block_table", group)].view(segments, -1) for group in range(len(table_arrays))]
        step = StepInputs(
            tokens=tokens,
            segments=segments,
            token_ids=views["token_ids"],
            positions=views["positions"],
            token_segment=views["token_segment"],
            segment_start=views["segment_start"],
            segment_length=views["segment_length"],
            segment_context=views["segment_context"],
            segment_slot=views["segment_slot"],
            want_rows=views["want_rows"],
            wanted=int(want_rows.size),
            max_segment_length=max(lengths, default=0),
            max_context=max_context or max((c + n for c, n in zip(contexts, lengths)), default=0),
            host_segment_start=host_segments.start,
            host_segment_length=host_segments.length,
            host_segment_context=host_segments.context,
            plans={key: {name: views[("plan", key, name)] for name in arrays} for key, arrays in host_plans.items()},
            host_plans=host_plans,
        )
        return BuiltStep(step, block_tables, layout, packed, device_buffer)


@dataclass
class _RecordedStep:
    """A step recorded as a CUDA graph, with the fixed buffers it reads and writes."""

    graph: torch.cuda.CUDAGraph | None
    buffer: torch.Tensor
    logits: torch.Tensor | None = None
    uses: int = 0
    launches: int = 0  # kernels of this library in the recording
    layout: dict[object, tuple[int, int]] | None = None
    # The recorded buffer's image in pinned host memory, kept between steps: only what changed is rewritten.
    host: torch.Tensor | None = None
    host_view: np.ndarray | None = None
    copied: torch.cuda.Event | None = None
    requests: tuple = ()
    blocks_written: list | None = None  # per group, per row: block-table entries already in the image


class Executor:
    """Runs steps.  With ``use_graphs`` on, steps of at most ``GRAPH_MAX_TOKENS`` tokens are replayed
    from CUDA graphs: a step's *shape* is the lengths of its portions, the places wanted in each, and
    the block tables' width (a multiple of ``TABLE_WIDTH_STEP`` pages, which also bounds the
    contexts).  The first step of a shape runs kernel by kernel; a shape that comes again is recorded,
    and from then on such steps write their description into the recorded buffers and replay.  Decode
    steps (one token per request, its logits wanted) are recorded at their first occurrence and only
    rewrite what changed in their description.  A recorded graph's logits buffer is reused by the
    next replay of the same shape."""

    TABLE_WIDTH_STEP = 64  # block-table columns come in multiples of this when graphs are used
    MAX_GRAPHS = 48
    GRAPH_MAX_TOKENS = REPLAY_MAX_TOKENS  # longer steps are bound by their kernels, not by their launches

    def __init__(self, model: DecoderModel, cache: CacheManager, runtime: Runtime, use_graphs: bool = False) -> None:
        self.model = model
        self.cache = cache
        self.runtime = runtime
        self.vocab_size = model.plan.vocab_size
        self.builder = BatchBuilder(cache, runtime.device, self.vocab_size, model.step_planners())
        self.steps_run = 0
        self.tokens_run = 0
        self.graph_replays = 0
        self.graph_rebinds = 0  # replays whose recorded rows were rewritten for other requests
        self.use_graphs = use_graphs and all(getattr(block.mixer, "graph_safe", False) for block in model.blocks)
        self._graphs: dict[tuple, _RecordedStep] = {}
        self._seen_shapes: dict[tuple, int] = {}

    @property
    def last_h2d_bytes(self) -> int:
        return self.builder.last_h2d_bytes

    # ----------------------------------------------------------------------- graphs
    def _graph_key(self, entries: Sequence[StepEntry]) -> tuple | None:
        if not self.use_graphs or not entries:
            return None
        lengths = tuple(len(entry.tokens) for entry in entries)
        if sum(lengths) > self.GRAPH_MAX_TOKENS:
            return None
        page = self.cache.page_size
        longest = max(self.cache.length(entry.request_id) + len(entry.tokens) for entry in entries)
        width = -(-(-(-longest // page)) // self.TABLE_WIDTH_STEP) * self.TABLE_WIDTH_STEP
        if all(length == 1 and len(entry.want) == 1 for length, entry in zip(lengths, entries)):
            return "decode", len(entries), width
        return lengths, tuple(tuple(int(place) for place in entry.want) for entry in entries), width

    def _record(self, recorded: _RecordedStep, built: BuiltStep) -> None:
        views = self.cache.views(built.block_tables, built.inputs.segment_slot)
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            recorded.logits = self.model.forward(built.inputs, views)
        recorded.launches = ops.launch_count() - before
        ops.add_launches(-recorded.launches)  # recording launched nothing
        recorded.graph = graph
        recorded.layout = built.layout

    def _feed(self, buffer: torch.Tensor, layout: dict, entries: Sequence[StepEntry], previous_sampled: torch.Tensor | None) -> None:
        """Fills in, on the device, the token ids that entries take from the step before (after the
        description's upload and before anything reads it, all on one stream)."""
        if not any(entry.token_source >= 0 for entry in entries):
            return
        if previous_sampled is None:
            raise StepError("an entry takes its last token from the step before, but no sampled ids were given")

        def section(name: str) -> torch.Tensor:
            offset, size = layout[name]
            return buffer[offset : offset + size]

        ops.feed_tokens(section("token_ids"), section("segment_start"), section("segment_length"), section("token_source"), previous_sampled, self.runtime.status)

    def _step_with_graph(self, entries: Sequence[StepEntry], key: tuple, previous_sampled: torch.Tensor | None = None) -> torch.Tensor | None:
        """Runs the step from its shape's recording, making the recording if it is due; ``None``
        if this shape is not (yet) worth recording."""
        width = key[-1]
        is_decode = key[0] == "decode"
        recorded = self._graphs.get(key)
        if recorded is None:
            self._seen_shapes[key] = self._seen_shapes.get(key, 0) + 1
            if not is_decode and self._seen_shapes[key] < 2:
                if len(self._seen_shapes) > 4096:
                    self._seen_shapes.clear()
                return None
            if len(self._graphs) >= self.MAX_GRAPHS:
                del self._graphs[min(self._graphs, key=lambda k: self._graphs[k].uses)]
            recorded = _RecordedStep(None, torch.empty(0, dtype=torch.int32, device=self.runtime.device))
            self._graphs[key] = recorded
        recorded.uses += 1
        context_bound = width * self.cache.page_size
        if recorded.graph is None:
            # Run it for real, then record the same launches, reading the same buffer, for later steps.
            built = self.builder.build(entries, table_width=width, max_context=context_bound)
            recorded.buffer = built.buffer
            self._feed(built.buffer, built.layout, entries, previous_sampled)
            views = self.cache.views(built.block_tables, built.inputs.segment_slot)
            logits = self.model.forward(built.inputs, views)
            self._record(recorded, built)
            recorded.requests = tuple(self.cache.requests[entry.request_id].serial for entry in entries)
            if is_decode:
                self._start_image(recorded, built, entries)
            return logits
        if is_decode:
            self._refresh_decode_inputs(recorded, entries)
        else:
            built = self.builder.build(entries, table_width=width, target=recorded.buffer, max_context=context_bound)
            if built.layout != recorded.layout:
                # a part's work lists changed size although the portions did not: this shape cannot be replayed
                del self._graphs[key]
                self._seen_shapes[key] = -(1 << 30)
                self._feed(built.buffer, built.layout, entries, previous_sampled)
                views = self.cache.views(built.block_tables, built.inputs.segment_slot)
                return self.model.forward(built.inputs, views)
        assert recorded.layout is not None
        self._feed(recorded.buffer, recorded.layout, entries, previous_sampled)
        recorded.graph.replay()
        ops.add_launches(recorded.launches)
        self.graph_replays += 1
        assert recorded.logits is not None
        return recorded.logits

    def _start_image(self, recorded: _RecordedStep, built: BuiltStep, entries: Sequence[StepEntry]) -> None:
        """A decode recording keeps its description's image in pinned memory; later steps rewrite
        only what changes from step to step."""
        recorded.host = torch.zeros(recorded.buffer.numel(), dtype=torch.int32, pin_memory=True)
        recorded.host_view = recorded.host.numpy()
        recorded.host_view[:] = built.packed
        groups = len(self.cache.groups)
        recorded.blocks_written = [
            [len(self.cache.requests[entry.request_id].blocks[group]) for entry in entries] for group in range(groups)
        ]

    def _refresh_decode_inputs(self, recorded: _RecordedStep, entries: Sequence[StepEntry]) -> None:
        """Brings a recorded decode step's description up to date for these entries.  What depends on
        the portions' lengths only (and those are all one) stays as recorded; token ids, positions,
        contexts, slots and the work lists of parts that look at contexts are rewritten; block-table
        rows only grow while the same requests stay in the same places."""
        cache = self.cache
        layout = recorded.layout
        image = recorded.host_view
        assert layout is not None and image is not None
        if recorded.copied is not None:
            recorded.copied.synchronize()  # the last copy out of the image is done
        batch = len(entries)
        groups = len(cache.groups)
        table_views = []
        for group in range(groups):
            offset, size = layout[("block_table", group)]
            table_views.append(image[offset : offset + size].reshape(batch, -1))
        requests = tuple(cache.requests[entry.request_id].serial for entry in entries)
        if requests != recorded.requests or recorded.blocks_written is None:
            self.graph_rebinds += 1
            for table in table_views:
                table[:] = -1
            recorded.requests = requests
            recorded.blocks_written = [[0] * batch for _ in range(groups)]
        token_ids = image[layout["token_ids"][0] :]
        positions = image[layout["positions"][0] :]
        contexts = image[layout["segment_context"][0] :]
        slots = image[layout["segment_slot"][0] :]
        sources = image[layout["token_source"][0] :]
        lengths = []
        for row, entry in enumerate(entries):
            record = cache.requests[entry.request_id]
            length = record.length
            lengths.append(length)
            cache.reserve(entry.request_id, length + 1)
            token_ids[row] = entry.tokens[0]
            positions[row] = length
            contexts[row] = length
            slots[row] = record.slot
            sources[row] = entry.token_source
            for group_index, group in enumerate(cache.groups):
                blocks = record.blocks[group_index]
                if group.window is not None:
                    table_views[group_index][row, : len(blocks)] = blocks  # pages drop out at the front as the window moves
                else:
                    written = recorded.blocks_written[group_index][row]
                    if len(blocks) > written:
                        table_views[group_index][row, written : len(blocks)] = blocks[written:]
                        recorded.blocks_written[group_index][row] = len(blocks)
        if self.builder.planners:
            segments = HostSegments(tuple(range(batch)), (1,) * batch, tuple(lengths))
            for key, arrays in self.builder.plan_parts(segments, only_context_dependent=True).items():
                for name, array in arrays.items():
                    offset, size = layout[("plan", key, name)]
                    if array.size != size:
                        raise RuntimeError(f"{type(self.builder.planners[key]).__name__}.plan_step changed the size of {name!r} between steps of one shape")
                    image[offset : offset + size] = array
        recorded.buffer.copy_(recorded.host, non_blocking=True)
        if recorded.copied is None:
            recorded.copied = torch.cuda.Event()
        recorded.copied.record()
        self.builder.last_h2d_bytes = recorded.buffer.numel() * 4

    # -------------------------------------------------------------------------- run
    def step(self, entries: Sequence[StepEntry], previous_sampled: torch.Tensor | None = None) -> torch.Tensor:
        """Runs the batch; returns float32 logits ``[wanted, vocab]`` on the device.  ``previous_sampled``:
        int32 token ids on the device (the step before's sampled tokens) for entries with a ``token_source``."""
        self.builder.validate(entries)
        if not entries:
            return self.runtime.empty(0, self.vocab_size, dtype=torch.float32)
        key = self._graph_key(entries)
        logits = self._step_with_graph(entries, key, previous_sampled) if key is not None else None
        if logits is None:
            built = self.builder.build(entries)
            self._feed(built.buffer, built.layout, entries, previous_sampled)
            views = self.cache.views(built.block_tables, built.inputs.segment_slot)
            logits = self.model.forward(built.inputs, views)
        tokens = sum(len(entry.tokens) for entry in entries)
        for entry in entries:
            self.cache.commit(entry.request_id, self.cache.length(entry.request_id) + len(entry.tokens))
        self.steps_run += 1
        self.tokens_run += tokens
        return logits

    def check_status(self) -> None:
        """Raises if a kernel reported an error (synchronises the device)."""
        code = int(self.runtime.status.item())
        if code != 0:
            names = {1: "a block-table entry outside the pool", 2: "a state slot outside the slot array",
                     3: "a token id outside the vocabulary", 4: "a bounded wait gave up"}
            self.runtime.status.zero_()
            raise RuntimeError(f"a kernel reported: {names.get(code, code)}")
