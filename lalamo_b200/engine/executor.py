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
from ..parts.base import ATTENTION_ALONE_LIMIT, ATTENTION_TILE, Runtime, StepInputs
from ..parts.model import DecoderModel

__all__ = ["BatchBuilder", "Executor", "StepEntry", "StepError"]


class StepError(ValueError):
    """A step was malformed (unknown request, token outside the vocabulary, bad ``want``)."""


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


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


class BatchBuilder:
    """Turns a list of entries into the device-side description of the batch: reserves the pages
    the new tokens need and uploads token ids, positions, segment tables and block tables in one
    copy from pinned memory."""

    def __init__(self, cache: CacheManager, device: torch.device, vocab_size: int) -> None:
        self.cache = cache
        self.vocab_size = vocab_size
        self._staging = _Staging(device)
        self.last_h2d_bytes = 0

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
            for token in entry.tokens:
                if not 0 <= int(token) < self.vocab_size:
                    raise StepError(f"request {entry.request_id!r}: token {token} is outside the vocabulary of {self.vocab_size}")
            for place in entry.want:
                if not 0 <= int(place) < len(entry.tokens):
                    raise StepError(f"request {entry.request_id!r}: want={place} is outside its {len(entry.tokens)} tokens")

    def pages_needed(self, entries: Sequence[StepEntry]) -> int:
        return sum(self.cache.pages_needed(e.request_id, self.cache.length(e.request_id) + len(e.tokens)) for e in entries)

    def build(
        self,
        entries: Sequence[StepEntry],
        table_width: int | None = None,
        target: torch.Tensor | None = None,
        max_context: int | None = None,
    ) -> tuple[StepInputs, list[torch.Tensor]]:
        """Reserves pages and builds the device-side description of the batch (one block table per
        cache group).  ``table_width`` fixes the block tables' width, ``target`` is a device buffer
        to fill instead of a fresh one, ``max_context`` overrides the batch's longest context with a
        larger bound: together they make the description's addresses and shapes repeatable, which a
        captured CUDA graph needs."""
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
        tables = cache.block_table_rows([entry.request_id for entry in entries], table_width)
        table_arrays = [np.asarray(rows, dtype=np.int32).reshape(segments, -1) for rows in tables]

        alone, tiles = [], []
        for start, length in zip(starts.tolist(), lengths):
            if length <= ATTENTION_ALONE_LIMIT:
                alone.extend(range(start, start + length))
            else:
                tiles.extend((first, min(ATTENTION_TILE, start + length - first)) for first in range(start, start + length, ATTENTION_TILE))
        alone_tokens = np.asarray(alone, dtype=np.int32)
        tile_records = np.asarray(tiles, dtype=np.int32).reshape(-1)
        sections = [token_ids, positions, token_segment, starts, np.asarray(lengths, np.int32), np.asarray(contexts, np.int32), slots, want_rows,
                    alone_tokens, tile_records]
        sections += [table.reshape(-1) for table in table_arrays]
        packed = np.concatenate(sections) if sections else np.zeros(0, np.int32)
        if packed.size == 0:
            packed = np.zeros(1, np.int32)
        device_buffer = self._staging.upload(packed, target)
        self.last_h2d_bytes = packed.size * 4

        views: list[torch.Tensor] = []
        offset = 0
        for section in sections:
            views.append(device_buffer[offset : offset + section.size])
            offset += section.size
        block_tables = [view.view(segments, -1) for view in views[10:]]
        step = StepInputs(
            tokens=tokens,
            segments=segments,
            token_ids=views[0],
            positions=views[1],
            token_segment=views[2],
            segment_start=views[3],
            segment_length=views[4],
            segment_context=views[5],
            segment_slot=views[6],
            want_rows=views[7],
            wanted=int(want_rows.size),
            max_segment_length=max(lengths, default=0),
            max_context=max_context or max((c + n for c, n in zip(contexts, lengths)), default=0),
            host_segment_start=tuple(int(s) for s in starts),
            host_segment_length=tuple(lengths),
            host_segment_context=tuple(contexts),
            alone_tokens=views[8],
            num_alone=int(alone_tokens.size),
            tiles=views[9],
            num_tiles=int(tile_records.size // 2),
        )
        return step, block_tables

@dataclass
class _CapturedStep:
    """A decode step recorded as a CUDA graph, with the fixed buffers it reads and writes."""

    graph: torch.cuda.CUDAGraph | None
    buffer: torch.Tensor
    logits: torch.Tensor | None = None
    uses: int = 0
    launches: int = 0  # kernels of this library in the recording
    # The recorded buffer's image in pinned host memory, kept between steps: only what changed is rewritten.
    host: torch.Tensor | None = None
    host_view: np.ndarray | None = None
    copied: torch.cuda.Event | None = None
    requests: tuple = ()
    blocks_written: list | None = None  # per group, per row: block-table entries already in the image


class Executor:
    """Runs steps.  Steps in which every request brings exactly one token and wants its logits
    (decoding) are replayed from CUDA graphs when ``use_graphs`` is on: the first step of a given
    shape (batch size, block-table width, context bound) runs kernel by kernel and is then recorded;
    later steps of that shape copy their description into the recorded buffers and replay.  A
    recorded graph's logits buffer is reused by the next replay of the same shape."""

    TABLE_WIDTH_STEP = 64  # block-table columns come in multiples of this when graphs are used
    MAX_GRAPHS = 24

    def __init__(self, model: DecoderModel, cache: CacheManager, runtime: Runtime, use_graphs: bool = False) -> None:
        self.model = model
        self.cache = cache
        self.runtime = runtime
        self.vocab_size = model.plan.vocab_size
        self.builder = BatchBuilder(cache, runtime.device, self.vocab_size)
        self.steps_run = 0
        self.tokens_run = 0
        self.graph_replays = 0
        self.graph_rebinds = 0  # replays whose recorded rows were rewritten for other requests
        self.use_graphs = use_graphs and all(getattr(block.mixer, "graph_safe", False) for block in model.blocks)
        self._graphs: dict[tuple[int, int], _CapturedStep] = {}

    @property
    def last_h2d_bytes(self) -> int:
        return self.builder.last_h2d_bytes

    # ----------------------------------------------------------------------- graphs
    def _graph_key(self, entries: Sequence[StepEntry]) -> tuple[int, int] | None:
        if not self.use_graphs or not entries:
            return None
        if any(len(entry.tokens) != 1 or list(entry.want) != [0] for entry in entries):
            return None
        page = self.cache.page_size
        longest = max(self.cache.length(entry.request_id) for entry in entries) + 1
        width = -(-(-(-longest // page)) // self.TABLE_WIDTH_STEP) * self.TABLE_WIDTH_STEP
        return len(entries), width

    def _step_with_graph(self, entries: Sequence[StepEntry], key: tuple[int, int]) -> torch.Tensor:
        batch, width = key
        context_bound = width * self.cache.page_size
        groups = len(self.cache.groups)
        captured = self._graphs.get(key)
        if captured is None:
            if len(self._graphs) >= self.MAX_GRAPHS:
                del self._graphs[min(self._graphs, key=lambda k: self._graphs[k].uses)]
            words = 9 * batch + groups * batch * width
            captured = _CapturedStep(None, torch.zeros(words, dtype=torch.int32, device=self.runtime.device))
            self._graphs[key] = captured
        captured.uses += 1
        if captured.graph is not None:
            self._refresh_recorded_inputs(captured, entries, batch, width)
            captured.graph.replay()
            ops.add_launches(captured.launches)
            self.graph_replays += 1
            assert captured.logits is not None
            return captured.logits
        step, block_tables = self.builder.build(entries, table_width=width, target=captured.buffer, max_context=context_bound)
        # First step of this shape: run it for real, then record the same launches for later steps.
        views = self.cache.views(block_tables, step.segment_slot)
        logits = self.model.forward(step, views)
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            captured.logits = self.model.forward(step, views)
        captured.launches = ops.launch_count() - before
        ops.add_launches(-captured.launches)  # recording launched nothing
        captured.graph = graph
        return logits

    def _refresh_recorded_inputs(self, captured: _CapturedStep, entries: Sequence[StepEntry], batch: int, width: int) -> None:
        """Brings a recorded step's input buffer up to date for these entries: the layout is
        :meth:`BatchBuilder.build`'s for ``batch`` one-token portions, the constant parts are written
        once, and block-table rows only grow while the same requests stay in the same places."""
        cache = self.cache
        groups = len(cache.groups)
        if captured.host is None:
            captured.host = torch.zeros(captured.buffer.numel(), dtype=torch.int32, pin_memory=True)
            image = captured.host.numpy()
            count = np.arange(batch, dtype=np.int32)
            image[2 * batch : 3 * batch] = count  # token_segment
            image[3 * batch : 4 * batch] = count  # segment_start
            image[4 * batch : 5 * batch] = 1  # segment_length
            image[7 * batch : 8 * batch] = count  # want_rows
            image[8 * batch : 9 * batch] = count  # alone_tokens
            image[9 * batch :] = -1  # block tables
            captured.host_view = image
        elif captured.copied is not None:
            captured.copied.synchronize()  # the last copy out of the image is done
        image = captured.host_view
        assert image is not None
        requests = tuple(cache.requests[entry.request_id].serial for entry in entries)
        if requests != captured.requests or captured.blocks_written is None:
            if captured.blocks_written is not None:
                self.graph_rebinds += 1
            image[9 * batch :] = -1
            captured.requests = requests
            captured.blocks_written = [[0] * batch for _ in range(groups)]
        tables = image[9 * batch :].reshape(groups, batch, width)
        for row, entry in enumerate(entries):
            record = cache.requests[entry.request_id]
            length = record.length
            cache.reserve(entry.request_id, length + 1)
            image[row] = entry.tokens[0]
            image[batch + row] = length
            image[5 * batch + row] = length
            image[6 * batch + row] = record.slot
            for group_index, group in enumerate(cache.groups):
                blocks = record.blocks[group_index]
                if group.window is not None:
                    tables[group_index, row, : len(blocks)] = blocks  # pages drop out at the front as the window moves
                else:
                    written = captured.blocks_written[group_index][row]
                    if len(blocks) > written:
                        tables[group_index, row, written : len(blocks)] = blocks[written:]
                        captured.blocks_written[group_index][row] = len(blocks)
        captured.buffer.copy_(captured.host, non_blocking=True)
        if captured.copied is None:
            captured.copied = torch.cuda.Event()
        captured.copied.record()
        self.builder.last_h2d_bytes = captured.buffer.numel() * 4

    # -------------------------------------------------------------------------- run
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the batch; returns float32 logits ``[wanted, vocab]`` on the device."""
        self.builder.validate(entries)
        if not entries:
            return self.runtime.empty(0, self.vocab_size, dtype=torch.float32)
        key = self._graph_key(entries)
        if key is not None:
            logits = self._step_with_graph(entries, key)
            tokens = len(entries)
        else:
            step, block_tables = self.builder.build(entries)
            views = self.cache.views(block_tables, step.segment_slot)
            logits = self.model.forward(step, views)
            tokens = step.tokens
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
