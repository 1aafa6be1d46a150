"""The cache manager: paged keys/values with a block table per request, grouped by retention
rule, and slots for per-request state of fixed size.

* Every schedule entry whose mixer declares a :class:`PagedKVNeed` gets its own key and value
  tensors ``[pages, page_size, groups, head_dim]``.  Entries with the same retention rule (all
  keys, or a window of ``w``) form a *group*: one page pool and one block table per request serve
  the whole group, since such layers hold the same positions.  Groups have pages of their own.
* Pages are given back when a request ends, and, in a windowed group, as soon as the window has
  passed them; they are handed out again (last freed first) without being cleared.
* Every entry with a :class:`SlotStateNeed` gets a tensor ``[slots, *shape]``; a request holds
  one slot index for all of them, zeroed at admission by one kernel over a table of the state
  tensors (address, bytes per slot).
* ``poison_freed=True`` (for tests) overwrites pages and slots with NaN the moment they are given
  back, so that anything read from memory a request does not hold shows in the logits.

The reference has no counterpart: it holds one contiguous cache per sequence
(``lalamo/modules/token_mixers/kv_cache.py:225-330``) and never gives memory back.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from ..parts.base import CacheNeed, CacheView, PagedKVNeed, PagedKVView, Runtime, SlotStateNeed, SlotStateView
from .pages import OutOfPages, PagePool, SlotPool

__all__ = ["CacheLayout", "CacheManager", "RequestCache", "plan_cache_layout"]


@dataclass
class _Group:
    window: int | None
    entries: list[int]  # schedule entries whose pages this group holds
    pool: PagePool


@dataclass
class RequestCache:
    slot: int
    serial: int = 0  # unique per admission: tells a request from a later one that reuses its name
    length: int = 0  # tokens in the cache
    blocks: dict[int, list[int]] = field(default_factory=dict)  # group -> page per block, -1 = given back


@dataclass
class CacheLayout:
    """Which group and which tensors each schedule entry uses (host-only, testable without a GPU)."""

    entry_group: list[int | None]  # group index of the entry's paged cache (own or borrowed)
    entry_owner: list[int | None]  # the entry whose tensors it uses
    group_windows: list[int | None]
    group_entries: list[list[int]]
    slot_entries: list[int]


def plan_cache_layout(needs: list[CacheNeed | None], cache_from: list[int | None]) -> CacheLayout:
    windows: list[int | None] = []
    group_entries: list[list[int]] = []
    entry_group: list[int | None] = [None] * len(needs)
    entry_owner: list[int | None] = [None] * len(needs)
    slot_entries: list[int] = []
    for index, need in enumerate(needs):
        source = cache_from[index]
        if source is not None:
            if needs[source] is None or cache_from[source] is not None:
                raise ValueError(f"schedule entry {index} reads the cache of entry {source}, which owns none")
            entry_owner[index] = source
            entry_group[index] = entry_group[source]
            continue
        if isinstance(need, PagedKVNeed):
            if need.window not in windows:
                windows.append(need.window)
                group_entries.append([])
            group = windows.index(need.window)
            group_entries[group].append(index)
            entry_group[index] = group
            entry_owner[index] = index
        elif isinstance(need, SlotStateNeed):
            slot_entries.append(index)
            entry_owner[index] = index
        elif need is not None:
            raise ValueError(f"schedule entry {index}: unknown cache need {type(need).__name__}")
    return CacheLayout(entry_group, entry_owner, windows, group_entries, slot_entries)


class CacheManager:
    def __init__(
        self,
        needs: list[CacheNeed | None],
        cache_from: list[int | None],
        runtime: Runtime | None,
        *,
        page_size: int,
        num_pages: int,
        num_slots: int,
        poison_freed: bool = False,
    ) -> None:
        """``runtime=None`` makes a manager without device tensors (for host-side tests)."""
        if page_size < 1 or num_pages < 0 or num_slots < 1:
            raise ValueError("page_size and num_slots must be positive and num_pages non-negative")
        self.page_size = page_size
        self.num_pages = num_pages
        self.num_slots = num_slots
        self.runtime = runtime
        self.needs = needs
        self.layout = plan_cache_layout(needs, cache_from)
        self.groups = [
            _Group(window, entries, PagePool(num_pages, name=f"group {index} (window {window})"))
            for index, (window, entries) in enumerate(zip(self.layout.group_windows, self.layout.group_entries))
        ]
        self.slots = SlotPool(num_slots)
        self.requests: dict[object, RequestCache] = {}
        self.k_pages: dict[int, torch.Tensor] = {}
        self.v_pages: dict[int, torch.Tensor] = {}
        self.states: dict[int, torch.Tensor] = {}
        self.extra_states: dict[str, torch.Tensor] = {}
        self.poison_freed = poison_freed
        self._slot_table: torch.Tensor | None = None  # int64 [states, 2] on the device, built when first needed
        self._slot_bytes = 0
        self._admissions = 0
        if runtime is not None:
            for group in self.groups:
                for entry in group.entries:
                    need = needs[entry]
                    assert isinstance(need, PagedKVNeed)
                    # keys [page][row][group][channel]; values transposed, [page][group][channel][row]
                    self.k_pages[entry] = torch.zeros((num_pages, page_size, need.num_groups, need.head_dim), dtype=runtime.dtype, device=runtime.device)
                    self.v_pages[entry] = torch.zeros((num_pages, need.num_groups, need.head_dim, page_size), dtype=runtime.dtype, device=runtime.device)
            for entry in self.layout.slot_entries:
                need = needs[entry]
                assert isinstance(need, SlotStateNeed)
                self.states[entry] = torch.zeros((num_slots, *need.shape), dtype=need.dtype or runtime.dtype, device=runtime.device)

    # ------------------------------------------------------------------ slot states
    def add_slot_state(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A further per-request state ``[slots, *shape]`` (for instance a sampler's token counts),
        zeroed at admission like the mixers' states."""
        if name not in self.extra_states:
            assert self.runtime is not None
            self.extra_states[name] = torch.zeros((self.num_slots, *shape), dtype=dtype, device=self.runtime.device)
            self._slot_table = None
        return self.extra_states[name]

    _POISON = 0x7FC07FC0  # NaN as one float32 and as two bfloat16; a huge count as int32

    def _fill_slot(self, slot: int, pattern: int) -> None:
        """One launch writes ``pattern`` over the slot in every state tensor."""
        if self.runtime is None:
            return
        if self._slot_table is None:
            states = [state for state in list(self.states.values()) + list(self.extra_states.values()) if state[0].numel()]
            records = [[state.data_ptr(), state[0].numel() * state.element_size()] for state in states]
            self._slot_bytes = max((record[1] for record in records), default=0)
            self._slot_table = torch.tensor(records, dtype=torch.int64).reshape(-1, 2).to(self.runtime.device)
        if self._slot_table.shape[0]:
            ops.fill_slots(self._slot_table, self._slot_bytes, slot, pattern)

    def _poison_pages(self, group_index: int, pages: list[int]) -> None:
        if not self.poison_freed or self.runtime is None or not pages:
            return
        index = torch.tensor(pages, dtype=torch.long, device=self.runtime.device)
        for entry in self.groups[group_index].entries:
            self.k_pages[entry][index] = float("nan")
            self.v_pages[entry][index] = float("nan")

    # --------------------------------------------------------------------- requests
    def admit(self, request_id: object) -> RequestCache:
        """Gives the request a state slot (zeroed) and empty block tables."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.slots.allocate()
        self._fill_slot(slot, 0)
        self._admissions += 1
        record = RequestCache(slot=slot, serial=self._admissions, blocks={index: [] for index in range(len(self.groups))})
        self.requests[request_id] = record
        return record

    def pages_needed(self, request_id: object, new_length: int) -> int:
        """Pages (in the fullest group) that :meth:`reserve` would take."""
        record = self.requests[request_id]
        blocks = -(-new_length // self.page_size)
        return max((max(0, blocks - len(record.blocks[g])) for g in range(len(self.groups))), default=0)

    def blocks_held(self, request_id: object) -> int:
        """Blocks (of page_size positions, from position 0) the request's block tables cover."""
        record = self.requests[request_id]
        return min((len(blocks) for blocks in record.blocks.values()), default=0)

    def free_pages(self) -> int:
        """Pages free in the fullest group."""
        return min((group.pool.free_count for group in self.groups), default=self.num_pages)

    def reserve(self, request_id: object, new_length: int) -> None:
        """Makes sure pages exist for positions ``< new_length`` in every group; all or nothing."""
        record = self.requests[request_id]
        blocks = -(-new_length // self.page_size)
        wanted = [max(0, blocks - len(record.blocks[g])) for g in range(len(self.groups))]
        for group, count in zip(self.groups, wanted):
            if count > group.pool.free_count:
                raise OutOfPages(count, group.pool.free_count, group.pool.name)
        for index, (group, count) in enumerate(zip(self.groups, wanted)):
            record.blocks[index].extend(group.pool.allocate(count))

    def commit(self, request_id: object, new_length: int) -> None:
        """Records that the cache now holds ``new_length`` tokens and gives back the pages that
        every later query's window has passed (keys ``j <= new_length - window``)."""
        record = self.requests[request_id]
        if new_length < record.length:
            raise ValueError("a request's cache cannot shrink")
        record.length = new_length
        for index, group in enumerate(self.groups):
            if group.window is None:
                continue
            first_needed = new_length - group.window + 1  # lowest key a query at position >= new_length sees
            dead_blocks = max(0, first_needed) // self.page_size
            blocks = record.blocks[index]
            released = [blocks[b] for b in range(min(dead_blocks, len(blocks))) if blocks[b] >= 0]
            for b in range(min(dead_blocks, len(blocks))):
                blocks[b] = -1
            group.pool.release(released)
            self._poison_pages(index, released)

    def release(self, request_id: object) -> None:
        """Ends the request: all its pages and its slot go back to the pools."""
        record = self.requests.pop(request_id)
        for index, group in enumerate(self.groups):
            pages = [page for page in record.blocks[index] if page >= 0]
            group.pool.release(pages)
            self._poison_pages(index, pages)
        self.slots.release(record.slot)
        if self.poison_freed:
            self._fill_slot(record.slot, self._POISON)

    def length(self, request_id: object) -> int:
        return self.requests[request_id].length

    def check(self) -> None:
        """Invariants: every page is free or held by exactly one request; likewise slots."""
        for index, group in enumerate(self.groups):
            group.pool.check()
            held: set[int] = set()
            for request_id, record in self.requests.items():
                for page in record.blocks[index]:
                    if page < 0:
                        continue
                    if page in held:
                        raise AssertionError(f"page {page} of group {index} is held twice")
                    if not group.pool.is_held(page):
                        raise AssertionError(f"page {page} of group {index} is used by {request_id!r} but free")
                    held.add(page)
            if len(held) != group.pool.held_count:
                raise AssertionError(f"group {index}: {group.pool.held_count - len(held)} pages are lost")
        self.slots.check()
        slots = [record.slot for record in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slots.held_count:
            raise AssertionError("state slots are shared or lost")

    # ------------------------------------------------------------------------ steps
    def block_table_rows(self, request_ids: list[object], width: int | None = None) -> list[list[list[int]]]:
        """Per group, one row of page indices per request (``-1`` padded to a common width)."""
        tables: list[list[list[int]]] = []
        for index in range(len(self.groups)):
            rows = [self.requests[request_id].blocks[index] for request_id in request_ids]
            columns = max(1, width or 0, max((len(row) for row in rows), default=0))
            tables.append([row + [-1] * (columns - len(row)) for row in rows])
        return tables

    def views(self, block_tables: list[torch.Tensor], segment_slot: torch.Tensor) -> list[CacheView | None]:
        """The cache of every schedule entry for one step (``block_tables``: one device tensor per group)."""
        result: list[CacheView | None] = []
        for entry, owner in enumerate(self.layout.entry_owner):
            if owner is None:
                result.append(None)
                continue
            owns = owner == entry
            group = self.layout.entry_group[entry]
            if group is not None:
                result.append(PagedKVView(owns, self.k_pages[owner], self.v_pages[owner], block_tables[group]))
            else:
                result.append(SlotStateView(owns, self.states[owner], segment_slot))
        return result

    def bytes_held(self, request_id: object) -> int:
        """Bytes of cache a step reads for this request (keys, values and states)."""
        record = self.requests[request_id]
        total = 0
        for index, group in enumerate(self.groups):
            live = record.length if group.window is None else min(record.length, group.window)
            for entry in group.entries:
                pages = self.k_pages[entry]
                total += 2 * live * pages.shape[2] * pages.shape[3] * pages.element_size()
        for state in self.states.values():
            total += state[0].numel() * state.element_size()
        return total
