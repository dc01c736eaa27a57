"""The cache: a slot per sequence, keys and values per layer run, each sequence with its own length.

Runs of the schedule whose mixers need the same thing (kv heads, key and value head sizes, retention:
all keys or a window of them) form a group; every group has storage, a page pool and a page table of
its own.  Storage of a group is two tensors, keys [runs, pages, kv_heads, page_size, key size] and
values [runs, pages, kv_heads, page_size, value size]; a sequence holds whole pages of `page_size`
positions, and `block_table[i]` names the page with positions [i*page_size, (i+1)*page_size).  A
window group gives pages back as soon as no later query can see them, and when the engine states
the longest step it will be given, such a group is made with only the pages its window can hold.
Page 0 of every group is never handed out: padding rows of a fixed-size decode batch point at it.

integrallis/models' model for groups with different needs is LayeredKvCache, with a LayerSpec
(keyDim, valueDim, LINEAR | RING, ringCapacity) per layer
(backend-java/.../cache/LayeredKvCache.java:35-64); its per-sequence length is Session.nextPosition
(backend-java/.../llama/LlamaForwardPass.java:50-68) and rewinding is discardFrom
(backend-java/.../cache/KvCache.java:161-173).

Everything in this file is host bookkeeping and runs without a GPU; the storage tensors are made
by the caller-provided `allocate` function.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .pages import CacheFull, FreeList

PAGE_SIZE = 64


@dataclass(frozen=True)
class KvRequest:
    """What one attention-like mixer needs of the cache.  window None: every earlier position
    stays; n: only the n positions that end at the newest query.  `head_dim` is the size of a key
    head; a value head has `value_dim` (None: the same), as the reference's LayerSpec keeps keyDim and
    valueDim apart (backend-java/.../cache/LayeredKvCache.java:35-64)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None

    @property
    def value_head_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


class CacheGroup:
    def __init__(self, request: KvRequest, runs: Sequence[int], num_pages: int, page_size: int):
        self.request = request
        self.runs = list(runs)  # schedule indices that own storage here, in storage order
        self.page_size = page_size
        self.num_pages = num_pages  # usable pages; storage has one more (page 0, padding)
        self.pages = FreeList(num_pages, first=1, what="cache page")
        self.tables: Dict[int, List[int]] = {}  # slot -> page per block, -1 where given back
        self.keys = None    # [runs, num_pages + 1, kv_heads, page_size, key head size]
        self.values = None  # [runs, num_pages + 1, kv_heads, page_size, value head size]

    def run_index(self, run: int) -> int:
        return self.runs.index(run)

    def pages_needed(self, slot: int, new_length: int) -> int:
        have = len(self.tables[slot])
        return max(0, -(-new_length // self.page_size) - have)

    def extend(self, slot: int, new_length: int) -> int:
        """Takes the pages `new_length` positions need beyond those held; returns how many it took."""
        table = self.tables[slot]
        need = self.pages_needed(slot, new_length)
        for _ in range(need):
            table.append(self.pages.take())
        return need

    def drop_invisible(self, slot: int, length: int) -> int:
        """After `length` positions are stored, a window group frees the pages no later query sees:
        the next query sits at position >= length and sees keys >= length - window + 1.  Returns how
        many pages it gave back."""
        window = self.request.window
        if window is None:
            return 0
        first_visible = length - window + 1
        table = self.tables[slot]
        dropped = 0
        for block in range(len(table)):
            if (block + 1) * self.page_size <= first_visible:
                if table[block] >= 0:
                    self.pages.give_back(table[block])
                    table[block] = -1
                    dropped += 1
            else:
                break
        return dropped

    def truncate(self, slot: int, length: int) -> None:
        table = self.tables[slot]
        keep = -(-length // self.page_size)
        while len(table) > keep:
            page = table.pop()
            if page >= 0:
                self.pages.give_back(page)

    def release(self, slot: int) -> None:
        for page in self.tables.pop(slot):
            if page >= 0:
                self.pages.give_back(page)


class KvCache:
    """Slots, lengths and page tables of all groups.

    `requests[i]` is what run i of the schedule asks for (None: that run keeps no keys and values);
    `cache_from[i]` names the earlier run whose storage run i reads instead of owning some.
    `max_tokens` is the most positions that live sequences hold at any time, each sequence's count
    rounded up to whole pages; a group that keeps every position gets that many.  A window group
    needs, per sequence, the pages that hold its window and the tokens of the step in flight (a step's
    keys are all stored before any page is given back): with `max_step_tokens` (the most tokens a step
    brings to one sequence; the caller must then refuse longer steps) it gets
    max_slots x (pages of window - 1 + max_step_tokens, and one more for the page boundary), if that is
    less; without it, as many as the other groups.
    """

    def __init__(self, requests: Sequence[Optional[KvRequest]], cache_from: Sequence[Optional[int]], max_tokens: int,
                 max_slots: Optional[int] = None, page_size: int = PAGE_SIZE, max_step_tokens: Optional[int] = None):
        if page_size <= 0 or page_size % 32:
            raise ValueError(f"page_size must be a positive multiple of 32, got {page_size}")
        if max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {max_tokens}")
        self.page_size = page_size
        self.num_pages = -(-max_tokens // page_size)
        self.max_slots = max_slots if max_slots is not None else self.num_pages
        if self.max_slots <= 0:
            raise ValueError(f"max_slots must be positive, got {self.max_slots}")
        self.slots = FreeList(self.max_slots, what="slot")
        self.lengths: Dict[int, int] = {}
        # A stamp per open slot that changes whenever a page table of the slot does, and that no slot ever
        # carries twice: whoever keeps a copy of a slot's page tables (a captured step does) compares stamps
        # to know whether the copy still holds.  A slot id alone does not say so: it is handed out again.
        self.table_stamps: Dict[int, int] = {}
        self._last_stamp = 0
        self.groups: List[CacheGroup] = []
        self.run_location: Dict[int, Tuple[int, int]] = {}  # run -> (group index, index in the group's storage)
        by_key: Dict[KvRequest, CacheGroup] = {}
        for run, request in enumerate(requests):
            if request is None or cache_from[run] is not None:
                continue
            group = by_key.get(request)
            if group is None:
                group = CacheGroup(request, [], self.pages_for(request, max_step_tokens), page_size)
                by_key[request] = group
                self.groups.append(group)
            group.runs.append(run)
            self.run_location[run] = (self.groups.index(group), len(group.runs) - 1)
        for run, source in enumerate(cache_from):
            if source is None or requests[run] is None:
                continue
            if source not in self.run_location:
                raise ValueError(f"run {run} reads the cache of run {source}, which stores none")
            owner = self.groups[self.run_location[source][0]].request
            mine = requests[run]
            if ((owner.num_kv_heads, owner.head_dim, owner.value_head_dim) !=
                    (mine.num_kv_heads, mine.head_dim, mine.value_head_dim)):
                raise ValueError(
                    f"run {run} reads the cache of run {source} but asks for {mine.num_kv_heads} kv heads of "
                    f"{mine.head_dim} (values {mine.value_head_dim}), the owner stores {owner.num_kv_heads} of "
                    f"{owner.head_dim} (values {owner.value_head_dim})")
            self.run_location[run] = self.run_location[source]

    # ---------------------------------------------------------------- storage

    def pages_for(self, request: KvRequest, max_step_tokens: Optional[int]) -> int:
        """Usable pages of the group of `request`."""
        if request.window is None or max_step_tokens is None:
            return self.num_pages
        if max_step_tokens <= 0:
            raise ValueError(f"max_step_tokens must be positive, got {max_step_tokens}")
        # positions a sequence holds at most while a step is in flight, wherever they start in a page
        per_slot = -(-(request.window - 1 + max_step_tokens) // self.page_size) + 1
        return min(self.num_pages, self.max_slots * per_slot)

    def allocate_storage(self, allocate: Callable[[Tuple[int, ...]], object]) -> int:
        """Creates each group's keys and values with `allocate(shape)`; returns the number of elements."""
        total = 0
        for group in self.groups:
            r = group.request
            for name, width in (("keys", r.head_dim), ("values", r.value_head_dim)):
                shape = (len(group.runs), group.num_pages + 1, r.num_kv_heads, self.page_size, width)
                setattr(group, name, allocate(shape))
                n = 1
                for s in shape:
                    n *= s
                total += n
        return total

    def pools(self, run: int):
        """(group index, keys pool, values pool) of a run: [pages, kv_heads, page_size, key or value head size]."""
        g, i = self.run_location[run]
        group = self.groups[g]
        return g, group.keys[i], group.values[i]

    # ---------------------------------------------------------------- slots

    def _stamp(self, slot: int) -> None:
        self._last_stamp += 1
        self.table_stamps[slot] = self._last_stamp

    def open_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for group in self.groups:
            group.tables[slot] = []
        self._stamp(slot)
        return slot

    def release(self, slot: int) -> None:
        self._require(slot)
        for group in self.groups:
            group.release(slot)
        del self.lengths[slot]
        del self.table_stamps[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        self._require(slot)
        return self.lengths[slot]

    def live_slots(self) -> List[int]:
        return sorted(self.lengths)

    def _require(self, slot: int) -> None:
        if slot not in self.lengths:
            raise KeyError(f"slot {slot} is not open")

    # ---------------------------------------------------------------- growth

    def can_append(self, appends: Sequence[Tuple[int, int]]) -> bool:
        try:
            self._check_append(appends)
            return True
        except CacheFull:
            return False

    def _check_append(self, appends: Sequence[Tuple[int, int]]) -> None:
        for group in self.groups:
            need = sum(group.pages_needed(slot, self.lengths[slot] + n) for slot, n in appends)
            if need > group.pages.free:
                raise CacheFull(
                    f"the step needs {need} more cache pages of {self.page_size} positions, {group.pages.free} are free "
                    f"(the cache was sized for {self.num_pages * self.page_size} positions"
                    + (f"; this group keeps a window of {group.request.window} and has {group.num_pages} pages)"
                       if group.num_pages != self.num_pages else ")"))

    def append(self, appends: Sequence[Tuple[int, int]]) -> None:
        """Makes room for n more positions in each (slot, n).  Checks everything first: on CacheFull
        nothing has changed.  Lengths move in `commit`."""
        seen = set()
        for slot, n in appends:
            self._require(slot)
            if slot in seen:
                raise ValueError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n <= 0:
                raise ValueError(f"slot {slot}: a step must bring at least one token, got {n}")
        self._check_append(appends)
        for slot, n in appends:
            if sum(group.extend(slot, self.lengths[slot] + n) for group in self.groups):
                self._stamp(slot)

    def commit(self, appends: Sequence[Tuple[int, int]]) -> None:
        for slot, n in appends:
            self.lengths[slot] += n
            if sum(group.drop_invisible(slot, self.lengths[slot]) for group in self.groups):
                self._stamp(slot)

    def rewind(self, slot: int, length: int) -> None:
        """Forgets the positions >= length.  A window group that already gave back pages the shorter
        sequence would need cannot rewind that far."""
        self._require(slot)
        if not 0 <= length <= self.lengths[slot]:
            raise ValueError(f"slot {slot}: cannot rewind to {length}, it holds {self.lengths[slot]} positions")
        for group in self.groups:
            window = group.request.window
            if window is not None:
                first_needed = max(0, length - window + 1) // self.page_size
                table = group.tables[slot]
                if any(table[b] < 0 for b in range(first_needed, min(len(table), -(-length // self.page_size)))):
                    raise ValueError(f"slot {slot}: a window group no longer holds the positions a rewind to {length} needs")
        for group in self.groups:
            group.truncate(slot, length)
        self.lengths[slot] = length
        self._stamp(slot)

    # ---------------------------------------------------------------- checks

    def check(self) -> None:
        """Bookkeeping invariants: no slot or page lost, held twice, or shared by two sequences."""
        self.slots.check()
        if set(self.lengths) != self.slots._held:
            raise AssertionError("open slots and held slots differ")
        for group in self.groups:
            group.pages.check()
            seen = set()
            for slot, table in group.tables.items():
                if slot not in self.lengths:
                    raise AssertionError(f"a page table exists for closed slot {slot}")
                for page in table:
                    if page < 0:
                        continue
                    if page in seen:
                        raise AssertionError(f"page {page} is in two page tables")
                    if not group.pages.is_held(page):
                        raise AssertionError(f"page {page} is in a page table but not held")
                    seen.add(page)
            if len(seen) != group.pages.held:
                raise AssertionError(f"{group.pages.held - len(seen)} held pages are in no page table")
