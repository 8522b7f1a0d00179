"""Host-side bookkeeping of the paged cache: pools, block tables, state slots.

The reference keeps one contiguous, fully pre-allocated K/V tensor per request and
layer (app/runtime/kv_cache.py:31-38), writes at ``length`` and moves ``length`` only
on ``advance`` after all layers ran (kv_cache.py:53-72), and composes per-layer
caches of different kinds by layer index (app/runtime/mamba_cache.py:21-70). Here:

* keys and values live in fixed-size pages; every *group* of schedule entries with
  the same geometry and lifetime rule has a pool and, per request, a block table
  (logical page -> physical page) of its own;
* ``reserve`` gives a request pages for its next tokens before a step, ``commit``
  moves its length after the step (the reference's two-phase write);
* a group with a window W gives a page back as soon as its last position is
  ``<= length - W``: the next query sits at ``p >= length`` and needs ``j > p - W``,
  so no later query can see that page; its table entry becomes -1;
* a finished request gives everything back; freed pages are reused first (LIFO);
* beside the pages, every request holds one slot of fixed-size state
  (the analogue of the reference's conv/ssm state, mamba_cache.py:63-70), even
  when the architecture keeps nothing there.

Nothing here touches a device; storage.py owns the tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


class OutOfPages(RuntimeError):
    """A reservation that the pool cannot satisfy now. Nothing was taken."""


class CacheError(RuntimeError):
    """A use of the manager that breaks its rules (double free, unknown request...)."""


class PagePool:
    """Physical pages of one group: a LIFO free list plus an owner mark per page."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # pop() hands out page 0 first
        self._held = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self, count: int) -> list[int]:
        if count > len(self._free):
            raise OutOfPages(f"need {count} pages, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._held[page]:
                raise CacheError(f"page {page} was on the free list while held")
            self._held[page] = True
        return pages

    def release(self, pages: list[int]) -> None:
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise CacheError(f"page {page} is outside the pool")
            if not self._held[page]:
                raise CacheError(f"page {page} freed twice")
            self._held[page] = False
            self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]


class SlotPool:
    """Slots of fixed-size per-request state."""

    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_slots} state slots are in use")
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheError(f"state slot {slot} freed twice or never held")
        self._held[slot] = False
        self._free.append(slot)


@dataclass(frozen=True)
class GroupRule:
    """Lifetime rule of a group: ``window`` None keeps every page until the request ends."""

    window: int | None


@dataclass
class RequestRecord:
    request_id: str
    state_slot: int
    length: int = 0                     # committed tokens
    reserved: int = 0                   # tokens reserved beyond ``length``, not yet committed
    tables: list[list[int]] = field(default_factory=list)   # per group: logical -> physical / -1
    fresh_state: bool = True            # the state slot has not been zeroed for this request yet
    # the same tables as int32 arrays (-1 beyond the end), kept in step so that a step can copy a
    # whole row without converting a list
    table_arrays: list = field(default_factory=list)

    def mirror(self, group: int, first: int = 0) -> None:
        """Copies ``tables[group][first:]`` into the array mirror, growing it when needed."""
        table = self.tables[group]
        array = self.table_arrays[group]
        if len(table) > array.shape[0]:
            grown = np.full(max(2 * array.shape[0], len(table), 16), -1, dtype=np.int32)
            grown[:array.shape[0]] = array
            self.table_arrays[group] = array = grown
            first = min(first, len(table))
        if first < len(table):
            array[first:len(table)] = table[first:]
        array[len(table):] = -1


class CacheManager:
    def __init__(self, rules: list[GroupRule], pages_per_group: int | list[int], page_size: int,
                 num_state_slots: int) -> None:
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        counts = ([pages_per_group] * len(rules) if isinstance(pages_per_group, int)
                  else list(pages_per_group))
        if len(counts) != len(rules):
            raise ValueError("one page count per group is needed")
        self.rules = list(rules)
        self.page_size = page_size
        self.pools = [PagePool(count) for count in counts]
        self.slots = SlotPool(num_state_slots)
        self.requests: dict[str, RequestRecord] = {}
        self.pages_reused = 0            # allocations that handed out a page held before
        self._ever_held = [set() for _ in rules]

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: str) -> RequestRecord:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        record = RequestRecord(request_id=request_id, state_slot=self.slots.allocate(),
                               tables=[[] for _ in self.rules],
                               table_arrays=[np.full(16, -1, dtype=np.int32) for _ in self.rules])
        self.requests[request_id] = record
        return record

    def has_request(self, request_id: str) -> bool:
        return request_id in self.requests

    def record(self, request_id: str) -> RequestRecord:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def free_request(self, request_id: str) -> None:
        record = self.record(request_id)
        for group, table in enumerate(record.tables):
            self.pools[group].release([page for page in table if page >= 0])
        self.slots.release(record.state_slot)
        del self.requests[request_id]

    # ------------------------------------------------------------------ pages
    def _first_needed_logical(self, group: int, length: int) -> int:
        """First logical page a query at position >= length can still see."""
        window = self.rules[group].window
        if window is None:
            return 0
        return max(0, length - window + 1) // self.page_size

    def pages_needed(self, request_id: str, new_tokens: int) -> list[int]:
        """New pages per group that ``reserve(request_id, new_tokens)`` would take."""
        record = self.record(request_id)
        end = record.length + record.reserved + new_tokens
        last_logical = (end - 1) // self.page_size if end > 0 else -1
        return [max(0, last_logical + 1 - len(table)) for table in record.tables]

    def can_reserve(self, request_id: str, new_tokens: int) -> bool:
        needed = self.pages_needed(request_id, new_tokens)
        return all(n <= pool.free_count for n, pool in zip(needed, self.pools))

    def reserve(self, request_id: str, new_tokens: int) -> None:
        """Pages for positions [length + reserved, ... + new_tokens) in every group, or
        OutOfPages with nothing taken."""
        if new_tokens <= 0:
            raise CacheError("a reservation needs at least one token")
        record = self.record(request_id)
        needed = self.pages_needed(request_id, new_tokens)
        for group, count in enumerate(needed):
            if count > self.pools[group].free_count:
                raise OutOfPages(
                    f"request {request_id!r} needs {count} more pages in group {group}, "
                    f"{self.pools[group].free_count} free")
        for group, count in enumerate(needed):
            pages = self.pools[group].allocate(count)
            for page in pages:
                if page in self._ever_held[group]:
                    self.pages_reused += 1
                self._ever_held[group].add(page)
            if pages:
                first = len(record.tables[group])
                record.tables[group].extend(pages)
                record.mirror(group, first)
        record.reserved += new_tokens

    def commit(self, request_id: str, new_tokens: int) -> None:
        """The step that wrote ``new_tokens`` tokens is done: move the length and give back
        the pages no later query can see."""
        record = self.record(request_id)
        if new_tokens > record.reserved:
            raise CacheError(f"request {request_id!r} commits {new_tokens} tokens but reserved "
                             f"{record.reserved}")
        record.length += new_tokens
        record.reserved -= new_tokens
        record.fresh_state = False
        for group, table in enumerate(record.tables):
            keep_from = self._first_needed_logical(group, record.length)
            expired = []
            for logical in range(min(keep_from, len(table))):
                if table[logical] >= 0:
                    expired.append(table[logical])
                    table[logical] = -1
            if expired:
                self.pools[group].release(expired)
                record.mirror(group, 0)

    def cancel_reservation(self, request_id: str) -> None:
        """Drops an uncommitted reservation (a step that did not run)."""
        record = self.record(request_id)
        if record.reserved == 0:
            return
        keep = (record.length + self.page_size - 1) // self.page_size
        for group, table in enumerate(record.tables):
            extra = [page for page in table[keep:] if page >= 0]
            del table[keep:]
            self.pools[group].release(extra)
            record.mirror(group, min(keep, len(table)))
        record.reserved = 0

    def table_row(self, request_id: str, group: int, width: int) -> "np.ndarray":
        """The request's block table of ``group`` as int32[width], -1 where it holds no page."""
        record = self.record(request_id)
        array = record.table_arrays[group]
        if array.shape[0] < width:
            grown = np.full(width, -1, dtype=np.int32)
            grown[:array.shape[0]] = array
            record.table_arrays[group] = array = grown
        return array[:width]

    def slot_ids(self, request_id: str, group: int, start: int, count: int) -> "np.ndarray":
        """Physical slots (page * page_size + offset) of positions [start, start + count), int32."""
        record = self.record(request_id)
        positions = np.arange(start, start + count, dtype=np.int64)
        logical = positions // self.page_size
        if count > 0 and logical[-1] >= len(record.tables[group]):
            raise CacheError(f"position {start + count - 1} of {request_id!r} has no page in group {group}")
        pages = record.table_arrays[group][logical].astype(np.int64)
        if count > 0 and pages.min() < 0:
            bad = int(positions[np.argmax(pages < 0)])
            raise CacheError(f"position {bad} of {request_id!r} has no page in group {group}")
        return (pages * self.page_size + positions % self.page_size).astype(np.int32)

    # ------------------------------------------------------------------ inspection
    def free_pages(self) -> list[int]:
        return [pool.free_count for pool in self.pools]

    def held_pages(self, request_id: str, group: int) -> list[int]:
        return [page for page in self.record(request_id).tables[group] if page >= 0]

    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for group, pool in enumerate(self.pools):
            seen: dict[int, str] = {}
            for record in self.requests.values():
                for page in record.tables[group]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"group {group}: page {page} held by {seen[page]!r} and "
                                         f"{record.request_id!r}")
                    seen[page] = record.request_id
                    if not pool.is_held(page):
                        raise CacheError(f"group {group}: page {page} is in a table but marked free")
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise CacheError(f"group {group}: a page is on the free list twice")
            if free & seen.keys():
                raise CacheError(f"group {group}: pages both free and held: {sorted(free & seen.keys())}")
            if len(free) + len(seen) != pool.num_pages:
                raise CacheError(f"group {group}: {pool.num_pages - len(free) - len(seen)} pages lost")
            for record in self.requests.values():
                table = record.tables[group]
                array = record.table_arrays[group]
                if list(array[:len(table)]) != table or (array[len(table):] != -1).any():
                    raise CacheError(f"group {group}: the array mirror of {record.request_id!r} is stale")
        slots = [r.state_slot for r in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise CacheError("a state slot is held by two requests")
        if len(slots) + self.slots.free_count != self.slots.num_slots:
            raise CacheError("a state slot was lost")
