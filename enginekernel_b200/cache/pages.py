"""Host-side bookkeeping of the cache: sequence slots, pages, lengths.

The reference keeps one dense ``[batch, kv_heads, max_len, head_dim]`` tensor per layer,
a batch row standing for a sequence, and regrows it when a larger shape arrives
(engine/engine.py:226-263).  Here storage is cut into pages of ``PAGE`` tokens that a
sequence collects as it grows, so the cache is sized by the number of tokens it has to
hold, whatever their split into sequences, and never regrows.  A *slot* is a sequence's
handle: it owns the sequence's length and one page list per layer group.  Everything in
this module is plain Python and is tested without a GPU.
"""

from __future__ import annotations

from typing import Dict, List, Optional

PAGE = 64


class CacheError(RuntimeError):
    """No free slot or page, a length over the limit, or a slot misused."""


class FreeList:
    """Hands out the integers 0..n-1; refuses to take one back twice."""

    def __init__(self, n: int, what: str):
        self.n, self.what = n, what
        self._free = list(range(n - 1, -1, -1))      # pop() gives 0 first
        self._held = [False] * n

    def available(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.n} are in use)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held[i] = False
        self._free.append(i)

    def held(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]


class PageGroup:
    """The pages of one layer group and which slot holds which.

    ``window``: the group's layers read only the last ``window`` keys, so pages that lie
    wholly before the window of every later token are handed back as a sequence grows.
    """

    def __init__(self, num_pages: int, num_slots: int, max_pages_per_slot: int,
                 window: Optional[int] = None):
        self.pool = FreeList(num_pages, "cache page")
        self.window = window
        self.max_pages_per_slot = max_pages_per_slot
        # logical page index -> physical page (or -1), per slot
        self.table: List[List[int]] = [[-1] * max_pages_per_slot for _ in range(num_slots)]
        self.dirty: set = set()                       # slots whose table row changed
        self._trim_mark: Dict[int, int] = {}          # slot -> first logical page still kept

    def cover(self, slot: int, length: int) -> None:
        """Make sure pages exist for positions [trimmed start, length)."""
        row = self.table[slot]
        last = (length + PAGE - 1) // PAGE
        if last > self.max_pages_per_slot:
            raise CacheError(f"a sequence of {length} tokens exceeds the cache's limit of "
                             f"{self.max_pages_per_slot * PAGE} tokens per sequence")
        missing = [lp for lp in range(self._trim_mark.get(slot, 0), last) if row[lp] < 0]
        if len(missing) > self.pool.available():
            raise CacheError(f"the cache is full: {len(missing)} more pages of {PAGE} tokens are "
                             f"needed, {self.pool.available()} of {self.pool.n} are free")
        for lp in missing:
            row[lp] = self.pool.take()
        if missing:
            self.dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Hand back pages no token at position >= ``length`` can see (window groups)."""
        if self.window is None:
            return
        first_visible = max(0, length - self.window + 1)   # oldest key the next token reads
        keep_from = first_visible // PAGE
        row = self.table[slot]
        for lp in range(self._trim_mark.get(slot, 0), min(keep_from, self.max_pages_per_slot)):
            if row[lp] >= 0:
                self.pool.give_back(row[lp])
                row[lp] = -1
                self.dirty.add(slot)
        self._trim_mark[slot] = max(self._trim_mark.get(slot, 0), keep_from)

    def release(self, slot: int) -> None:
        row = self.table[slot]
        for lp, p in enumerate(row):
            if p >= 0:
                self.pool.give_back(p)
                row[lp] = -1
        self._trim_mark.pop(slot, None)
        self.dirty.add(slot)

    def pages_of(self, slot: int) -> List[int]:
        return [p for p in self.table[slot] if p >= 0]


class SlotBook:
    """Slots, their lengths, and their pages in every group."""

    def __init__(self, num_slots: int, groups: List[PageGroup], max_len: int):
        self.slots = FreeList(num_slots, "sequence slot")
        self.groups = groups
        self.max_len = max_len
        self.length = [0] * num_slots
        self.generation = [0] * num_slots            # counts how often a slot was taken

    def open(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        self.generation[s] += 1
        return s

    def _check_held(self, slot: int) -> None:
        if not (0 <= slot < self.slots.n and self.slots._held[slot]):
            raise CacheError(f"sequence slot {slot} is not open")

    def reserve(self, slot: int, new_length: int) -> None:
        """Pages for the sequence to grow to ``new_length`` tokens, in every group."""
        self.reserve_all([(slot, new_length)])

    def reserve_all(self, wanted) -> None:
        """Pages for several sequences at once, ``wanted`` = (slot, new length) pairs: either every
        sequence gets its pages in every group, or none gets any and CacheError says why."""
        wanted = list(wanted)
        for slot, new_length in wanted:
            self._check_held(slot)
            if new_length > self.max_len:
                raise CacheError(f"a sequence of {new_length} tokens exceeds the limit of "
                                 f"{self.max_len} positions")
        # all-or-nothing over the sequences and the groups: count first, then take
        for g in self.groups:
            missing = 0
            for slot, new_length in wanted:
                row = g.table[slot]
                last = (new_length + PAGE - 1) // PAGE
                if last > g.max_pages_per_slot:
                    raise CacheError(f"a sequence of {new_length} tokens exceeds the cache's limit of "
                                     f"{g.max_pages_per_slot * PAGE} tokens per sequence")
                start = g._trim_mark.get(slot, 0)
                missing += sum(1 for lp in range(start, last) if row[lp] < 0)
            if missing > g.pool.available():
                raise CacheError(f"the cache is full: {missing} more pages of {PAGE} tokens are "
                                 f"needed, {g.pool.available()} of {g.pool.n} are free")
        for g in self.groups:
            for slot, new_length in wanted:
                g.cover(slot, new_length)

    def advance(self, slot: int, n: int) -> None:
        self._check_held(slot)
        self.length[slot] += n
        for g in self.groups:
            g.trim(slot, self.length[slot])

    def close(self, slot: int) -> None:
        self._check_held(slot)
        for g in self.groups:
            g.release(slot)
        self.length[slot] = 0
        self.slots.give_back(slot)

    def open_slots(self) -> List[int]:
        return self.slots.held()
