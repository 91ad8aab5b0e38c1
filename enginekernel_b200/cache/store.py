"""Device storage of the cache: key/value pages and fixed-size per-sequence state.

Cache entries (one per scheduled mixer that keeps something) with equal
:class:`~enginekernel_b200.parts.spec.CacheSpec` form a group.  A ``kv`` group owns
``pages[entry, k|v, page, kv_head, PAGE, head_dim]`` in the engine's dtype and a block
table ``[slot, logical page] -> page``; a ``state`` group owns
``data[entry, slot, *shape]``, zeroed whenever a sequence takes the slot.  Sizes are fixed
at construction from the number of tokens to hold (``max_tokens``, counted per sequence
in whole pages), the number of sequences alive at once and the longest sequence.

The reference's cache is a list of per-layer tensors indexed by batch row, with the
split-K workspace and the per-step device counters kept in its graph objects
(engine/engine.py:172-174, 239-263, 273-282).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..parts.spec import CacheSpec
from .pages import PAGE, CacheError, PageGroup, SlotBook

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class EntryView:
    """What one scheduled mixer sees of the cache."""

    def __init__(self, spec: CacheSpec, group: "GroupStorage", index_in_group: int):
        self.spec = spec
        self._group = group
        self._i = index_in_group

    @property
    def k_pages(self):
        return self._group.pages[self._i, 0]

    @property
    def v_pages(self):
        return self._group.pages[self._i, 1]

    @property
    def block_table(self):
        return self._group.block_table

    @property
    def state(self):
        """[slots, *shape] for ``state`` entries."""
        return self._group.data[self._i]


class GroupStorage:
    def __init__(self, spec: CacheSpec, entries: List[int], dtype, device, num_pages: int,
                 num_slots: int, max_pages_per_slot: int):
        self.spec, self.entries = spec, entries
        self.page_group: Optional[PageGroup] = None
        self.pages = self.block_table = self.data = None
        if spec.kind == "kv":
            self.page_group = PageGroup(num_pages, num_slots, max_pages_per_slot, spec.window)
            self.pages = torch.zeros((len(entries), 2, num_pages, spec.heads, PAGE, spec.head_dim),
                                     dtype=dtype, device=device)
            self.block_table = torch.zeros((num_slots, max_pages_per_slot), dtype=torch.int32,
                                           device=device)
            pin = torch.device(device).type == "cuda"
            self.host_table = torch.zeros((num_slots, max_pages_per_slot), dtype=torch.int32,
                                          pin_memory=pin)
        elif spec.kind == "state":
            self.data = torch.zeros((len(entries), num_slots) + tuple(spec.shape),
                                    dtype=_STATE_DTYPES[spec.state_dtype], device=device)
        else:
            raise CacheError(f"unknown cache kind {spec.kind!r} (kinds: kv, state)")

    def upload_table(self) -> None:
        g = self.page_group
        if g is None or not g.dirty:
            return
        lo, hi = min(g.dirty), max(g.dirty) + 1
        for s in g.dirty:
            row = g.table[s]
            self.host_table[s] = torch.tensor([p if p >= 0 else 0 for p in row], dtype=torch.int32)
        self.block_table[lo:hi].copy_(self.host_table[lo:hi], non_blocking=True)
        g.dirty.clear()

    def bytes(self) -> int:
        t = self.pages if self.pages is not None else self.data
        return t.numel() * t.element_size()


class SequenceCache:
    """Slots for sequences, storage for every cache entry of a model."""

    def __init__(self, entry_specs: Sequence[Optional[CacheSpec]], dtype, device,
                 max_tokens: int, max_slots: Optional[int] = None, max_len: Optional[int] = None):
        if max_tokens <= 0:
            raise CacheError("the cache must hold at least one token")
        self.dtype, self.device = dtype, torch.device(device)
        self.num_pages = (max_tokens + PAGE - 1) // PAGE
        self.max_len = min(max_len or max_tokens, self.num_pages * PAGE)
        self.max_pages_per_slot = (self.max_len + PAGE - 1) // PAGE
        self.num_slots = max(1, min(max_slots or 1024, self.num_pages))
        self.groups: List[GroupStorage] = []
        self._entry_view: Dict[int, EntryView] = {}
        by_key: Dict[tuple, List[int]] = {}
        specs: Dict[tuple, CacheSpec] = {}
        for i, spec in enumerate(entry_specs):
            if spec is None:
                continue
            by_key.setdefault(spec.group_key(), []).append(i)
            specs[spec.group_key()] = spec
        for key, entries in by_key.items():
            g = GroupStorage(specs[key], entries, dtype, self.device, self.num_pages,
                             self.num_slots, self.max_pages_per_slot)
            self.groups.append(g)
            for j, e in enumerate(entries):
                self._entry_view[e] = EntryView(specs[key], g, j)
        self.book = SlotBook(self.num_slots,
                             [g.page_group for g in self.groups if g.page_group is not None],
                             self.max_len)

    # -- slots ---------------------------------------------------------------
    def open(self) -> int:
        """A free slot for a new sequence: length 0, fixed-size state zeroed."""
        slot = self.book.open()
        for g in self.groups:
            if g.data is not None:
                g.data[:, slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.book.close(slot)

    def reserve(self, slot: int, new_length: int) -> None:
        self.book.reserve(slot, new_length)

    def reserve_all(self, wanted) -> None:
        """(slot, new length) pairs: all of them get their pages, or none does."""
        self.book.reserve_all(wanted)

    def advance(self, slot: int, n: int) -> None:
        self.book.advance(slot, n)

    def length(self, slot: int) -> int:
        self.book._check_held(slot)
        return self.book.length[slot]

    def free_tokens(self) -> int:
        pools = [g.page_group.pool.available() for g in self.groups if g.page_group is not None]
        return (min(pools) if pools else self.num_pages) * PAGE

    # -- device side -----------------------------------------------------------
    def upload_tables(self) -> None:
        for g in self.groups:
            g.upload_table()

    def entry(self, index: int) -> EntryView:
        try:
            return self._entry_view[index]
        except KeyError:
            raise CacheError(f"cache entry {index} holds nothing") from None

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)
