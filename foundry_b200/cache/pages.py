"""Host-side bookkeeping of the cache: sequence slots and token pages.

The reference's cache is one dense tensor pair per layer, [batch, kv heads,
max_cache_len, head_dim], created anew for every generation; the batch index
is the slot and nothing is ever given back (src/nn/kv_cache.rs:13-39,
src/generate/mod.rs:92-108). Here memory is a pool of pages of `PAGE` tokens;
a sequence holds a slot (its fixed-size record: length, state row) and, in
every layer group, as many pages as its length needs. Ending a sequence gives
slot and pages back to the pool, and the next sequence uses them again without
clearing: a sequence's length bounds every read.

These classes hold no device memory and are tested on the CPU: no page or slot
is lost, held twice or freed twice.
"""
from __future__ import annotations

from typing import Dict, List, Optional

PAGE = 64


class CacheError(RuntimeError):
    """Base class of cache failures."""


class CacheFull(CacheError):
    """No free page or slot is left (the reference's analogue is
    `CacheOverflow`, src/models/llama/model.rs:331-340)."""


class CacheMisuse(CacheError):
    """A slot or page was released twice, or used without being held."""


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


class FreeList:
    """Identifiers 0..n-1, handed out lowest-recently-freed first."""

    def __init__(self, count: int, what: str):
        if count < 0:
            raise ValueError(f"negative {what} count")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count - 1, -1, -1))  # pop() gives the lowest first
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def take(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}(s) wanted, {len(self._free)} of {self.count} free")
        got = [self._free.pop() for _ in range(n)]
        for i in got:
            self._held[i] = True
        return got

    def give(self, ids) -> None:
        for i in ids:
            if not 0 <= i < self.count or not self._held[i]:
                raise CacheMisuse(f"{self.what} {i} is released but not held")
            self._held[i] = False
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.count and self._held[i]

    def check(self) -> None:
        """Every id is either free once or held, never both."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise CacheMisuse(f"a {self.what} is on the free list twice")
        for i in range(self.count):
            if self._held[i] == (i in seen):
                raise CacheMisuse(f"{self.what} {i} is both free and held, or neither")


class GroupPages:
    """The pages of one layer group and which sequence holds which.

    `window` (tokens) bounds a sequence's pages: its pages then form a ring
    that position p enters at `(p // PAGE) % ring_pages`, and the ring holds
    at least `window` tokens behind every position.
    """

    def __init__(self, page_count: int, window: Optional[int] = None):
        self.pool = FreeList(page_count, "page")
        self.window = window
        self.ring_pages = 0 if window is None else pages_for(window) + 1
        self._of_slot: Dict[int, List[int]] = {}

    def pages_needed(self, length: int) -> int:
        n = pages_for(length)
        return n if self.window is None else min(n, self.ring_pages)

    def open(self, slot: int) -> None:
        if slot in self._of_slot:
            raise CacheMisuse(f"slot {slot} already holds pages in this group")
        self._of_slot[slot] = []

    def grow(self, slot: int, length: int) -> None:
        held = self._of_slot[slot]
        extra = self.pages_needed(length) - len(held)
        if extra > 0:
            held.extend(self.pool.take(extra))

    def close(self, slot: int) -> None:
        self.pool.give(self._of_slot.pop(slot))

    def pages(self, slot: int) -> List[int]:
        return self._of_slot[slot]


class SlotTable:
    """Sequence slots, their lengths, and their pages in every group."""

    def __init__(self, slot_count: int, groups: List[GroupPages]):
        self.slots = FreeList(slot_count, "slot")
        self.groups = groups
        self.length = [0] * slot_count
        self.epoch = [0] * slot_count  # how often each slot has been opened

    def open(self) -> int:
        (slot,) = self.slots.take(1)
        self.length[slot] = 0
        self.epoch[slot] += 1
        for group in self.groups:
            group.open(slot)
        return slot

    def can_grow(self, growth: Dict[int, int]) -> bool:
        """Whether all of `growth` (slot -> new length) fits at once."""
        for group in self.groups:
            need = sum(max(0, group.pages_needed(n) - len(group.pages(s)))
                       for s, n in growth.items())
            if need > group.pool.free:
                return False
        return True

    def grow(self, slot: int, length: int) -> None:
        """Reserve pages so that the slot can hold `length` tokens."""
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not held")
        if length < self.length[slot]:
            raise CacheMisuse(f"slot {slot} would shrink from {self.length[slot]} to {length}")
        for group in self.groups:
            group.grow(slot, length)
        self.length[slot] = length

    def forget_from(self, slot: int, length: int) -> None:
        """The slot's tokens from `length` on are given up: a step that was run
        on a guess and is not wanted leaves the sequence as it was before it.
        The slot keeps its pages (the next step writes the same rows again)."""
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not held")
        if not 0 <= length <= self.length[slot]:
            raise CacheMisuse(f"slot {slot} holds {self.length[slot]} tokens, it cannot forget "
                              f"from {length} on")
        self.length[slot] = length

    def close(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is released but not held")
        for group in self.groups:
            group.close(slot)
        self.slots.give([slot])
        self.length[slot] = 0

    def check(self) -> None:
        self.slots.check()
        for group in self.groups:
            group.pool.check()
            owned = [p for pages in group._of_slot.values() for p in pages]
            if len(owned) != len(set(owned)):
                raise CacheMisuse("a page is held by two sequences")
            if len(owned) != group.pool.held:
                raise CacheMisuse("a page is held by no sequence")
            for slot in group._of_slot:
                if not self.slots.is_held(slot):
                    raise CacheMisuse(f"pages are held by slot {slot}, which is free")
