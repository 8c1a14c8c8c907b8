"""Device storage of the cache and the per-sequence state, in layer groups.

A mixer states what it needs per sequence: keys and values for all positions
(`KVRequest(window=None)`), for a window of them (`window=W`), a state of fixed
size (`StateRequest`), or nothing. Cache entries with the same key-value shape
and policy form a group with storage and a page pool of its own:

    storage[entry, page, 0 = keys / 1 = values, kv head, row in page, head_dim]

so one (page, head) block of `PAGE x head_dim` elements is contiguous. The
reference holds `[batch, kv heads, max_cache_len, head_dim]` per layer, all
layers alike (src/nn/kv_cache.rs:13-39), and has no per-sequence state.

State rows are `state[entry][slot, ...]`; they are zeroed when a slot is
opened, because unlike keys and values (bounded by the length) a state carries
over whatever the last sequence left.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from .pages import PAGE, CacheFull, CacheMisuse, GroupPages, SlotTable, pages_for


@dataclass(frozen=True)
class KVRequest:
    kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: every earlier position stays readable


@dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheRequest = Union[KVRequest, StateRequest, None]


class KVGroup:
    def __init__(self, request: KVRequest, entries: List[int], page_count: int,
                 dtype: torch.dtype, device: torch.device):
        self.request = request
        self.entries = entries
        self.index_of = {e: i for i, e in enumerate(entries)}
        self.pages = GroupPages(page_count, request.window)
        self.storage = torch.zeros(
            (len(entries), page_count, 2, request.kv_heads, PAGE, request.head_dim),
            dtype=dtype, device=device)
        self._views: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    @property
    def ring_pages(self) -> int:
        return self.pages.ring_pages

    @property
    def window(self) -> int:
        return self.request.window or 0

    def kv(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        views = self._views.get(entry)
        if views is None:  # the views never change: made once per entry
            block = self.storage[self.index_of[entry]]
            views = self._views[entry] = (block[:, 0], block[:, 1])
        return views

    def bytes_per_token(self) -> int:
        r = self.request
        return len(self.entries) * 2 * r.kv_heads * r.head_dim * self.storage.element_size()


@dataclass
class KVView:
    """What a mixer run sees of the cache: one entry of one group."""
    group: KVGroup
    entry: int
    writes: bool

    @property
    def k(self) -> torch.Tensor:
        return self.group.kv(self.entry)[0]

    @property
    def v(self) -> torch.Tensor:
        return self.group.kv(self.entry)[1]


@dataclass
class StateView:
    """A state tensor [slots, ...]; a sequence's row is its slot."""
    rows: torch.Tensor
    entry: int
    writes: bool


class SequenceCache:
    """All cache memory of an engine: groups, state, and the slot table."""

    def __init__(self, requests: Mapping[int, CacheRequest], max_tokens: int, max_slots: int,
                 dtype: torch.dtype, device: torch.device):
        if max_tokens < PAGE:
            raise ValueError(f"the cache must hold at least one page of {PAGE} tokens")
        self.dtype, self.device = dtype, device
        self.max_tokens = pages_for(max_tokens) * PAGE
        page_count = self.max_tokens // PAGE
        self.max_slots = max(1, min(max_slots, page_count))
        by_key: Dict[KVRequest, List[int]] = {}
        self.state: Dict[int, torch.Tensor] = {}
        for entry in sorted(requests):
            req = requests[entry]
            if isinstance(req, KVRequest):
                by_key.setdefault(req, []).append(entry)
            elif isinstance(req, StateRequest):
                # one row more than slots: padding rows of a step point at the last row
                self.state[entry] = torch.zeros((self.max_slots + 1, *req.shape),
                                                dtype=req.dtype, device=device)
            elif req is not None:
                raise TypeError(f"cache entry {entry}: unknown request {req!r}")
        self.groups: List[KVGroup] = []
        self.group_of: Dict[int, KVGroup] = {}
        for req, entries in by_key.items():
            count = page_count
            if req.window is not None:
                count = min(page_count, self.max_slots * (pages_for(req.window) + 1))
            group = KVGroup(req, entries, count, dtype, device)
            self.groups.append(group)
            for e in entries:
                self.group_of[e] = group
        self.table = SlotTable(self.max_slots, [g.pages for g in self.groups])
        self.scratch_slot = self.max_slots  # state row that padding rows may scribble on

    # --------------------------------------------------------------- slots
    def open_sequence(self) -> int:
        slot = self.table.open()
        for rows in self.state.values():
            rows[slot].zero_()
        return slot

    def close_sequence(self, slot: int) -> None:
        self.table.close(slot)

    def length(self, slot: int) -> int:
        return self.table.length[slot]

    def reserve(self, growth: Mapping[int, int]) -> None:
        """Make room for every `slot -> new length` of a step, or change nothing."""
        if not self.table.can_grow(dict(growth)):
            raise CacheFull(
                f"the step needs more pages than are free "
                f"({[g.pages.pool.free for g in self.groups]} free of "
                f"{[g.pages.pool.count for g in self.groups]})")
        for slot, length in growth.items():
            self.table.grow(slot, length)

    def forget_from(self, slot: int, length: int) -> None:
        """Give up the slot's tokens from `length` on (see `SlotTable.forget_from`).
        Only keys and values can be forgotten: state of fixed size has been
        overwritten by the step, so a cache that holds any refuses."""
        if self.state:
            raise CacheMisuse("per-sequence state cannot be taken back a step")
        self.table.forget_from(slot, length)

    def step_token_limit(self) -> Optional[int]:
        """The most tokens one sequence may bring in one step, or None for no
        limit. A step writes all its keys before any of them is read, and a
        windowed group's pages are a ring of `ring_pages * PAGE` rows in which
        position p takes the row of p - ring_pages * PAGE: a step of c tokens
        from position s on leaves s's window (s - window, s] intact only if
        s + c - 1 - ring_pages * PAGE < s - window + 1."""
        limits = [g.ring_pages * PAGE - g.window + 1 for g in self.groups if g.window]
        return min(limits) if limits else None

    def free_tokens(self) -> int:
        return min((g.pages.pool.free for g in self.groups), default=0) * PAGE

    # --------------------------------------------------------------- views
    def view(self, entry: int, writes: bool):
        if entry in self.group_of:
            return KVView(self.group_of[entry], entry, writes)
        if entry in self.state:
            return StateView(self.state[entry], entry, writes)
        return None

    def page_table_rows(self, group: KVGroup, slots: Sequence[int], width: int) -> List[List[int]]:
        rows = []
        for slot in slots:
            pages = group.pages.pages(slot) if slot >= 0 else []
            rows.append(list(pages) + [0] * (width - len(pages)))
        return rows

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)
