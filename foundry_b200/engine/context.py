"""The description of one step that every part reads.

The reference passes one scalar `past_seen_tokens` for the whole batch and
builds positions and a dense mask from it on the host each step
(src/models/llama/model.rs:176-177, src/nn/masking.rs:11-32). Here every token
carries its own position and sequence, so sequences of unequal length run as
one packed batch and no mask is ever materialised.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.store import KVGroup, SequenceCache


@dataclass
class SequenceStep:
    """One sequence's share of a step: its slot, its next tokens, and the
    places among these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    n_tokens: int  # rows of every activation tensor, padding included
    n_seqs: int
    n_want: int
    token_ids: torch.Tensor  # int32 [n_tokens]
    positions: torch.Tensor  # int32 [n_tokens]
    seq_of_token: torch.Tensor  # int32 [n_tokens]; -1 marks padding
    want_rows: torch.Tensor  # int32 [n_want]: token rows whose logits are wanted
    slots: torch.Tensor  # int32 [n_seqs]: each sequence's slot (its state row)
    cu_tokens: torch.Tensor  # int32 [n_seqs + 1]
    kv_lens: torch.Tensor  # int32 [n_seqs]: sequence lengths after this step
    slots_host: List[int]
    cu_tokens_host: List[int]
    kv_lens_host: List[int]
    is_decode: bool  # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int
    _tables: Dict[int, torch.Tensor] = field(default_factory=dict)
    # The weight that the step streams after the part being run (a prefetch
    # hint, set by the model and the blocks as they go; None = unknown).
    reads_after_part: Optional[torch.Tensor] = None

    def page_table(self, group: KVGroup) -> torch.Tensor:
        """int32 [n_seqs, width]: the pages of each sequence in `group`."""
        return self._tables[id(group)]


def build_context(cache: SequenceCache, steps: Sequence[SequenceStep], vocab_size: int,
                  device: torch.device, max_positions: Optional[int] = None) -> StepContext:
    """Validate a step, reserve its cache pages, and upload its description.
    Nothing is changed when validation or the reservation fails."""
    if not steps:
        raise ValueError("a step needs at least one sequence")
    seen = set()
    growth: Dict[int, int] = {}
    for s in steps:
        if s.slot in seen:
            raise ValueError(f"slot {s.slot} appears twice in one step")
        seen.add(s.slot)
        if not cache.table.slots.is_held(s.slot):
            raise ValueError(f"slot {s.slot} is not open")
        if len(s.tokens) == 0:
            raise ValueError(f"slot {s.slot} brings no token")  # EmptyInput, model.rs:323-329
        for t in s.tokens:
            if not 0 <= int(t) < vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab_size}")
        for w in s.want:
            if not 0 <= int(w) < len(s.tokens):
                raise ValueError(f"wanted place {w} is outside the {len(s.tokens)} tokens given")
        new_len = cache.length(s.slot) + len(s.tokens)
        if max_positions is not None and new_len > max_positions:
            raise ValueError(f"slot {s.slot} would reach {new_len} positions, the model's "
                             f"limit is {max_positions}")
        growth[s.slot] = new_len
    starts = [cache.length(s.slot) for s in steps]
    cache.reserve(growth)

    n_seqs = len(steps)
    lens = [len(s.tokens) for s in steps]
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    token_ids = np.empty(T, np.int32)
    positions = np.empty(T, np.int32)
    seq_of = np.empty(T, np.int32)
    want_rows: List[int] = []
    for i, s in enumerate(steps):
        a, b = cu[i], cu[i + 1]
        token_ids[a:b] = np.asarray(s.tokens, dtype=np.int64)
        positions[a:b] = np.arange(starts[i], starts[i] + lens[i])
        seq_of[a:b] = i
        want_rows.extend(a + int(w) for w in s.want)
    kv_lens = [starts[i] + lens[i] for i in range(n_seqs)]
    slots = [s.slot for s in steps]

    # one packed int32 upload: fixed fields, then one page table per group
    fields = [token_ids, positions, seq_of, np.asarray(want_rows, np.int32),
              np.asarray(slots, np.int32), np.asarray(cu, np.int32), np.asarray(kv_lens, np.int32)]
    tables = []
    for group in cache.groups:
        width = max(1, max(len(group.pages.pages(slot)) for slot in slots))
        tables.append((group, width))
        fields.append(np.asarray(cache.page_table_rows(group, slots, width), np.int32).reshape(-1))
    offsets = np.cumsum([0] + [f.size for f in fields])
    packed = torch.from_numpy(np.concatenate(fields)).to(device)
    part = [packed[offsets[i]:offsets[i + 1]] for i in range(len(fields))]
    ctx = StepContext(
        n_tokens=T, n_seqs=n_seqs, n_want=len(want_rows),
        token_ids=part[0], positions=part[1], seq_of_token=part[2], want_rows=part[3],
        slots=part[4], cu_tokens=part[5], kv_lens=part[6],
        slots_host=slots, cu_tokens_host=cu, kv_lens_host=kv_lens,
        is_decode=all(n == 1 for n in lens), max_q_len=max(lens), max_kv_len=max(kv_lens))
    for i, (group, width) in enumerate(tables):
        ctx._tables[id(group)] = part[7 + i].view(n_seqs, width)
    return ctx
