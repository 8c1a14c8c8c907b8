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
    # Host copies; None in a step that is replayed from a captured graph (its
    # kernels were recorded once and may not depend on host-side step values)
    slots_host: Optional[List[int]]
    cu_tokens_host: Optional[List[int]]
    kv_lens_host: Optional[List[int]]
    is_decode: bool  # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int
    # Whether the sequences' lengths differ much (a hint for kernels that share work
    # among sequences; in a replayed step it is fixed when the step is captured)
    unequal_lengths: bool = False
    # In a replayed prompt step: an upper bound of the number of query blocks of
    # 64 rows over all sequences (the attention's grid), else None
    query_blocks_bound: Optional[int] = None
    # ... and whether some sequence brings 64 tokens or more (the choice between
    # the two prompt-attention kernels, made as a plain step makes it)
    long_queries: bool = False
    _tables: Dict[int, torch.Tensor] = field(default_factory=dict)
    # The weight that the step streams after the part being run (a prefetch
    # hint, set by the model and the blocks as they go; None = unknown).
    reads_after_part: Optional[torch.Tensor] = None
    # An `ops.ResidualSink` when the result of the part being run goes into a sum
    # with the residual rows and a norm whose consumer takes it unscaled; the
    # part's last projection may then do both (set like `reads_after_part`).
    residual_sink: Optional[object] = None
    # Tensors derived from the step that several parts share (the rotary angles of
    # the step's positions, the same for every layer). Whoever runs another step on
    # the same context clears it first (`Model.forward` does).
    shared: Dict[object, torch.Tensor] = field(default_factory=dict)

    def page_table(self, group: KVGroup) -> torch.Tensor:
        """int32 [n_seqs, width]: the pages of each sequence in `group`."""
        return self._tables[id(group)]


@dataclass
class StepPlan:
    """A validated step on the host, its cache pages reserved."""
    token_ids: np.ndarray
    positions: np.ndarray
    seq_of: np.ndarray
    want_rows: List[int]
    slots: List[int]
    cu: List[int]
    kv_lens: List[int]
    tables: list  # (group, width, rows [n_seqs][width]) per cache group


def check_steps(cache: SequenceCache, steps: Sequence[SequenceStep], vocab_size: int,
                max_positions: Optional[int] = None) -> Dict[int, int]:
    """Validate a step; returns slot -> length after the step. Changes nothing."""
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
    return growth


def plan_step(cache: SequenceCache, steps: Sequence[SequenceStep], vocab_size: int,
              max_positions: Optional[int] = None) -> StepPlan:
    """Validate a step and reserve its cache pages. Nothing is changed when
    validation or the reservation fails."""
    growth = check_steps(cache, steps, vocab_size, max_positions)
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
    tables = []
    for group in cache.groups:
        width = max(1, max(len(group.pages.pages(slot)) for slot in slots))
        tables.append((group, width, cache.page_table_rows(group, slots, width)))
    return StepPlan(token_ids, positions, seq_of, want_rows, slots, cu, kv_lens, tables)


def lengths_are_unequal(lengths: Sequence[int]) -> bool:
    """Whether the longest of several sequences is well beyond their mean (a
    quarter more, and at least four pages)."""
    if len(lengths) < 2:
        return False
    mean = sum(lengths) / len(lengths)
    return max(lengths) > 1.25 * mean and max(lengths) - mean >= 256


def build_context(cache: SequenceCache, steps: Sequence[SequenceStep], vocab_size: int,
                  device: torch.device, max_positions: Optional[int] = None,
                  plan: Optional[StepPlan] = None) -> StepContext:
    """Validate a step, reserve its cache pages, and upload its description
    (or upload a step already planned)."""
    if plan is None:
        plan = plan_step(cache, steps, vocab_size, max_positions)
    n_seqs, T = len(plan.slots), int(plan.token_ids.size)
    lens = [plan.cu[i + 1] - plan.cu[i] for i in range(n_seqs)]
    # one packed int32 upload: fixed fields, then one page table per group
    fields = [plan.token_ids, plan.positions, plan.seq_of, np.asarray(plan.want_rows, np.int32),
              np.asarray(plan.slots, np.int32), np.asarray(plan.cu, np.int32),
              np.asarray(plan.kv_lens, np.int32)]
    for _, _, rows in plan.tables:
        fields.append(np.asarray(rows, np.int32).reshape(-1))
    offsets = np.cumsum([0] + [f.size for f in fields])
    packed = torch.from_numpy(np.concatenate(fields)).to(device)
    part = [packed[offsets[i]:offsets[i + 1]] for i in range(len(fields))]
    ctx = StepContext(
        n_tokens=T, n_seqs=n_seqs, n_want=len(plan.want_rows),
        token_ids=part[0], positions=part[1], seq_of_token=part[2], want_rows=part[3],
        slots=part[4], cu_tokens=part[5], kv_lens=part[6],
        slots_host=plan.slots, cu_tokens_host=plan.cu, kv_lens_host=plan.kv_lens,
        is_decode=all(n == 1 for n in lens), max_q_len=max(lens), max_kv_len=max(plan.kv_lens),
        unequal_lengths=lengths_are_unequal(plan.kv_lens))
    for i, (group, width, _) in enumerate(plan.tables):
        ctx._tables[id(group)] = part[7 + i].view(n_seqs, width)
    return ctx
