"""The generation loop: requests in, token ids out, one batch after another.

What the reference's loop does (src/generate/mod.rs:45-90): the prompts of a
batch are run in one step and give each row its first new token; then one
token per row and step; a row that produced a stop token keeps it and takes
no more (mod.rs:260-281); `max_new_tokens` counts the prompt step's token;
`max_new_tokens == 0` returns empty rows without touching the device
(mod.rs:53-59). Differences: prompts may have unequal lengths (the reference
raises `RaggedBatch`, mod.rs:217-223); a finished row leaves the batch at once
and its slot and pages go back to the pool (the reference keeps feeding it
until all rows are done, mod.rs:70-88); more requests than fit are run as
further batches; the next token may be sampled.

The loop decides on the host and only talks to a `StepBackend`, so its
decisions are tested without a GPU. It tells the backend when it expects to
come back with the same rows and the tokens it is about to receive (`more`),
so that a backend may have that step running while the loop decides.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Protocol, Sequence

from ..cache.pages import PAGE, pages_for
from ..sampling.params import SamplingParams
from .context import SequenceStep


class GenerateError(ValueError):
    """Base class of the loop's refusals (src/generate/error.rs)."""


class EmptyBatch(GenerateError): pass
class EmptyPrompt(GenerateError): pass
class PromptTooLong(GenerateError): pass


@dataclass
class Generation:
    """New tokens only, a row per request in request order
    (src/generate/mod.rs:31-36), and the host-clock durations."""
    token_ids: List[List[int]]
    finish_reason: List[str]  # "stop" | "length"
    prefill: float = 0.0  # seconds, summed over batches
    decode_steps: List[float] = field(default_factory=list)
    batches: List[List[int]] = field(default_factory=list)  # request indices of each batch


class StepBackend(Protocol):
    def open_sequence(self) -> int: ...
    def close_sequence(self, slot: int) -> None: ...
    def free_slots(self) -> int: ...
    def free_tokens(self) -> int: ...
    def capacity_tokens(self) -> int: ...
    def max_positions(self) -> int: ...
    def step_select(self, steps: Sequence[SequenceStep], params: SamplingParams,
                    keys: Sequence[int], counts: Sequence[int], more: bool = False) -> List[int]: ...


def is_stopped(row: Sequence[int], eos_token_ids: Sequence[int]) -> bool:
    """A row is finished once its last token is a stop token
    (src/generate/mod.rs:260-265)."""
    return bool(row) and row[-1] in eos_token_ids


def tokens_held(prompt_len: int, max_new_tokens: int) -> int:
    """Cache tokens a request can come to hold: prompt plus all new tokens but
    the last (which is never fed back), in whole pages."""
    return pages_for(prompt_len + max(0, max_new_tokens - 1)) * PAGE


def plan_batch(pending: Sequence[int], prompt_lens: Sequence[int], max_new_tokens: int,
               free_slots: int, free_tokens: int, max_batch: Optional[int]) -> List[int]:
    """The longest prefix of `pending` that fits the free slots and pages."""
    batch: List[int] = []
    need = 0
    for r in pending:
        cost = tokens_held(prompt_lens[r], max_new_tokens)
        if len(batch) >= free_slots or need + cost > free_tokens:
            break
        if max_batch is not None and len(batch) >= max_batch:
            break
        batch.append(r)
        need += cost
    return batch


def generate(backend: StepBackend, prompts: Sequence[Sequence[int]], max_new_tokens: int,
             eos_token_ids: Sequence[int] = (), sampling: SamplingParams = SamplingParams(),
             max_batch: Optional[int] = None, ignore_eos: bool = False) -> Generation:
    if len(prompts) == 0:
        raise EmptyBatch("the batch holds no prompt")
    if any(len(p) == 0 for p in prompts):
        raise EmptyPrompt("a prompt holds no token")
    n = len(prompts)
    result = Generation(token_ids=[[] for _ in range(n)], finish_reason=["length"] * n)
    if max_new_tokens <= 0:
        return result
    lens = [len(p) for p in prompts]
    limit = backend.max_positions()
    for r, length in enumerate(lens):
        if length + max_new_tokens - 1 > limit:
            raise PromptTooLong(f"request {r}: {length} prompt tokens + {max_new_tokens} new "
                                f"exceed the model's {limit} positions")
        if tokens_held(length, max_new_tokens) > backend.capacity_tokens():
            raise PromptTooLong(f"request {r} needs {tokens_held(length, max_new_tokens)} cache "
                                f"tokens, the cache holds {backend.capacity_tokens()}")
    stops = () if ignore_eos else tuple(eos_token_ids)
    pending = list(range(n))
    while pending:
        batch = plan_batch(pending, lens, max_new_tokens, backend.free_slots(),
                           backend.free_tokens(), max_batch)
        if not batch:
            raise PromptTooLong(f"request {pending[0]} does not fit the free cache")
        pending = pending[len(batch):]
        result.batches.append(list(batch))
        _run_batch(backend, batch, prompts, max_new_tokens, stops, sampling, result)
    return result


def _run_batch(backend, batch, prompts, max_new_tokens, stops, sampling, result) -> None:
    slot_of = {r: backend.open_sequence() for r in batch}
    live = list(batch)
    try:
        started = time.perf_counter()
        steps = [SequenceStep(slot_of[r], list(prompts[r]), [len(prompts[r]) - 1]) for r in live]
        tokens = backend.step_select(steps, sampling, live, [0] * len(live))
        result.prefill += time.perf_counter() - started
        live = _append(backend, live, tokens, slot_of, stops, max_new_tokens, result)
        while live:
            started = time.perf_counter()
            steps = [SequenceStep(slot_of[r], [result.token_ids[r][-1]], [0]) for r in live]
            counts = [len(result.token_ids[r]) for r in live]
            # unless a stop token ends a row, the same rows come back with the tokens
            # of this step: the backend may start that step before it returns
            more = all(c + 1 < max_new_tokens for c in counts)
            tokens = backend.step_select(steps, sampling, live, counts, more)
            result.decode_steps.append(time.perf_counter() - started)
            live = _append(backend, live, tokens, slot_of, stops, max_new_tokens, result)
    finally:
        for r in live:  # only after an error: give back what is still held
            backend.close_sequence(slot_of[r])


def _append(backend, live, tokens, slot_of, stops, max_new_tokens, result) -> List[int]:
    """Give each live row its token; rows that end give their slot back now."""
    still = []
    for r, token in zip(live, tokens):
        row = result.token_ids[r]
        row.append(int(token))
        if is_stopped(row, stops):
            result.finish_reason[r] = "stop"
        elif len(row) >= max_new_tokens:
            result.finish_reason[r] = "length"
        else:
            still.append(r)
            continue
        backend.close_sequence(slot_of[r])
    return still
