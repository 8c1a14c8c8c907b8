"""The generation loop's decisions, on a scripted backend without a GPU:
batches of unequal prompts, stop tokens, rows that end earlier and give their
slot back, as many batches one after another as the requests need. The stop
rule's cases are the reference's (src/generate/mod.rs:295-374)."""
import pytest

from foundry_b200.cache import PAGE, FreeList
from foundry_b200.engine.generate import (EmptyBatch, EmptyPrompt, PromptTooLong, generate,
                                          is_stopped, plan_batch, tokens_held)
from foundry_b200.sampling import SamplingParams


class ScriptedBackend:
    """Token t of request r is script[r][t]. Tracks slots and cache tokens the
    way the engine does and records every step."""

    def __init__(self, script, slots=4, capacity=64 * PAGE, positions=10_000):
        self.script, self.capacity, self.positions = script, capacity, positions
        self.slots = FreeList(slots, "slot")
        self.length = {}
        self.log = []
        self.more = []  # what the loop said about coming back, a step

    def open_sequence(self):
        (s,) = self.slots.take(1)
        self.length[s] = 0
        return s

    def close_sequence(self, slot):
        self.slots.give([slot])
        del self.length[slot]

    def free_slots(self):
        return self.slots.free

    def _held(self):
        return sum(-(-n // PAGE) * PAGE for n in self.length.values())

    def free_tokens(self):
        return self.capacity - self._held()

    def capacity_tokens(self):
        return self.capacity

    def max_positions(self):
        return self.positions

    def step_select(self, steps, params, keys, counts, more=False):
        assert len({s.slot for s in steps}) == len(steps)
        self.more.append(more)
        for s in steps:
            assert self.slots.is_held(s.slot)
            self.length[s.slot] += len(s.tokens)
        assert self._held() <= self.capacity
        self.log.append([(k, list(s.tokens), c) for s, k, c in zip(steps, keys, counts)])
        return [self.script[k][c] for k, c in zip(keys, counts)]


def test_is_stopped_looks_at_the_last_token_only():
    assert is_stopped([4, 9], [9]) and is_stopped([9], [1, 9])
    assert not is_stopped([9, 4], [9]) and not is_stopped([], [9]) and not is_stopped([9], [])


def test_unequal_prompts_rows_end_earlier_and_keep_their_stop_token():
    script = {0: [10, 11, 99, 13], 1: [20, 99, 22, 23], 2: [30, 31, 32, 33]}
    backend = ScriptedBackend(script)
    out = generate(backend, [[1, 2, 3], [4], [5, 6]], 4, eos_token_ids=[99])
    assert out.token_ids == [[10, 11, 99], [20, 99], [30, 31, 32, 33]]
    assert out.finish_reason == ["stop", "stop", "length"]
    # prompts in one step; then one token each, finished rows no longer fed
    assert backend.log[0] == [(0, [1, 2, 3], 0), (1, [4], 0), (2, [5, 6], 0)]
    assert backend.log[1] == [(0, [10], 1), (1, [20], 1), (2, [30], 1)]
    assert backend.log[2] == [(0, [11], 2), (2, [31], 2)]
    assert backend.log[3] == [(2, [32], 3)]
    assert len(backend.log) == 4 and len(out.decode_steps) == 3
    assert backend.slots.free == 4 and backend.length == {}
    # the loop expects to come back with the same rows while none reaches its limit
    # with the step's token (a stop token it cannot foresee); never for prompts
    assert backend.more == [False, True, True, False]


def test_the_prompt_step_gives_the_first_token_and_zero_tokens_touch_nothing():
    backend = ScriptedBackend({0: [5, 6]})
    assert generate(backend, [[1]], 1).token_ids == [[5]]
    assert len(backend.log) == 1  # no decode step for a single new token
    backend = ScriptedBackend({0: [5]})
    out = generate(backend, [[1], [2]], 0)
    assert out.token_ids == [[], []] and backend.log == []


def test_stop_token_at_the_prompt_step():
    backend = ScriptedBackend({0: [99], 1: [1, 2, 3]})
    out = generate(backend, [[1], [2]], 3, eos_token_ids=[99])
    assert out.token_ids == [[99], [1, 2, 3]] and out.finish_reason == ["stop", "length"]


def test_ignore_eos_runs_to_length():
    backend = ScriptedBackend({0: [99, 99, 99]})
    out = generate(backend, [[1]], 3, eos_token_ids=[99], ignore_eos=True)
    assert out.token_ids == [[99, 99, 99]] and out.finish_reason == ["length"]


def test_more_requests_than_slots_run_as_batches_one_after_another():
    script = {r: [r * 10 + t for t in range(3)] for r in range(7)}
    backend = ScriptedBackend(script, slots=3)
    out = generate(backend, [[r] * (r + 1) for r in range(7)], 3)
    assert out.batches == [[0, 1, 2], [3, 4, 5], [6]]
    assert out.token_ids == [script[r] for r in range(7)]
    assert backend.slots.free == 3


def test_batches_are_cut_by_cache_pages_too():
    # each request holds 2 pages (100 prompt tokens + new ones); the cache has 5 pages
    backend = ScriptedBackend({r: [1, 2] for r in range(4)}, slots=8, capacity=5 * PAGE)
    out = generate(backend, [[0] * 100] * 4, 2)
    assert out.batches == [[0, 1], [2, 3]]
    assert tokens_held(100, 2) == 2 * PAGE and tokens_held(64, 1) == PAGE
    assert plan_batch([0, 1, 2], [10, 10, 10], 4, free_slots=2, free_tokens=10 * PAGE,
                      max_batch=None) == [0, 1]
    assert plan_batch([0, 1, 2], [10, 10, 10], 4, 8, 10 * PAGE, max_batch=1) == [0]


def test_refusals():
    backend = ScriptedBackend({0: [1]}, capacity=2 * PAGE, positions=100)
    with pytest.raises(EmptyBatch):
        generate(backend, [], 1)
    with pytest.raises(EmptyPrompt):
        generate(backend, [[1], []], 1)
    with pytest.raises(PromptTooLong, match="positions"):
        generate(backend, [[1] * 99], 3)
    with pytest.raises(PromptTooLong, match="cache"):
        generate(ScriptedBackend({0: [1]}, capacity=PAGE), [[1] * 65], 2)
    assert backend.log == []


def test_slots_go_back_when_a_step_fails():
    class Failing(ScriptedBackend):
        def step_select(self, steps, params, keys, counts, more=False):
            if len(self.log) == 1:
                raise RuntimeError("device failure")
            return super().step_select(steps, params, keys, counts, more)
    backend = Failing({0: [1, 2, 3], 1: [4, 5, 6]})
    with pytest.raises(RuntimeError):
        generate(backend, [[1], [2]], 3)
    assert backend.slots.free == 4


def test_sampling_keys_and_counts_do_not_depend_on_the_batch():
    """A request's (key, count) stream is (its index, tokens generated so far)
    whichever batch it runs in."""
    script = {r: [1, 2, 3] for r in range(4)}
    a = ScriptedBackend(script, slots=4)
    generate(a, [[0]] * 4, 3, sampling=SamplingParams(temperature=0.8, seed=3))
    b = ScriptedBackend(script, slots=1)
    generate(b, [[0]] * 4, 3, sampling=SamplingParams(temperature=0.8, seed=3))
    seen = lambda backend: sorted((k, c) for step in backend.log for k, _, c in step)
    assert seen(a) == seen(b) == sorted((r, c) for r in range(4) for c in range(3))


def test_sampling_params():
    assert SamplingParams().greedy and not SamplingParams(temperature=0.5).greedy
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
