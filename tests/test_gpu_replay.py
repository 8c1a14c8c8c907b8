"""The engine against the plain implementation, for every way of cutting the
same requests into steps: each request alone and whole; whole but for the
last 32 tokens, which follow one by one; and batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages
are used again. In 32-bit and in bfloat16, on both tiny configurations.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [5, 11, 17, 70, 128, 33], "tiny_b": [1, 7, 40, 90, 200, 64, 65]}


@pytest.fixture(scope="module")
def oracle(tiny_folders):
    """{config: (requests, [logits [len, vocab] per request])} from the plain model."""
    out = {}
    for name, folder in tiny_folders.items():
        cfg, w = plain.read_model(folder)
        reqs = [tiny.random_tokens(100 + i, n, cfg["vocab_size"])
                for i, n in enumerate(LENGTHS[name])]
        out[name] = (reqs, [plain.forward(cfg, w, r).numpy() for r in reqs])
    return out


def make_engine(folder, dtype, max_tokens=1024, max_slots=16):
    from foundry_b200.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_slots=max_slots)


def run_whole(engine, tokens):
    from foundry_b200.engine import SequenceStep
    slot = engine.open_sequence()
    logits = engine.step([SequenceStep(slot, tokens, list(range(len(tokens))))])
    engine.close_sequence(slot)
    return logits.cpu().numpy()


def run_tail_one_by_one(engine, tokens, tail=32):
    from foundry_b200.engine import SequenceStep
    slot = engine.open_sequence()
    head = max(0, len(tokens) - tail)
    rows = []
    if head:
        rows.append(engine.step([SequenceStep(slot, tokens[:head], list(range(head)))]).cpu().numpy())
    for t in tokens[head:]:
        rows.append(engine.step([SequenceStep(slot, [t], [0])]).cpu().numpy())
    engine.close_sequence(slot)
    return np.concatenate(rows, 0)


def run_batches(engine, requests, batch_size, prompt_share=0.5):
    """Batches of `batch_size` requests: a first step with a prompt part of
    each, then one token each per step; a request that runs out of tokens ends
    and gives its slot back while the others go on."""
    from foundry_b200.engine import SequenceStep
    got = [None] * len(requests)
    for b0 in range(0, len(requests), batch_size):
        ids = list(range(b0, min(b0 + batch_size, len(requests))))
        slot = {r: engine.open_sequence() for r in ids}
        done = {r: max(1, int(len(requests[r]) * prompt_share)) for r in ids}
        rows = {r: [] for r in ids}
        logits = engine.step([SequenceStep(slot[r], requests[r][:done[r]], list(range(done[r])))
                              for r in ids]).cpu().numpy()
        at = 0
        for r in ids:
            rows[r].append(logits[at:at + done[r]])
            at += done[r]
        live = [r for r in ids if done[r] < len(requests[r])]
        for r in ids:
            if r not in live:
                engine.close_sequence(slot[r])
        while live:
            logits = engine.step([SequenceStep(slot[r], [requests[r][done[r]]], [0])
                                  for r in live]).cpu().numpy()
            for i, r in enumerate(live):
                rows[r].append(logits[i:i + 1])
                done[r] += 1
            for r in [r for r in live if done[r] == len(requests[r])]:
                engine.close_sequence(slot[r])
            live = [r for r in live if done[r] < len(requests[r])]
        for r in ids:
            got[r] = np.concatenate(rows[r], 0)
    engine.cache.table.check()
    assert engine.cache.table.slots.held == 0
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_each_request_alone_and_whole(tiny_folders, oracle, name, dtype):
    engine = make_engine(tiny_folders[name], dtype)
    requests, expected = oracle[name]
    for i, (tokens, want) in enumerate(zip(requests, expected)):
        tiny.assert_logits_close(run_whole(engine, tokens), want, dtype, f"{name} request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_last_32_tokens_one_by_one(tiny_folders, oracle, name, dtype):
    engine = make_engine(tiny_folders[name], dtype)
    requests, expected = oracle[name]
    for i, (tokens, want) in enumerate(zip(requests, expected)):
        got = run_tail_one_by_one(engine, tokens)
        tiny.assert_logits_close(got, want, dtype, f"{name} request {i} tail by tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_unequal_batches_with_slot_reuse(tiny_folders, oracle, name, dtype):
    # few pages: later batches must take the pages earlier ones gave back
    engine = make_engine(tiny_folders[name], dtype, max_tokens=512)
    requests, expected = oracle[name]
    for batch_size, share in ((3, 0.5), (2, 0.9), (4, 0.1)):
        got = run_batches(engine, requests, batch_size, share)
        for i, want in enumerate(expected):
            tiny.assert_logits_close(got[i], want, dtype,
                                     f"{name} request {i} in batches of {batch_size}")


MANY = 60  # requests of the crowded schedules below


@pytest.fixture(scope="module")
def crowd(tiny_folders):
    """{config: (requests, plain logits)}: many requests of unequal lengths,
    from one token to nearly the model's position limit."""
    out = {}
    for name, folder in tiny_folders.items():
        cfg, w = plain.read_model(folder)
        rng = np.random.default_rng(7)
        top = cfg["max_position_embeddings"] - 2
        lengths = [1, 2, top, 64, 65] + [int(n) for n in rng.integers(3, top, size=MANY - 5)]
        reqs = [tiny.random_tokens(900 + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)]
        out[name] = (reqs, [plain.forward(cfg, w, r).numpy() for r in reqs])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_twenty_and_forty_sequences_live_at_once(tiny_folders, crowd, name, dtype):
    """Single-token steps of 17 to 64 rows: batches of 20 and of 40 requests,
    prompts in one step, then one token each while the short ones end (so the
    live count walks down through the row buckets 64, 32, 16, ... with their
    padding rows), and the next batch takes the slots and pages given back."""
    requests, expected = crowd[name]
    longest = max(len(r) for r in requests)
    for batch_size, share in ((40, 0.5), (20, 0.3)):
        engine = make_engine(tiny_folders[name], dtype, max_slots=batch_size,
                             max_tokens=batch_size * (-(-longest // 64)) * 64)
        got = run_batches(engine, requests, batch_size, share)
        assert max(key[0] for key in engine._runners) == (64 if batch_size == 40 else 32)
        for i, want in enumerate(expected):
            tiny.assert_logits_close(got[i], want, dtype,
                                     f"{name} request {i} in batches of {batch_size}")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_float32_logits_do_not_depend_on_the_cutting(tiny_folders, oracle, name):
    """Beyond agreeing with the plain model, the 32-bit cuttings agree with
    one another far more tightly: same sums in the same order."""
    engine = make_engine(tiny_folders[name], "float32")
    requests, _ = oracle[name]
    whole = [run_whole(engine, r) for r in requests]
    tails = [run_tail_one_by_one(engine, r) for r in requests]
    batched = run_batches(engine, requests, 3)
    for w, t, b in zip(whole, tails, batched):
        assert np.abs(w - t).max() <= 2e-6 * max(1.0, np.abs(w).max())
        assert np.abs(w - b).max() <= 2e-6 * max(1.0, np.abs(w).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny_folders, oracle, tmp_path, dtype):
    """The replay program itself, as a user runs it: batches of unequal
    lengths, shorter requests ending earlier, slots used again."""
    name = "tiny_b"
    requests, expected = oracle[name]
    order = [0, 1, 2, 3, 5]
    steps, plan = [], []  # plan: per step, [(request, first position, count)]
    step_no = 0
    for batch in (order[:3], order[3:]):
        done = {r: max(1, len(requests[r]) // 2) for r in batch}
        steps.append({"step": step_no, "entries": [
            {"id": f"r{r}", "tokens": requests[r][:done[r]], "want": list(range(done[r]))}
            for r in batch], "end": [f"r{r}" for r in batch if done[r] == len(requests[r])]})
        plan.append([(r, 0, done[r]) for r in batch])
        step_no += 1
        live = [r for r in batch if done[r] < len(requests[r])]
        while live:
            ending = [r for r in live if done[r] + 1 == len(requests[r])]
            steps.append({"step": step_no, "entries": [
                {"id": f"r{r}", "tokens": [requests[r][done[r]]], "want": [0]} for r in live],
                "end": [f"r{r}" for r in ending]})
            plan.append([(r, done[r], 1) for r in live])
            for r in live:
                done[r] += 1
            live = [r for r in live if r not in ending]
            step_no += 1
    budget = max(sum(-(-len(requests[r]) // 64) * 64 for r in batch)
                 for batch in (order[:3], order[3:]))
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    out = tmp_path / "logits"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", tiny_folders[name],
         "--dtype", dtype, "--out", str(out), "--max-tokens", str(budget)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    vocab = expected[0].shape[1]
    all_got, all_want = [], []
    for s, rows in zip(steps, plan):
        got = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        want = np.concatenate([expected[r][p:p + n] for r, p, n in rows], 0)
        assert got.shape == want.shape, f"trace step {s['step']}"
        if dtype == "float32":
            tiny.assert_logits_close(got, want, dtype, f"trace step {s['step']}")
        else:  # a step of two rows is too small a sample for a 99.9 % rule: bound its worst
            scale = max(1.0, float(np.abs(want).max()))
            assert np.abs(got - want).max() <= 5e-2 * scale, f"trace step {s['step']}"
        all_got.append(got)
        all_want.append(want)
    tiny.assert_logits_close(np.concatenate(all_got), np.concatenate(all_want), dtype, "whole trace")
