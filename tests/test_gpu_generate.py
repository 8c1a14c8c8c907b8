"""Generation through the entry points: greedy tokens against the plain
implementation, stop tokens, rows that end earlier, slots used again, more
requests than slots, temperature sampling restated on the host, long decoding,
the first tokens of a sequence, and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def engine_for(folder, dtype, **kw):
    import foundry_b200 as fb
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_slots", 8)
    return fb.Engine.from_folder(folder, dtype=dtype, **kw)


def plain_greedy_is_decisive(cfg, w, prompt, tokens, margin):
    """Whether every greedy choice of the plain model along `tokens` beats the
    runner-up by `margin`: then a 16-bit engine must choose the same."""
    seq = list(prompt)
    for t in tokens:
        row = plain.forward(cfg, w, seq)[-1]
        top = torch.topk(row, 2).values
        if float(top[0] - top[1]) < margin:
            return False
        seq.append(t)
    return True


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_equals_the_plain_model(tiny_folders, name):
    cfg, w = plain.read_model(tiny_folders[name])
    prompts = [tiny.random_tokens(40 + i, n, cfg["vocab_size"]) for i, n in enumerate((5, 11, 17, 1, 40))]
    want = [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
    engine = engine_for(tiny_folders[name], "float32")
    out = engine.generate(prompts, 8, eos_token_id=[])
    assert out.token_ids == want
    assert out.finish_reason == ["length"] * 5 and len(out.decode_steps) == 7
    # bfloat16: equal wherever the plain model's choice is not a near tie
    # (the reference's generation rule, src/eval/generation.rs:132-176)
    got = engine_for(tiny_folders[name], "bfloat16").generate(prompts, 8, eos_token_id=[]).token_ids
    for p, g, t in zip(prompts, got, want):
        if g != t:
            k = next(i for i, (a, b) in enumerate(zip(g, t)) if a != b)
            row = plain.forward(cfg, w, list(p) + t[:k])[-1]
            assert float(row[t[k]] - row[g[k]]) < 0.05, (g, t)
    engine.cache.table.check()
    assert engine.cache.table.slots.held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_started_ahead_changes_no_token(tiny_folders, dtype):
    """`step_host(more=True)` starts the next step before it returns. Fed what
    it returned, the tokens are those of steps run one by one (bit for bit: the
    same kernels on the same inputs); fed something else, or with a row less,
    the step is taken back and the tokens are those of an engine that never
    ran ahead. Across a page boundary, sampled as well as greedy."""
    from foundry_b200 import SamplingParams
    from foundry_b200.engine import SequenceStep
    name = "tiny_b"
    cfg, _ = plain.read_model(tiny_folders[name])
    V = cfg["vocab_size"]
    prompts = [tiny.random_tokens(900 + i, n, V) for i, n in enumerate((61, 5, 33))]

    def run(ahead, sampling):
        engine = engine_for(tiny_folders[name], dtype)
        slots = [engine.open_sequence() for _ in prompts]
        tokens = engine.step_select([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)],
                                    sampling, [0, 1, 2], [0, 0, 0])
        session = engine.decode_session(slots, sampling, [0, 1, 2], [1, 1, 1])
        out, count = [tokens], 1
        for i in range(12):
            if i == 5:
                tokens = [(t + 1) % V for t in tokens]  # not what the step ahead was given
            tokens = session.step_host(tokens, more=ahead, counts=[count] * 3)
            assert session.has_ahead() == ahead
            out.append(tokens)
            count += 1
        # a row less: the engine's own session, through the loop's entry point
        session.cancel_ahead()
        lengths = [engine.cache.length(s) for s in slots]
        assert lengths == [len(p) + 12 for p in prompts]
        current = dict(enumerate(out[-1]))
        for rows in ([0, 1, 2], [0, 2], [0, 2], [2]):
            steps = [SequenceStep(slots[r], [current[r]], [0]) for r in rows]
            got = engine.step_select(steps, sampling, rows, [count] * len(rows), more=ahead)
            current.update(zip(rows, got))
            out.append(list(got))
            count += 1
        engine._settle()
        assert [engine.cache.length(s) for s in slots] == \
            [len(prompts[0]) + 15, len(prompts[1]) + 13, len(prompts[2]) + 16]
        # logits after steps ahead: the step function takes a matching step over,
        # or takes the guess back
        logits = engine.step([SequenceStep(slots[2], [3], [0])])
        for s in slots:
            engine.close_sequence(s)
        engine.cache.table.check()
        return out, logits.cpu()

    for sampling in (SamplingParams(), SamplingParams(temperature=0.9, seed=5)):
        plain_out, plain_logits = run(False, sampling)
        ahead_out, ahead_logits = run(True, sampling)
        assert ahead_out == plain_out
        assert torch.equal(ahead_logits, plain_logits)


def test_generation_ahead_with_stop_tokens_equals_the_plain_model(tiny_folders):
    """Rows end at different steps (a stop token that the loop cannot foresee,
    and lengths): each time the step that was started for all rows is taken
    back, and the survivors' tokens stay those of the plain model."""
    name = "tiny_a"
    cfg, w = plain.read_model(tiny_folders[name])
    prompts = [tiny.random_tokens(80 + i, n, cfg["vocab_size"]) for i, n in enumerate((9, 64, 3, 30))]
    free_run = [plain.greedy_generate(cfg, w, p, 12) for p in prompts]
    stops = [free_run[0][3], free_run[2][7]]
    want = [plain.greedy_generate(cfg, w, p, 12, eos=stops) for p in prompts]
    assert len({len(t) for t in want}) > 1  # rows do end at different steps
    engine = engine_for(tiny_folders[name], "float32")
    out = engine.generate(prompts, 12, eos_token_id=stops)
    assert out.token_ids == want
    assert engine.cache.table.slots.held == 0
    engine.cache.table.check()


def test_two_engines_on_two_streams_share_no_scratch(tiny_folders):
    """Kernels that pass partial results between their CTAs take their scratch
    from the engine that runs them: two engines working at the same time, each in
    a thread and on a stream of its own, generate what each generates alone."""
    import threading
    from foundry_b200.kernels import ops
    cfg, _ = plain.read_model(tiny_folders["tiny_b"])
    V = cfg["vocab_size"]
    prompts = [[tiny.random_tokens(300 + 7 * e + i, n, V) for i, n in enumerate((150, 9, 64))]
               for e in range(2)]
    engines = [engine_for(tiny_folders["tiny_b"], "bfloat16") for _ in range(2)]
    assert engines[0].scratch != engines[1].scratch
    alone = [e.generate(p, 24, eos_token_id=[]).token_ids for e, p in zip(engines, prompts)]
    with ops.scratch_owner(engines[0].scratch):
        a = ops._pair_scratch(torch.device("cuda:0"))[0]
    with ops.scratch_owner(engines[1].scratch):
        b = ops._pair_scratch(torch.device("cuda:0"))[0]
    assert a.data_ptr() != b.data_ptr()
    together, errors = [None, None], []

    def work(i):
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(3):
                    together[i] = engines[i].generate(prompts[i], 24, eos_token_id=[]).token_ids
                torch.cuda.current_stream().synchronize()
        except Exception as exc:  # surfaces in the main thread below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert together == alone
    key = engines[1].scratch
    del engines[1:]
    import gc
    gc.collect()
    assert not [k for k in ops._PAIR_SCRATCH if k[1] == key]  # an engine's scratch goes with it


def test_stop_tokens_early_rows_and_slot_reuse(tiny_folders):
    """Make a stop token of what the plain model generates third for one
    prompt: that row ends there (keeping the token) while the others go on,
    and later batches run in the slots and pages it gave back."""
    name = "tiny_b"
    cfg, w = plain.read_model(tiny_folders[name])
    prompts = [tiny.random_tokens(60 + i, n, cfg["vocab_size"]) for i, n in enumerate((7, 30, 3, 12, 9, 21))]
    free_run = [plain.greedy_generate(cfg, w, p, 10) for p in prompts]
    stop = free_run[0][2]
    want = [plain.greedy_generate(cfg, w, p, 10, eos=[stop]) for p in prompts]
    engine = engine_for(tiny_folders[name], "float32", max_slots=2, max_tokens=256)
    out = engine.generate(prompts, 10, eos_token_id=[stop])
    assert out.token_ids == want
    assert out.token_ids[0][-1] == stop and len(out.token_ids[0]) <= 3
    assert out.finish_reason[0] == "stop"
    assert out.batches == [[0, 1], [2, 3], [4, 5]]
    assert engine.cache.table.slots.held == 0
    engine.cache.table.check()
    # the config's own stop tokens apply when none are given
    assert engine_for(tiny_folders[name], "float32").generate(prompts[:1], 4).token_ids[0] == \
        plain.greedy_generate(cfg, w, prompts[0], 4, eos=cfg["eos_token_id"])


def test_temperature_sampling_is_the_host_restatement(tiny_folders):
    """Each sampled token is the argmax of logits / T + Gumbel noise, the noise
    being a function of (seed, request, count) only: recomputed here from the
    plain model's logits, and the same in another batching."""
    from foundry_b200 import SamplingParams
    name = "tiny_b"
    cfg, w = plain.read_model(tiny_folders[name])
    prompts = [tiny.random_tokens(80 + i, n, cfg["vocab_size"]) for i, n in enumerate((1, 7, 40, 90))]
    params = SamplingParams(temperature=0.8, seed=1234)
    engine = engine_for(tiny_folders[name], "float32")
    out = engine.generate(prompts, 16, eos_token_id=[], sampling=params)
    assert [len(r) for r in out.token_ids] == [16] * 4
    for r, (prompt, row) in enumerate(zip(prompts, out.token_ids)):
        seq = list(prompt)
        for count, token in enumerate(row):
            scores = plain.sample_scores(plain.forward(cfg, w, seq)[-1], 0.8, 1234, r, count)
            best = int(torch.argmax(scores))
            # equal, or a near tie of the two perturbed scores
            assert token == best or float(scores[best] - scores[token]) < 1e-3, (r, count)
            seq.append(token)
    assert len({tuple(r) for r in out.token_ids}) > 1
    one_by_one = engine_for(tiny_folders[name], "float32", max_slots=1).generate(
        prompts, 16, eos_token_id=[], sampling=params)
    assert one_by_one.token_ids == out.token_ids and len(one_by_one.batches) == 4
    other_seed = engine.generate(prompts, 16, eos_token_id=[],
                                 sampling=SamplingParams(temperature=0.8, seed=99))
    assert other_seed.token_ids != out.token_ids


def test_temperature_sampling_in_bfloat16(tiny_folders):
    """The 16-bit decode graph with temperature > 0 (random streams and counts
    uploaded every step). Its logits differ from the plain model's by 16-bit
    rounding, so a token is right when it is the plain model's choice or when
    the plain model scores it within that rounding of its choice; most tokens
    must be the plain choice itself. Checked along the engine's own sequence."""
    from foundry_b200 import SamplingParams
    name = "tiny_b"
    cfg, w = plain.read_model(tiny_folders[name])
    prompts = [tiny.random_tokens(80 + i, n, cfg["vocab_size"]) for i, n in enumerate((1, 7, 40, 90, 23))]
    temperature = 0.8
    params = SamplingParams(temperature=temperature, seed=4321)
    engine = engine_for(tiny_folders[name], "bfloat16")
    out = engine.generate(prompts, 16, eos_token_id=[], sampling=params)
    assert [len(r) for r in out.token_ids] == [16] * 5
    equal = total = 0
    for r, (prompt, row) in enumerate(zip(prompts, out.token_ids)):
        seq = list(prompt)
        for count, token in enumerate(row):
            logits = plain.forward(cfg, w, seq)[-1]
            scores = plain.sample_scores(logits, temperature, 4321, r, count)
            best = int(torch.argmax(scores))
            # the bound of `tiny.assert_logits_close` on a 16-bit logit, on both candidates
            slack = 2 * 1e-2 * max(1.0, float(logits.abs().max())) / temperature
            assert token == best or float(scores[best] - scores[token]) < slack, (r, count)
            equal += token == best
            total += 1
            seq.append(token)
    assert equal >= 0.9 * total, f"{equal} of {total} tokens are the plain model's choice"
    assert len({tuple(r) for r in out.token_ids}) > 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_ahead_of_the_device(tiny_folders, dtype):
    """The host may prepare steps faster than the device runs them: decode steps
    whose tokens stay on the device are queued without waiting, and so are
    portions of a prompt whose logits nobody asks for. Every step must still
    run with its own positions, lengths and page tables (the upload of a step's
    description is staged so that a later step cannot overwrite it). The device
    is kept busy first, so that everything below is queued before any of it runs."""
    from foundry_b200 import SamplingParams
    from foundry_b200.engine import SequenceStep
    name = "tiny_b"
    cfg, w = plain.read_model(tiny_folders[name])
    V = cfg["vocab_size"]
    prompts = [tiny.random_tokens(700 + i, n, V) for i, n in enumerate((60, 5, 33))]
    steps = 70  # across a page boundary for every sequence
    # with the host in every step
    engine = engine_for(tiny_folders[name], dtype)
    slots = [engine.open_sequence() for _ in prompts]
    first = engine.step_select([SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)],
                               SamplingParams(), [0, 1, 2], [0, 0, 0])
    session = engine.decode_session(slots)
    by_host, tokens = [first], first
    for _ in range(steps):
        tokens = session.step_host(tokens)
        by_host.append(tokens)
    for s in slots:
        engine.close_sequence(s)
    # the same, queued ahead
    engine = engine_for(tiny_folders[name], dtype)
    slots = [engine.open_sequence() for _ in prompts]
    engine.step([SequenceStep(s, p, []) for s, p in zip(slots, prompts)])
    session = engine.decode_session(slots)
    session.set_tokens(first)
    session.step()  # the first call of a bucket runs plainly and captures
    torch.cuda.synchronize()
    record = torch.zeros((steps, len(slots)), dtype=torch.int32, device="cuda:0")
    record[0].copy_(session.runner.next_tokens[:len(slots)])
    torch.cuda._sleep(400_000_000)  # a fifth of a second: the host gets far ahead
    for i in range(1, steps):
        session.step()
        record[i].copy_(session.runner.next_tokens[:len(slots)])
    queued = record.cpu().tolist()
    assert queued == by_host[1:]
    if dtype == "float32":  # and both are the plain model's greedy tokens
        for i, p in enumerate(prompts):
            want = plain.greedy_generate(cfg, w, p, 12)
            assert [first[i]] + [row[i] for row in queued[:11]] == want
    for s in slots:
        engine.close_sequence(s)
    # a prompt in ten portions of one bucket, none of them waited for
    tokens = tiny.random_tokens(77, 101, V)
    want = plain.forward(cfg, w, tokens).numpy()[-1:]
    slot = engine.open_sequence()
    engine.step([SequenceStep(slot, tokens[:10], [])])  # captures the bucket's graph
    torch.cuda.synchronize()
    torch.cuda._sleep(400_000_000)
    for at in range(10, 100, 10):
        engine.step([SequenceStep(slot, tokens[at:at + 10], [])])
    got = engine.step([SequenceStep(slot, tokens[100:], [0])]).cpu().numpy()
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 5e-2) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_model(tiny_folders, dtype):
    """200 single-token steps after a short prompt, across several page
    boundaries and graph re-captures: every step's logits are checked."""
    from foundry_b200.engine import SequenceStep
    name = "tiny_b"
    cfg, w = plain.read_model(tiny_folders[name])
    tokens = tiny.random_tokens(5, 230, cfg["vocab_size"])
    want = plain.forward(cfg, w, tokens).numpy()
    engine = engine_for(tiny_folders[name], dtype)
    slot = engine.open_sequence()
    rows = [engine.step([SequenceStep(slot, tokens[:30], list(range(30)))]).cpu().numpy()]
    for t in tokens[30:]:
        rows.append(engine.step([SequenceStep(slot, [t], [0])]).cpu().numpy())
    engine.close_sequence(slot)
    tiny.assert_logits_close(np.concatenate(rows), want, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(tiny_folders, dtype):
    """Position 0 and its neighbours, started in every way: a one-token prompt,
    then tokens one by one; two tokens then one; and the same in a slot that a
    longer sequence used before (stale keys behind the new length)."""
    from foundry_b200.engine import SequenceStep
    name = "tiny_a"
    cfg, w = plain.read_model(tiny_folders[name])
    tokens = tiny.random_tokens(9, 6, cfg["vocab_size"])
    want = plain.forward(cfg, w, tokens).numpy()
    engine = engine_for(tiny_folders[name], dtype, max_slots=1, max_tokens=128)
    for cuts in ([1, 1, 1, 1, 1, 1], [2, 1, 3], [6], [1, 5]):
        stale = engine.open_sequence()  # fill the only slot's pages with other keys
        engine.step([SequenceStep(stale, tiny.random_tokens(3, 100, cfg["vocab_size"]), [])])
        engine.close_sequence(stale)
        slot = engine.open_sequence()
        assert slot == stale
        rows, at = [], 0
        for n in cuts:
            rows.append(engine.step([SequenceStep(slot, tokens[at:at + n], list(range(n)))]).cpu().numpy())
            at += n
        engine.close_sequence(slot)
        tiny.assert_logits_close(np.concatenate(rows), want, dtype, f"cuts {cuts}")


def test_padding_changes_no_result(tiny_folders):
    """Three live sequences run in a four-row graph; the same three sequences
    beside a fourth give the same logits row for row."""
    from foundry_b200.engine import SequenceStep
    name = "tiny_b"
    cfg, _ = plain.read_model(tiny_folders[name])
    engine = engine_for(tiny_folders[name], "float32")
    prompts = [tiny.random_tokens(20 + i, n, cfg["vocab_size"]) for i, n in enumerate((9, 33, 64, 5))]

    def run(count):
        slots = [engine.open_sequence() for _ in range(count)]
        engine.step([SequenceStep(s, p, []) for s, p in zip(slots, prompts)])
        out = [engine.step([SequenceStep(s, [7 + i], [0]) for s in slots]).cpu().numpy()
               for i in range(3)]
        for s in slots:
            engine.close_sequence(s)
        return np.stack(out)

    three, four = run(3), run(4)
    assert np.array_equal(three, four[:, :3])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_replayed_equal_plain_launches(tiny_folders, dtype):
    """Prompt steps of up to 512 tokens run as replayed graphs over padded
    buckets. The same steps launched plainly give the same logits bit for bit:
    one bucket used three times with other lengths, sequence counts and wanted
    places (the second and third use replay the graph of the first), a
    continued prompt, a step that wants nothing, and the decode steps after."""
    from foundry_b200.engine import SequenceStep
    from foundry_b200.engine import prompt as prompt_graphs
    name = "tiny_b"
    cfg, _ = plain.read_model(tiny_folders[name])
    V = cfg["vocab_size"]
    rounds = [[(60, [0, 59]), (40, [39])],            # 100 tokens -> bucket (128, 2, 8, 4)
              [(90, [89, 1, 2]), (20, [19])],          # the same bucket, other cuts
              [(70, [69]), (30, [0, 29, 5])],
              [(5, [4])],                              # a small bucket
              [(16, []), (3, [])],                     # nothing wanted
              [(64, [63]), (64, [0]), (1, [0])],       # 129 tokens -> the 256-token bucket
              [(240, [239]), (240, [0, 239]), (40, [39])]]  # 520 tokens: launched plainly in both
    results = []
    for graphs in (True, False):
        engine = engine_for(tiny_folders[name], dtype, max_slots=4, max_tokens=1024)
        engine.use_graphs = graphs
        out = []
        for r, round_ in enumerate(rounds):
            slots = [engine.open_sequence() for _ in round_]
            prompts = [tiny.random_tokens(100 * r + i, n, V) for i, (n, _) in enumerate(round_)]
            out.append(engine.step([SequenceStep(s, p, w) for s, p, (_, w) in
                                    zip(slots, prompts, round_)]).cpu())
            # the prompts go on: 7 more tokens each, then two single tokens
            more = [tiny.random_tokens(100 * r + 50 + i, 7, V) for i in range(len(slots))]
            out.append(engine.step([SequenceStep(s, m, [6]) for s, m in zip(slots, more)]).cpu())
            for t in range(2):
                out.append(engine.step([SequenceStep(s, [11 + t], [0]) for s in slots]).cpu())
            for s in slots:
                engine.close_sequence(s)
        if graphs:
            keys = set(engine._prompts._runners)
            # rounds 2 and 3 replayed one graph; the seven-token steps of all rounds share theirs
            assert {(128, 2, 8, 4, True), (128, 2, 8, 4, False)} <= keys and len(keys) <= 9, keys
            assert any(k[0] == 256 for k in keys), keys
        results.append(out)
    assert prompt_graphs.PROMPT_GRAPH_TOKENS == 512
    for a, b in zip(*results):
        assert a.shape == b.shape and torch.equal(a, b)


def test_a_kernel_that_gave_up_is_an_error_of_the_call(tiny_folders, monkeypatch):
    """No logits or tokens leave the engine once a kernel has recorded that a
    bounded wait ran out. The record is a stand-in here (no wait is made to run
    out on the GPU): each entry point must look at it after it synchronised."""
    import ctypes
    from foundry_b200.engine import SequenceStep
    from foundry_b200.kernels import ops
    engine = engine_for(tiny_folders["tiny_a"], "bfloat16")
    fake = (ctypes.c_int * 4)()
    monkeypatch.setattr(ops, "_MIRROR", [fake])

    def fail():
        fake[0], fake[1], fake[2], fake[3] = 1, 2, 3, 4

    slot = engine.open_sequence()
    engine.step([SequenceStep(slot, [1, 2, 3], [2])])  # nothing recorded: fine
    fail()
    with pytest.raises(ops.KernelError, match="bounded wait"):
        engine.step([SequenceStep(slot, [4, 5], [1])])
    engine.step([SequenceStep(slot, [6], [0])])  # the record was cleared with the report
    fail()
    with pytest.raises(ops.KernelError, match="bounded wait"):
        engine.step([SequenceStep(slot, [7], [0])])
    session = engine.decode_session([slot])
    fail()
    with pytest.raises(ops.KernelError, match="bounded wait"):
        session.step_host([8])
    engine.close_sequence(slot)
    fail()
    with pytest.raises(ops.KernelError, match="bounded wait"):
        engine.generate([[1, 2, 3]], 4, eos_token_id=[])
    assert engine.cache.table.slots.held == 0  # the loop gave its slots back
    assert engine.generate([[1, 2, 3]], 4, eos_token_id=[]).token_ids[0]


def test_refusals_of_the_step_function(tiny_folders):
    from foundry_b200.cache import CacheFull
    from foundry_b200.engine import SequenceStep
    engine = engine_for(tiny_folders["tiny_a"], "float32", max_slots=2, max_tokens=128)
    slot = engine.open_sequence()
    with pytest.raises(ValueError, match="vocabulary"):
        engine.step([SequenceStep(slot, [256], [0])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([SequenceStep(slot, [1], [0]), SequenceStep(slot, [2], [0])])
    with pytest.raises(ValueError, match="not open"):
        engine.step([SequenceStep(1, [1, 2], [0])])
    with pytest.raises(ValueError, match="no token"):
        engine.step([SequenceStep(slot, [], [])])
    with pytest.raises(ValueError, match="wanted place"):
        engine.step([SequenceStep(slot, [1, 2], [2])])
    with pytest.raises(ValueError, match="positions"):
        engine.step([SequenceStep(slot, [1] * 129, [])])
    other = engine.open_sequence()
    engine.step([SequenceStep(slot, [1] * 65, [])])
    with pytest.raises(CacheFull):
        engine.step([SequenceStep(other, [1] * 65, [])])  # 2 pages held, 2 more wanted of 2
    assert engine.cache.length(other) == 0 and engine.cache.length(slot) == 65  # nothing changed
    engine.cache.table.check()


def test_command_line_run(tiny_folders):
    cfg, w = plain.read_model(tiny_folders["tiny_a"])
    prompt = [5, 17, 3, 200]
    want = plain.greedy_generate(cfg, w, prompt, 6, eos=[cfg["eos_token_id"]])
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", "--model",
                           tiny_folders["tiny_a"], "--prompt-ids", "5,17,3,200", "--max-new-tokens",
                           "6", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert json.loads(proc.stdout.strip()) == want
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", "--model",
                           tiny_folders["tiny_a"], "--prompt-ids", "5,999", "--max-new-tokens", "2"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "vocabulary" in proc.stderr


def test_command_line_bench_writes_a_report(tiny_folders, tmp_path):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--model",
                           tiny_folders["tiny_b"], "--prompt-tokens", "20", "--new-tokens", "5",
                           "--runs", "2", "--batch-size", "3", "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    assert report["config"]["prompt_tokens"] == 20 and len(report["runs"]) == 2
    assert len(report["prompt_ids"]) == 3 and len(report["prompt_ids"][0]) == 20
    assert len(report["runs"][0]["decode_step_ns"]) == 4  # new tokens count the prompt step's
    assert all(len(r) == 5 for r in report["runs"][0]["token_ids"])
    assert report["runs"][0]["token_ids"] == report["runs"][1]["token_ids"]
    assert report["metrics"]["decode_tokens_per_s"]["count"] == 2
    assert report["metadata"]["model_parameter_count"] > 0


def test_command_line_with_a_named_configuration_and_random_weights(tmp_path):
    """`--config NAME --random-weights SEED` stands in for a folder in both
    subcommands; the tokens are those of the same engine built in this process,
    and the report holds the step's bytes and operations with their fractions."""
    import foundry_b200 as fb
    from foundry_b200.bench.presets import preset
    want = fb.Engine.from_random(preset("tiny-a"), 3, dtype="float32", max_tokens=256,
                                 max_slots=2).generate([[5, 17, 3], [9]], 5, eos_token_id=[])
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", "--config",
                           "tiny-a", "--random-weights", "3", "--prompt-ids", "5,17,3",
                           "--prompt-ids", "9", "--max-new-tokens", "5", "--dtype", "float32",
                           "--ignore-eos", "--max-seq-len", "100"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [json.loads(line) for line in proc.stdout.split()] == want.token_ids
    for bad in (["--config", "tiny-a"], ["--config", "no-such", "--random-weights", "1"],
                ["--model", "x", "--config", "tiny-a", "--random-weights", "1"]):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", *bad,
                               "--prompt-ids", "1", "--max-new-tokens", "1"],
                              capture_output=True, text=True, timeout=600)
        assert proc.returncode != 0 and "Traceback" not in proc.stderr, proc.stderr[-500:]
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0}))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--config",
                           "tiny-b", "--random-weights", "1", "--prompt-tokens", "40",
                           "--new-tokens", "4", "--runs", "2", "--batch-size", "2", "--context",
                           "128", "--peaks", str(peaks), "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    decode, prompt = report["decode_step_model"], report["prompt_step_model"]
    assert decode["peaks"] == "measured" and decode["peak_gb_per_s"] == 6000.0
    assert decode["bytes_read"] > 0 and 0 < decode["fraction_of_peak"] < 1
    assert abs(decode["fraction_of_peak"] - decode["achieved_gb_per_s"] / 6000.0) < 1e-9
    assert prompt["flops"] > 0 and 0 < prompt["fraction_of_peak"] < 1
    assert report["metadata"]["model_parameter_count"] == 457824 + 0 or \
        report["metadata"]["model_parameter_count"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_a_page_table_growth(tmp_path, dtype):
    """A sequence that grows from 8 to 9 pages while another stays short: the
    decode graph is re-captured with a wider page table in the middle of the
    run, and a far key (position 3) must still be found from position 530."""
    import foundry_b200 as fb
    from foundry_b200.config import LlamaConfig
    from foundry_b200.engine import SequenceStep
    cfg_doc = {**tiny.CONFIGS["tiny_a"], "max_position_embeddings": 1024}
    folder = fb.write_model_folder(str(tmp_path / "long"), LlamaConfig.parse(cfg_doc), 3, std=tiny.STD)
    cfg, w = plain.read_model(folder)
    long_tokens = tiny.random_tokens(1, 540, cfg["vocab_size"])
    short_tokens = tiny.random_tokens(2, 60, cfg["vocab_size"])
    want_long = plain.forward(cfg, w, long_tokens).numpy()
    want_short = plain.forward(cfg, w, short_tokens).numpy()
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_slots=2)
    a, b = engine.open_sequence(), engine.open_sequence()
    engine.step([SequenceStep(a, long_tokens[:500], []), SequenceStep(b, short_tokens[:20], [])])
    rows_a, rows_b = [], []
    for i in range(40):
        out = engine.step([SequenceStep(a, [long_tokens[500 + i]], [0]),
                           SequenceStep(b, [short_tokens[20 + i]], [0])]).cpu().numpy()
        rows_a.append(out[0:1])
        rows_b.append(out[1:2])
    assert engine._session.runner.width == 16 and \
        any(key[:2] == (2, 8) for key in engine._runners)  # both graphs were used
    tiny.assert_logits_close(np.concatenate(rows_a), want_long[500:540], dtype, "long sequence")
    tiny.assert_logits_close(np.concatenate(rows_b), want_short[20:60], dtype, "short sequence")
