"""Host-side measurement helpers against the reference's pinned values."""
from foundry_b200.bench import BenchConfig, SplitMix64, summarize, token_rows


def test_splitmix64_first_outputs_of_seed_0():
    # src/bench/rng.rs:52-62
    rng = SplitMix64(0)
    assert [rng.next_u64() for _ in range(3)] == [
        0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_below_is_uniform_over_the_bound_and_one_gives_zero():
    rng = SplitMix64(3)
    assert [rng.below(1) for _ in range(4)] == [0, 0, 0, 0]  # src/bench/rng.rs:65-73
    rng = SplitMix64(7)
    draws = [rng.below(10) for _ in range(2000)]
    assert set(draws) == set(range(10))
    rows = token_rows(SplitMix64(0), 2, 5, 128256)
    assert len(rows) == 2 and all(0 <= t < 128256 for r in rows for t in r)
    assert rows == token_rows(SplitMix64(0), 2, 5, 128256)


def test_summary_statistics():
    # percentiles interpolate linearly between ranks (src/bench/stats.rs:60-101)
    s = summarize([1.0, 2.0, 3.0, 4.0])
    assert s.count == 4 and s.mean == 2.5 and s.min == 1.0 and s.max == 4.0
    assert s.p50 == 2.5 and abs(s.p25 - 1.75) < 1e-12 and abs(s.p90 - 3.7) < 1e-12
    assert abs(s.variance - 5.0 / 3.0) < 1e-12  # sample variance, n - 1
    assert summarize([]) is None and summarize([5.0]).stdev == 0.0


def test_new_tokens_count_the_prompt_steps_token():
    # src/bench/mod.rs:72-77
    assert BenchConfig(512, 128).decode_step_count() == 127
    assert BenchConfig(0, 128).decode_step_count() == 128
    assert BenchConfig(512, 0).decode_step_count() == 0
