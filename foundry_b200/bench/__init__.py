"""Measurement in the reference's manner: seeded token ids, warm-up, runs,
per-run rates and their summaries (src/bench/)."""
from .rng import SplitMix64, token_rows
from .runner import BenchConfig, run_bench
from .stats import Summary, summarize

__all__ = ["SplitMix64", "token_rows", "BenchConfig", "run_bench", "Summary", "summarize"]
