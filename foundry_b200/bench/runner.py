"""`foundry bench`: prompt processing and decoding on random token ids.

Follows src/bench/mod.rs:146-371. A run starts from an empty cache, optionally
fills `depth` tokens (untimed), processes the prompt in one step (its output is
new token 1), then decodes one token per step. `new_tokens` counts the prompt
step's token; with `prompt_tokens == 0` decoding starts from random ids.
Timing scope `forward` stops the clock when the logits exist (device
synchronised); `generation` (default) when the chosen token is on the host.
Rates per run: prompt tokens/s = batch x prompt / prompt step time; decode
tokens/s = batch x steps / sum of step times (tools/reference/README.md:83-102).
"""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass
from typing import Dict, Optional

import torch

from ..engine.context import SequenceStep
from ..kernels import ops
from ..sampling import SamplingParams
from .costs import decode_step_bytes, load_peaks, roofline, step_flops
from .rng import SplitMix64, token_rows
from .stats import summarize


@dataclass(frozen=True)
class BenchConfig:
    prompt_tokens: int
    new_tokens: int
    timing_scope: str = "generation"  # or "forward"
    depth: int = 0
    warmup_runs: int = 1
    warmup_ms: int = 0
    runs: int = 10
    batch_size: int = 1
    seed: int = 0
    profile: Optional[str] = None  # "steps" | "kernels" (src/nn/profile.rs:7-13)

    def decode_step_count(self) -> int:
        # src/bench/mod.rs:72-77
        return max(0, self.new_tokens - (1 if self.prompt_tokens > 0 else 0))


def _one_run(engine, cfg: BenchConfig, depth_ids, prompt_ids, start_ids) -> Dict:
    greedy = SamplingParams()
    slots = [engine.open_sequence() for _ in range(cfg.batch_size)]
    sample: Dict = {"prompt_step_ns": None, "decode_step_ns": [], "token_ids": [[] for _ in slots]}
    try:
        torch.cuda.synchronize()
        if cfg.depth:
            engine.step([SequenceStep(s, ids, []) for s, ids in zip(slots, depth_ids)])
            torch.cuda.synchronize()

        def timed(steps):
            if cfg.profile:
                ops.PROFILER.take()
            started = time.perf_counter_ns()
            logits = engine.step(steps)
            if cfg.timing_scope == "forward":
                torch.cuda.synchronize()
                elapsed = time.perf_counter_ns() - started
                tokens = engine.sampler.select(logits, greedy).tolist()
            else:
                tokens = engine.sampler.select(logits, greedy).tolist()
                elapsed = time.perf_counter_ns() - started
            return tokens, elapsed

        run_started = time.perf_counter_ns()
        if cfg.prompt_tokens:
            tokens, ns = timed([SequenceStep(s, ids, [len(ids) - 1])
                                for s, ids in zip(slots, prompt_ids)])
            sample["prompt_step_ns"] = ns
            sample["first_token_ns"] = time.perf_counter_ns() - run_started
            if cfg.profile:
                sample["prompt_profile"] = ops.PROFILER.take()
            for row, t in zip(sample["token_ids"], tokens):
                row.append(t)
        else:
            tokens = list(start_ids)
        for _ in range(cfg.decode_step_count()):
            tokens, ns = timed([SequenceStep(s, [t], [0]) for s, t in zip(slots, tokens)])
            sample["decode_step_ns"].append(ns)
            if cfg.profile:
                sample.setdefault("decode_profiles", []).append(ops.PROFILER.take())
            for row, t in zip(sample["token_ids"], tokens):
                row.append(t)
        sample["generation_ns"] = time.perf_counter_ns() - run_started
    finally:
        for s in slots:
            engine.close_sequence(s)
    return sample


def run_bench(engine, cfg: BenchConfig, peaks: Optional[Dict] = None) -> Dict:
    if cfg.prompt_tokens == 0 and cfg.new_tokens == 0:
        raise ValueError("nothing to measure: prompt_tokens and new_tokens are both 0")
    vocab = engine.spec.vocab_size
    ops.PROFILER.start(cfg.profile)
    if cfg.profile == "kernels":
        engine.use_graphs = False  # per-kernel times need one launch at a time
    rng = SplitMix64(cfg.seed)
    depth_ids = token_rows(rng, cfg.batch_size, cfg.depth, vocab)
    prompt_ids = token_rows(rng, cfg.batch_size, cfg.prompt_tokens, vocab)
    start_ids = token_rows(rng, 1, cfg.batch_size, vocab)[0] if cfg.prompt_tokens == 0 else None
    warm_started, warm_runs = time.perf_counter(), 0
    while warm_runs < cfg.warmup_runs or (time.perf_counter() - warm_started) * 1e3 < cfg.warmup_ms:
        _one_run(engine, cfg, depth_ids, prompt_ids, start_ids)
        warm_runs += 1
    torch.cuda.reset_peak_memory_stats()
    runs = [_one_run(engine, cfg, depth_ids, prompt_ids, start_ids) for _ in range(cfg.runs)]
    prompt_rates = [cfg.batch_size * cfg.prompt_tokens / (r["prompt_step_ns"] * 1e-9)
                    for r in runs if r["prompt_step_ns"]]
    decode_rates = [cfg.batch_size * len(r["decode_step_ns"]) / (sum(r["decode_step_ns"]) * 1e-9)
                    for r in runs if r["decode_step_ns"]]
    output_rates = [cfg.batch_size * cfg.new_tokens / (r["generation_ns"] * 1e-9) for r in runs
                    if cfg.new_tokens]

    def js(values):
        s = summarize(values)
        return None if s is None else s.to_json()

    ops.PROFILER.start(None)
    decode_profiles = [p for r in runs for p in r.get("decode_profiles", [])]

    def per_step(field):
        return [sum(k.get(field, 0) for k in p["kernels"].values()) for p in decode_profiles]

    profile_metrics = {}
    if decode_profiles:
        profile_metrics = {
            "decode_dispatch_count": js(per_step("dispatch_count")),
            "decode_allocation_count": js([p["allocation_count"] for p in decode_profiles]),
            "decode_allocated_bytes": js([p["allocated_bytes"] for p in decode_profiles]),
        }
        if cfg.profile == "kernels":
            profile_metrics["decode_gpu_busy_ns"] = js([p["gpu_busy_ns"] for p in decode_profiles])
    # what the steps have to move and to compute, and the share of the hardware's
    # rates they reached (the mean step of all runs)
    peaks = peaks or load_peaks()
    decode_ns = [ns for r in runs for ns in r["decode_step_ns"]]
    prompt_ns = [r["prompt_step_ns"] for r in runs if r["prompt_step_ns"]]
    context = [cfg.depth + cfg.prompt_tokens + cfg.decode_step_count() / 2.0] * cfg.batch_size
    step_bytes = decode_step_bytes(engine, context)
    decode_model = {"bytes_read": step_bytes, "achieved_gb_per_s": None, "peak_gb_per_s":
                    peaks["hbm_gbs"], "fraction_of_peak": None, "peaks": peaks["source"]}
    if decode_ns:
        line = roofline(step_bytes, summarize(decode_ns).mean * 1e-9, peaks["hbm_gbs"], "GB/s")
        decode_model.update(achieved_gb_per_s=line["achieved"], fraction_of_peak=line["frac"])
    prompt_model = None
    if cfg.prompt_tokens:
        flops = step_flops(engine.model, [cfg.prompt_tokens] * cfg.batch_size,
                           [cfg.depth] * cfg.batch_size, wanted_rows=cfg.batch_size)
        prompt_model = {"flops": flops, "achieved_tflop_per_s": None, "peak_tflop_per_s":
                        peaks["bf16_tflops"], "fraction_of_peak": None, "peaks": peaks["source"]}
        if prompt_ns:
            line = roofline(flops, summarize(prompt_ns).mean * 1e-9, peaks["bf16_tflops"], "TFLOP/s")
            prompt_model.update(achieved_tflop_per_s=line["achieved"], fraction_of_peak=line["frac"])
    return {
        "config": asdict(cfg),
        "depth_ids": depth_ids, "prompt_ids": prompt_ids, "start_ids": start_ids,
        "warmup_run_count": warm_runs,
        "runs": runs,
        "metrics": {
            "prompt_step_ns": js([r["prompt_step_ns"] for r in runs if r["prompt_step_ns"]]),
            "decode_step_ns": js([ns for r in runs for ns in r["decode_step_ns"]]),
            "generation_ns": js([r["generation_ns"] for r in runs]),
            "prompt_tokens_per_s": js(prompt_rates),
            "decode_tokens_per_s": js(decode_rates),
            "output_tokens_per_s": js(output_rates),
            **profile_metrics,
        },
        "decode_step_model": decode_model,
        "prompt_step_model": prompt_model,
        "peak_memory_bytes": torch.cuda.max_memory_allocated(),
        "peak_memory_source": "torch.cuda.max_memory_allocated",
    }
