#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.2-3B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences. The model has the layer
sizes of the 3B benchmark configuration with random bfloat16 weights; the
cache is sized for 4,096 tokens per sequence, and the timed steps run at a
mean context of 3,072 tokens, the mean of decoding from 2,048 to 4,096.
One JSON line is printed:

  value     decoded tokens per second, timed on the device with CUDA events:
            after the warm-up steps, BLOCKS blocks of --steps steps each are
            timed one after another and the median block is reported (`steps`
            and `ms_per_step` describe one block); a step reads 6.4 GB of
            weights, far more than the 126 MB L2, so no L2 flush is needed
  e2e       the same through the Python entry point: token ids go in from
            pinned host memory and come back to the host every step
  prefill   one 2,048-token prompt in one step: tokens/s and the fraction of
            the bf16 tensor-core peak its FLOPs reach
  roofline  the decode step's bytes (every weight once, the live sequences'
            cache) / time, against the measured copy bandwidth
  points    decode tokens/s at batch 1 and 64, and the two other benchmark
            configurations with their own workloads and rooflines:
            llama_1b (16 layers; 32 prompts of 1..4096 tokens prefilled in one
            step, 512 steps at temperature 1, context 8192) and llama_8b
            (32 layers, separate head; 16 prompts of 1..8192 tokens, 256
            greedy steps, context 16384)

For --gpus N > 1 one line says that the library is single-GPU, exit code 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_DECODE_B1 = 6.92  # tok/s, Apple M4 Pro (the reference's report.json)
PUBLISHED_PREFILL_512 = 132.6

BLOCKS = 5  # timed blocks of --steps decode steps; the median one is reported
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, sustained, source)."""
    from foundry_b200.bench.costs import load_peaks
    got = load_peaks(os.path.join(ROOT, "MEASURED_PEAKS.json"))
    return got["hbm_gbs"], got["bf16_tflops"], got["bf16_tflops_sustained"], got["source"]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, reasons, sm_max = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            try:
                clocks.append(int(row[0]))
                sm_max = int(row[1])
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": sm_max,
                "reasons": sorted(reasons), "samples": len(clocks)}


def fill(engine, batch: int, length: int, seed: int, chunk_tokens: int = 8192):
    """Open `batch` sequences and run `length` random tokens into each cache."""
    from foundry_b200.bench import SplitMix64, token_rows
    from foundry_b200.engine import SequenceStep
    rows = token_rows(SplitMix64(seed), batch, length, 128000)
    slots = [engine.open_sequence() for _ in range(batch)]
    per = max(1, chunk_tokens // batch)
    for start in range(0, length, per):
        engine.step([SequenceStep(s, r[start:start + per], []) for s, r in zip(slots, rows)])
    return slots


def median_block(blocks):
    """The block of median duration among (ms per step, ...) tuples."""
    return sorted(blocks, key=lambda blk: blk[0])[len(blocks) // 2]


def time_decode(engine, slots, steps: int, warmup: int, blocks: int, sampler=None, sampling=None):
    """Device-timed decode steps (tokens stay on the device): `blocks` blocks
    of `steps` steps, each bracketed by CUDA events on the launching stream.
    Returns [(ms per step, mean context lengths of the block)], the launches of
    one block, the clock record."""
    import torch
    from foundry_b200.kernels import ops
    session = engine.decode_session(slots, sampling) if sampling else engine.decode_session(slots)
    session.set_tokens([1] * len(slots))
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    out, launches = [], 0
    for _ in range(blocks):
        before = [engine.cache.length(s) for s in slots]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.launch_count()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            session.step()
        end.record()
        torch.cuda.synchronize()
        launches = ops.launch_count() - launches0
        out.append((start.elapsed_time(end) / steps, [c + steps / 2.0 for c in before]))
    clocks = sampler.stop() if sampler else None
    ops.raise_on_device_failure()
    return out, launches, clocks


def time_e2e(engine, slots, steps: int, warmup: int, blocks: int):
    """The public call a user makes for one decode step: host token ids in
    (from pinned memory), host token ids out, every step; as the generation
    loop calls it, saying that it will come back with the tokens it receives
    (the step after is then started before this one's tokens are handed out;
    not after a block's last step, so that a block runs exactly `steps`).
    Host clock, median block."""
    import torch
    session = engine.decode_session(slots)
    tokens = [1] * len(slots)
    for _ in range(warmup):
        tokens = session.step_host(tokens)
    out = []
    for _ in range(blocks):
        torch.cuda.synchronize()
        started = time.perf_counter()
        for i in range(steps):
            tokens = session.step_host(tokens, more=i + 1 < steps)
        torch.cuda.synchronize()
        out.append(((time.perf_counter() - started) / steps,))
    return median_block(out)[0], session.h2d_bytes_per_step, session.d2h_bytes_per_step


def ragged_lengths(seed: int, count: int, longest: int):
    """`count` prompt lengths uniform in [1, longest] from SplitMix64(seed)."""
    from foundry_b200.bench import SplitMix64
    rng = SplitMix64(seed)
    return [1 + rng.below(longest) for _ in range(count)]


def workload_point(name: str, preset_name: str, prompts: int, longest: int, seed: int,
                   decode_steps: int, temperature: float, context: int, layers: int = 0) -> dict:
    """One of the other benchmark configurations with its own workload:
    `prompts` prompts of unequal lengths prefilled in ONE step (timed on the
    device, after one untimed run of the same step), then `decode_steps`
    single-token steps of all of them (greedy, or sampled at `temperature`),
    with the decode step's bytes (weights once + the live cache at the middle
    of the run) against the measured copy bandwidth and the prompt step's
    operations against the measured tensor-core rate."""
    import torch
    from foundry_b200 import SamplingParams
    from foundry_b200.bench import SplitMix64, token_rows
    from foundry_b200.bench.costs import decode_step_bytes, step_flops
    from foundry_b200.bench.presets import preset
    from foundry_b200.config import resolve_architecture
    from foundry_b200.engine import Engine, SequenceStep
    doc = preset(preset_name)
    full_layers = doc["num_hidden_layers"]
    if layers:
        doc["num_hidden_layers"] = layers
    cfg = resolve_architecture(doc).parse_config(doc)
    hbm_gbs, tflops_burst, _, source = peaks()
    engine = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=prompts * context,
                                max_slots=prompts, norm_std=0.0)
    lengths = ragged_lengths(seed, prompts, longest)
    rng = SplitMix64(seed + 1000)
    rows = [token_rows(rng, 1, n, 128000)[0] for n in lengths]
    prefill_ms = None
    for timed in (False, True):
        slots = [engine.open_sequence() for _ in rows]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([SequenceStep(s, r, [len(r) - 1]) for s, r in zip(slots, rows)])
        b.record()
        torch.cuda.synchronize()
        prefill_ms = a.elapsed_time(b)
        if not timed:
            for s in slots:
                engine.close_sequence(s)
    flops = step_flops(engine.model, lengths, wanted_rows=prompts)
    sampling = SamplingParams(temperature, seed) if temperature > 0 else None
    # the run in three timed blocks; the median block is reported, as for the main metric
    # (without noise that is the middle third of the run, at the run's mean context)
    per_block = max(1, decode_steps // 3)
    blocks, launches, _ = time_decode(engine, slots, per_block, 3, 3, sampling=sampling)
    ms, mean_ctx = median_block(blocks)
    step_bytes = decode_step_bytes(engine, mean_ctx)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    for s in slots:
        engine.close_sequence(s)
    del engine
    torch.cuda.empty_cache()
    tokens = sum(lengths)
    return {
        "model": preset_name, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
        "prompts": prompts, "prompt_tokens": tokens, "context": context,
        "decode_steps": 3 * per_block, "temperature": temperature,
        "prefill": {"value": tokens / (prefill_ms * 1e-3), "tokens": tokens, "ms": prefill_ms,
                    "flops": flops, "frac": flops / (prefill_ms * 1e-3) / (tflops_burst * 1e12)},
        "decode": {"value": prompts / (ms * 1e-3), "ms_per_step": ms, "gpu_launches": launches,
                   "mean_context": sum(mean_ctx) / len(mean_ctx),
                   "block_ms_per_step": [round(b[0], 4) for b in blocks]},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": achieved / hbm_gbs, "bytes_per_step": step_bytes, "of": source},
    }


def run(args) -> dict:
    import torch
    from foundry_b200.bench import SplitMix64, token_rows
    from foundry_b200.bench.costs import decode_step_bytes, step_flops
    from foundry_b200.bench.presets import preset
    from foundry_b200.config import resolve_architecture
    from foundry_b200.engine import Engine, SequenceStep

    doc = preset("llama-3.2-3b")
    full_layers = doc["num_hidden_layers"]
    layers = args.layers or full_layers
    doc["num_hidden_layers"] = layers
    cfg = resolve_architecture(doc).parse_config(doc)
    hbm_gbs, tflops_burst, tflops_sustained, source = peaks()
    batch = args.batch
    max_batch = max(batch, 64 if not args.skip_points else batch)
    engine = Engine.from_random(cfg, seed=0, dtype="bfloat16",
                                max_tokens=max_batch * CONTEXT, max_slots=max_batch, norm_std=0.0)
    engine.use_graphs = not args.no_graphs

    # ---------------------------------------------------------------- prefill
    prompt = token_rows(SplitMix64(1), 1, PREFILL_TOKENS, 128000)[0]
    prefill_ms = []
    for it in range(3 + 5):  # three warm-up runs, the median of five
        slot = engine.open_sequence()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([SequenceStep(slot, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        engine.close_sequence(slot)
        if it >= 3:
            prefill_ms.append(a.elapsed_time(b))
    p_ms = sorted(prefill_ms)[len(prefill_ms) // 2]
    p_flops = step_flops(engine.model, [PREFILL_TOKENS])
    prefill = {"value": PREFILL_TOKENS / (p_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": p_ms,
               "frac": p_flops / (p_ms * 1e-3) / (tflops_burst * 1e12), "flops": p_flops,
               "peak_tflops": tflops_burst,
               # beside the burst peak (a product alone on a cool chip): the rate the same
               # library product holds in a seconds-long loop under the power cap
               "frac_of_sustained": p_flops / (p_ms * 1e-3) / (tflops_sustained * 1e12),
               "peak_tflops_sustained": tflops_sustained}

    # ----------------------------------------------------------------- decode
    # the timed blocks are centred on 3/4 of the context: the mean of decoding from
    # a 2,048-token prompt to 4,096 tokens
    blocks = max(1, args.blocks)
    e2e_steps = max(8, args.steps // 2)
    while blocks > 1 and CONTEXT * 3 // 4 + (blocks * args.steps) // 2 + blocks * e2e_steps + \
            3 * args.warmup + 16 > CONTEXT:
        blocks -= 1
    start_ctx = max(1, CONTEXT * 3 // 4 - (blocks * args.steps + args.warmup) // 2)
    points = {}

    def decode_at(b, steps, warmup, n_blocks, with_clocks):
        # every point's timed steps are centred on the same context length
        first = max(1, CONTEXT * 3 // 4 - (n_blocks * steps + warmup) // 2)
        slots = fill(engine, b, first, seed=10 + b)
        sampler = ClockSampler() if with_clocks else None
        timed, launches, clocks = time_decode(engine, slots, steps, warmup, n_blocks, sampler)
        return slots, timed, launches, clocks

    slots, timed, launches, clocks = decode_at(batch, args.steps, args.warmup, blocks, True)
    ms, mean_ctx = median_block(timed)
    step_bytes = decode_step_bytes(engine, mean_ctx)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    for s in slots:
        engine.close_sequence(s)
    # the end-to-end blocks on sequences of their own, centred on the same context
    # length as the device-timed blocks (behind them they would read a longer cache)
    first = max(1, CONTEXT * 3 // 4 - (blocks * e2e_steps + args.warmup) // 2)
    slots = fill(engine, batch, first, seed=10 + batch)
    e2e_s, h2d, d2h = time_e2e(engine, slots, e2e_steps, args.warmup, blocks)
    for s in slots:
        engine.close_sequence(s)
    if not args.skip_points:
        for b in (1, 64):
            pslots, ptimed, _, _ = decode_at(b, e2e_steps, args.warmup, 3, False)
            points[f"decode_b{b}"] = b / (median_block(ptimed)[0] * 1e-3)
            for s in pslots:
                engine.close_sequence(s)
    del engine
    torch.cuda.empty_cache()
    if not args.skip_points and not args.skip_workloads:
        # the two other benchmark configurations, each with its own workload
        for key, spec in (("llama_1b", ("llama-3.2-1b", 32, 4096, 3, 512, 1.0, 8192)),
                          ("llama_8b", ("llama-3.1-8b", 16, 8192, 4, 256, 0.0, 16384))):
            point = workload_point(key, *spec)
            points[key] = point
            points[f"{key}_decode_tok_s"] = point["decode"]["value"]
            points[f"{key}_decode_frac"] = point["roofline"]["frac"]
            points[f"{key}_prefill_tok_s"] = point["prefill"]["value"]
            points[f"{key}_prefill_frac"] = point["prefill"]["frac"]

    value = batch / (ms * 1e-3)
    return {
        "metric": "decode tok/s at batch 8 (Llama-3.2-3B shape, bf16, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "vs_published_other_hw": {"decode_b1_over_6.92": (points.get("decode_b1") or 0) / PUBLISHED_DECODE_B1
                                  if points else None,
                                  "prefill_over_132.6": prefill["value"] / PUBLISHED_PREFILL_512},
        "dtype": "bf16", "data": "synthetic: random token ids (SplitMix64), random-init weights N(0, 0.02)",
        "config": {
            "model": "llama-3.2-3b-shape", "layers": layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": batch, "seq_len": CONTEXT, "context_start": start_ctx + args.warmup,
            "context_end": start_ctx + args.warmup + blocks * args.steps,
            "timed_blocks": blocks, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (6.4 GB of weights per step)",
            "peaks": source,
        },
        "block_ms_per_step": [round(t, 4) for t, _ in timed],
        "e2e": {"value": batch / e2e_s, "unit": "tokens/s", "ms_per_step": e2e_s * 1e3,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "timed_blocks": blocks,
                "steps_per_block": e2e_steps},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": achieved / hbm_gbs, "bytes_per_step": step_bytes, "of": source},
        "points": points,
        "clocks": clocks,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0,
                        help="fewer layers than the configuration's 28 (both numbers are reported)")
    parser.add_argument("--blocks", type=int, default=BLOCKS,
                        help="timed blocks of --steps steps; the median block is reported")
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the 1B and 8B workload points")
    parser.add_argument("--no-graphs", action="store_true",
                        help="launch decode kernels one by one (for profilers)")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "stratorys/foundry is a Rust crate whose only device backend is Metal on "
                          "macOS; it has no setup.py or pyproject.toml (pip: 'not installable'), no "
                          "cargo here, and no CPU or CUDA path to run"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    args.warmup = max(3, args.warmup)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
