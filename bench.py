#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.2-3B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences. The model has the layer
sizes of the 3B benchmark configuration with random bfloat16 weights; the
cache is sized for 4,096 tokens per sequence, and the timed steps run at a
mean context of 3,072 tokens, the mean of decoding from 2,048 to 4,096.
One JSON line is printed:

  value     decoded tokens per second, timed on the device with CUDA events
            (warm-up first; a step reads 6.4 GB of weights, far more than the
            126 MB L2, so no L2 flush is needed between steps)
  e2e       the same through the Python entry point: token ids go in from
            pinned host memory and come back to the host every step
  prefill   one 2,048-token prompt in one step: tokens/s and the fraction of
            the bf16 tensor-core peak its FLOPs reach
  roofline  the decode step's bytes (every weight once, the live sequences'
            cache) / time, against the measured copy bandwidth
  points    decode tokens/s at batch 1 and 64

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

CONFIG_3B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 28,
    "hidden_size": 3072, "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 8192, "vocab_size": 128256, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
FULL_LAYERS = 28
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, sustained, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            doc = json.load(handle)
        return (float(doc["hbm_gbs"]), float(doc["bf16_tflops"]),
                float(doc.get("bf16_tflops_sustained", doc["bf16_tflops"])), "measured")
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, 1400.0, "fallback"


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


def weight_and_cache_bytes(engine, context_lens) -> int:
    """Bytes a decode step has to read: every weight it uses once, and the
    keys and values of the live sequences."""
    return engine.model.weight_bytes_read_per_step() + \
        engine.cache.bytes_per_token() * int(sum(context_lens))


def prefill_flops(cfg, tokens: int, layers: int) -> float:
    """Products of a whole-prompt step: projections, causal attention, and the
    output head on the one wanted row."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv, d, a = cfg.q_size, cfg.kv_size, cfg.head_dim, cfg.num_attention_heads
    linear = 2.0 * tokens * (h * (q + 2 * kv) + q * h + 3 * h * i)
    attention = 2.0 * 2.0 * a * d * tokens * (tokens + 1) / 2.0
    return layers * (linear + attention) + 2.0 * h * v


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


def time_decode(engine, slots, steps: int, warmup: int, sampler=None):
    """Device-timed decode steps (tokens stay on the device) and the launches made."""
    import torch
    from foundry_b200.kernels import ops
    session = engine.decode_session(slots)
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count()
    if sampler:
        sampler.start()
    start.record()
    for _ in range(steps):
        session.step()
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = start.elapsed_time(end)
    return ms / steps, ops.launch_count() - launches0, clocks, session


def time_e2e(engine, slots, steps: int, warmup: int):
    """The public call a user makes for one decode step: host token ids in
    (from pinned memory), host token ids out."""
    import torch
    session = engine.decode_session(slots)
    tokens = [1] * len(slots)
    for _ in range(warmup):
        tokens = session.step_host(tokens)
    torch.cuda.synchronize()
    started = time.perf_counter()
    for _ in range(steps):
        tokens = session.step_host(tokens)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    return seconds / steps, session.h2d_bytes_per_step, session.d2h_bytes_per_step


def run(args) -> dict:
    import torch
    from foundry_b200.config import LlamaConfig
    from foundry_b200.engine import Engine, SequenceStep
    from foundry_b200.bench import SplitMix64, token_rows

    layers = args.layers or FULL_LAYERS
    cfg = LlamaConfig.parse({**CONFIG_3B, "num_hidden_layers": layers})
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
    p_flops = prefill_flops(cfg, PREFILL_TOKENS, layers)
    prefill = {"value": PREFILL_TOKENS / (p_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": p_ms,
               "frac": p_flops / (p_ms * 1e-3) / (tflops_burst * 1e12), "flops": p_flops,
               "peak_tflops": tflops_burst}

    # ----------------------------------------------------------------- decode
    start_ctx = CONTEXT * 3 // 4 - (args.steps + args.warmup) // 2
    points = {}

    def decode_at(b, steps, warmup, with_clocks):
        slots = fill(engine, b, start_ctx, seed=10 + b)
        sampler = ClockSampler() if with_clocks else None
        ms, launches, clocks, session = time_decode(engine, slots, steps, warmup, sampler)
        ctx_lens = [engine.cache.length(s) for s in slots]
        result = (ms, launches, clocks, ctx_lens)
        return slots, result

    slots, (ms, launches, clocks, ctx_lens) = decode_at(batch, args.steps, args.warmup, True)
    mean_ctx = [c - args.steps / 2.0 for c in ctx_lens]
    step_bytes = weight_and_cache_bytes(engine, mean_ctx)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e_s, h2d, d2h = time_e2e(engine, slots, max(8, args.steps // 2), args.warmup)
    for s in slots:
        engine.close_sequence(s)
    if not args.skip_points:
        for b in (1, 64):
            pslots, (pms, _, _, _) = decode_at(b, max(8, args.steps // 2), args.warmup, False)
            points[f"decode_b{b}"] = b / (pms * 1e-3)
            for s in pslots:
                engine.close_sequence(s)

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
            "model": "llama-3.2-3b-shape", "layers": layers, "layers_full": FULL_LAYERS,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": batch, "seq_len": CONTEXT, "context_start": start_ctx + args.warmup,
            "context_end": start_ctx + args.warmup + args.steps, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (6.4 GB of weights per step)",
            "peaks": source,
        },
        "e2e": {"value": batch / e2e_s, "unit": "tokens/s", "ms_per_step": e2e_s * 1e3,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
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
    parser.add_argument("--skip-points", action="store_true")
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
