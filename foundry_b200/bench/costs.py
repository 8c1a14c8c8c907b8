"""What a step has to move and to compute, and the peaks to hold it against.

The reference's report gives rates only (src/bench/metrics.rs:60-150); here a
rate also says how far it is from what the hardware allows: a decode step is
bound by the bytes it must read (every weight it uses once, and the keys and
values of the live sequences), a prompt step by the floating-point work of its
products. Both figures follow from the loaded model, not from a table of sizes.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Sequence

# An earlier measurement on B200, used when no measured figures are at hand.
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks(path: Optional[str] = None) -> Dict:
    """{hbm_gbs, bf16_tflops, bf16_tflops_sustained, source}: the measured copy
    bandwidth and tensor-core rate from a JSON file with these keys (`path`, or
    `$FOUNDRY_B200_PEAKS`), else the fallback figures."""
    path = path or os.environ.get("FOUNDRY_B200_PEAKS")
    if path:
        try:
            with open(path) as handle:
                doc = json.load(handle)
            burst = float(doc["bf16_tflops"])
            return {"hbm_gbs": float(doc["hbm_gbs"]), "bf16_tflops": burst,
                    "bf16_tflops_sustained": float(doc.get("bf16_tflops_sustained", burst)),
                    "source": "measured"}
        except (OSError, KeyError, ValueError, TypeError):
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


def decode_step_bytes(engine, context_lens: Sequence[float]) -> int:
    """Bytes a single-token step reads: the weights once, and the cached keys and
    values of sequences of these lengths."""
    return int(engine.model.weight_bytes_read_per_step()
               + engine.cache.bytes_per_token() * float(sum(context_lens)))


def step_flops(model, token_counts: Sequence[int], starts: Optional[Sequence[int]] = None,
               wanted_rows: int = 1) -> float:
    """Floating-point operations of one step in which sequence i brings
    `token_counts[i]` tokens behind `starts[i]` cached ones: two per weight of
    every layer that runs and per token, the mixers' own work on the cache
    (what a mixer reports through `context_flops`), and the output head on the
    wanted rows."""
    starts = list(starts) if starts is not None else [0] * len(token_counts)
    tokens = float(sum(token_counts))
    spec = model.spec
    expected = model.expected_tensors()
    total = 0.0
    for entry in spec.schedule:
        block = model.blocks[entry.layer]
        prefix = block.prefix + "."
        weights = sum(_numel(e.shape) for name, e in expected.items()
                      if name.startswith(prefix) and len(e.shape) == 2)
        total += 2.0 * tokens * weights
        probe = getattr(block.mixer, "context_flops", None)
        if callable(probe):
            total += float(probe(token_counts, starts))
    return total + 2.0 * wanted_rows * spec.hidden_size * spec.vocab_size


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def roofline(bytes_or_flops: float, seconds: float, peak: float, unit: str) -> Dict:
    """{achieved, peak, unit, frac} of a step: `peak` in GB/s (with bytes) or
    TFLOP/s (with operations)."""
    scale = 1e9 if unit == "GB/s" else 1e12
    achieved = bytes_or_flops / seconds / scale if seconds > 0 else 0.0
    return {"achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak}
