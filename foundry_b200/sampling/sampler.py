"""Token selection on the device: one kernel launch per step.

`uniform24` / `gumbel_scores` restate the kernel's random stream on the host
(csrc/sampling.cu) so that a sampled token can be checked without a GPU.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams

_M1, _M2, _GOLDEN = 0xbf58476d1ce4e5b9, 0x94d049bb133111eb, 0x9e3779b97f4a7c15
_MASK = (1 << 64) - 1


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def stream_key(seed: int, key: int) -> int:
    """The random stream of sequence `key` under `seed`, as a signed 64-bit
    integer: mix64(seed + GOLDEN * (key + 1)). Formed once per sequence on the
    host; the kernel mixes in the step and the token id."""
    z = (seed + _GOLDEN * (key + 1)) & _MASK
    z = ((z ^ (z >> 30)) * _M1) & _MASK
    z = ((z ^ (z >> 27)) * _M2) & _MASK
    z ^= z >> 31
    return z - (1 << 64) if z >= (1 << 63) else z


def uniform24(seed: int, key: int, step: int, count: int) -> np.ndarray:
    """u_i in (0, 1) for token ids 0..count-1, as float32, bit-equal to the kernel's."""
    with np.errstate(over="ignore"):
        z = np.uint64(stream_key(seed, key) & _MASK)
        z = _mix64(z + np.uint64(_GOLDEN) * np.uint64(step + 1))
        i = np.arange(1, count + 1, dtype=np.uint64)
        z = _mix64(z + np.uint64(_GOLDEN) * i)
    return ((z >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)


def gumbel_scores(logits: np.ndarray, temperature: float, seed: int, key: int,
                  step: int) -> np.ndarray:
    """logit_i / T - log(-log(u_i)) in float32: the quantity whose argmax is the sample."""
    u = uniform24(seed, key, step, logits.shape[-1])
    inv_t = np.float32(1.0) / np.float32(temperature)
    return logits.astype(np.float32) * inv_t - np.log(-np.log(u)).astype(np.float32)


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def select(self, logits: torch.Tensor, params: SamplingParams,
               keys: Optional[Sequence[int]] = None,
               steps: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One token per logits row, int32 on the device."""
        n = logits.shape[0]
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if params.greedy:
            return ops.select_tokens(logits, out, None)
        streams = [stream_key(params.seed, int(k)) for k in keys]
        meta = torch.tensor([streams, list(steps)], dtype=torch.int64).to(logits.device)
        temp = torch.full((n,), float(params.temperature), dtype=torch.float32,
                          device=logits.device)
        return ops.select_tokens(logits, out, temp, meta[0], meta[1])
