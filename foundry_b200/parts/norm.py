"""RMS normalisation, fused with the residual sum that precedes it.

y = x * 1/sqrt(mean(x^2) + eps) * w, the statistics in 32-bit
(src/nn/norm.rs:31-51: square, sum, * 1/H, + eps, sqrt, reciprocal). The
reference rounds x*r to 16 bits before the weight multiply; here the product
is rounded once, at the end. The weight is held in float32 (exact for a
bfloat16 file; a 32-bit file stays as stored).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_norm


@register_norm("rms_norm")
class RMSNorm(Part):
    replay_safe = True  # forward reads nothing of the step on the host

    def __init__(self, size: int, eps: float, *, dtype: torch.dtype, device: torch.device):
        self.size, self.eps = size, float(eps)
        self.dtype, self.device = dtype, device
        self.weight: Optional[torch.Tensor] = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.weight": ExpectedTensor((self.size,))}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.weight = fetch(f"{prefix}.weight").to(torch.float32).contiguous()

    def sink(self, resid: torch.Tensor) -> Optional[ops.ResidualSink]:
        """What the projection in front of this norm needs to make the sum and
        prepare the norm itself (bfloat16 steps only)."""
        if self.dtype != torch.bfloat16 or self.weight is None:
            return None
        return ops.ResidualSink(resid, self.weight, self.eps)

    def add_norm(self, resid: torch.Tensor, delta, out: Optional[torch.Tensor] = None):
        """resid += delta (a tensor, split-K `ops.Planes`, or None); returns
        norm(resid) in the activation dtype. A delta that a projection made
        with this norm's `sink` comes back as an `ops.RowScaled`."""
        if isinstance(delta, ops.NormPending):
            return ops.add_rmsnorm(resid, delta, self.weight, self.eps, None)
        if out is None:
            out = torch.empty(resid.shape, dtype=self.dtype, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
