"""Projections: y = x W^T, W stored [out, in] row-major, no bias
(src/nn/linear.rs:19-36).

Several projections of the same input are held as one matrix, their rows
concatenated at load time (q, k, v; gate, up), so that one product serves
them; the tensor names in the files stay the separate Hugging Face ones.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part


def matmul_nt(x, w: torch.Tensor, out: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, allow_planes: bool = False,
              then_reads: Optional[torch.Tensor] = None,
              residual: Optional[ops.ResidualSink] = None):
    """out[M,N] = x[M,K] @ w[N,K]^T, accumulated in 32-bit, by the kernel that
    fits the element type and the shape. With `allow_planes` a split-K product
    may come back as `ops.Planes` (float32 partial results) for a consumer that
    sums them while it reads. `then_reads` names the weights the step streams
    next, a hint that the single-token kernel turns into an L2 prefetch. `x` may
    be an `ops.RowScaled`; with `residual` the product may add its result to the
    residual rows itself and return an `ops.NormPending` (see `ops.gemm_bf16`)."""
    M, N = x.shape[0], w.shape[0]
    if x.dtype != w.dtype:
        raise ops.KernelError(
            f"projection input is {x.dtype} but the weight is {w.dtype}; a weight file stored "
            f"in 32 bits needs --dtype float32")
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
        return ops.gemm_simt(x, w, out)
    return ops.gemm_bf16(x, w, out, out_dtype, allow_planes, then_reads, residual)


class Linear(Part):
    """One or more named [out_i, in] matrices applied as a single product."""

    def __init__(self, in_features: int, outs: Sequence[Tuple[str, int]], *, dtype: torch.dtype,
                 device: torch.device):
        self.in_features = in_features
        self.outs = list(outs)  # (name suffix such as "q_proj", rows)
        self.out_features = sum(n for _, n in self.outs)
        self.dtype, self.device = dtype, device
        self.weight: Optional[torch.Tensor] = None

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {f"{prefix}.{name}.weight": ExpectedTensor((rows, self.in_features))
                for name, rows in self.outs}

    def load(self, prefix: str, fetch: Fetch) -> None:
        parts = [fetch(f"{prefix}.{name}.weight") for name, _ in self.outs]
        kinds = {p.dtype for p in parts}
        if len(kinds) != 1:
            raise ops.KernelError(f"{prefix}: fused projections are stored in different dtypes")
        self.weight = parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, 0).contiguous()

    def forward(self, x, out: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, allow_planes: bool = False,
                then_reads: Optional[torch.Tensor] = None,
                residual: Optional[ops.ResidualSink] = None):
        return matmul_nt(x, self.weight, out, out_dtype, allow_planes, then_reads, residual)
