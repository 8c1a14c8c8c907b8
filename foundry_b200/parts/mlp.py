"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(src/models/llama/mlp.rs:49-58); SiLU is x / (1 + exp(-x)) in 32-bit
(src/nn/activation.rs:18-27). gate and up are one fused product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import Fetch, Part, register_feed_forward
from .linear import Linear, matmul_nt


@register_feed_forward("swiglu")
class SwiGLU(Part):
    replay_safe = True  # forward reads nothing of the step on the host
    accepts_row_scaled = True  # the gate/up product applies a deferred norm's row scale

    def __init__(self, hidden_size: int, intermediate_size: int, *, dtype: torch.dtype,
                 device: torch.device):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.gate_up: torch.Tensor = None  # [2I, H]: row 2i is gate i, row 2i+1 is up i
        self.down = Linear(intermediate_size, [("down_proj", hidden_size)], dtype=dtype,
                           device=device)

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        shape = (self.intermediate_size, self.hidden_size)
        return {f"{prefix}.gate_proj.weight": ExpectedTensor(shape),
                f"{prefix}.up_proj.weight": ExpectedTensor(shape),
                **self.down.expected_tensors(prefix)}

    def load(self, prefix: str, fetch: Fetch) -> None:
        gate, up = fetch(f"{prefix}.gate_proj.weight"), fetch(f"{prefix}.up_proj.weight")
        if gate.dtype != up.dtype:
            raise ops.KernelError(f"{prefix}: gate and up projections are stored in different dtypes")
        # rows interleaved so that a product tile holds matching gate / up pairs
        self.gate_up = torch.stack([gate, up], 1).reshape(2 * self.intermediate_size,
                                                          self.hidden_size).contiguous()
        self.down.load(prefix, fetch)

    def first_weight(self):
        return self.gate_up

    def forward(self, ctx, x):
        hidden = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16:
            ops.gemm_bf16_silu_mul(x, self.gate_up, hidden,  # activation in the epilogue
                                   then_reads=self.down.weight)
        else:
            ops.silu_mul(matmul_nt(ops.plain(x), self.gate_up), hidden, interleaved=True)
        return self.down.forward(hidden, allow_planes=True,
                                 then_reads=getattr(ctx, "reads_after_part", None),
                                 residual=getattr(ctx, "residual_sink", None))
