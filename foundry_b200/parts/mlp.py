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
from .linear import Linear


@register_feed_forward("swiglu")
class SwiGLU(Part):
    def __init__(self, hidden_size: int, intermediate_size: int, *, dtype: torch.dtype,
                 device: torch.device):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.gate_up = Linear(hidden_size, [("gate_proj", intermediate_size),
                                            ("up_proj", intermediate_size)],
                              dtype=dtype, device=device)
        self.down = Linear(intermediate_size, [("down_proj", hidden_size)], dtype=dtype,
                           device=device)

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {**self.gate_up.expected_tensors(prefix), **self.down.expected_tensors(prefix)}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.gate_up.load(prefix, fetch)
        self.down.load(prefix, fetch)

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        gate_up = self.gate_up.forward(x)
        hidden = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        ops.silu_mul(gate_up, hidden)
        return self.down.forward(hidden)
