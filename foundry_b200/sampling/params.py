"""How the next token is chosen.

The reference chooses greedily and in no other way: argmax over the
vocabulary, the lowest index among equal logits (src/generate/mod.rs:192-204,
src/metal/kernels/reduce.metal:67-68). `temperature = 0` is that rule.
A positive temperature samples from softmax(logits / temperature); the draw is
a pure function of (seed, request index, number of tokens the request has
generated), so a request's tokens do not depend on its batch.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if not (self.temperature >= 0.0):
            raise ValueError(f"temperature must not be negative, got {self.temperature}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
