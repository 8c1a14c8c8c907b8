"""SplitMix64, the generator the reference draws benchmark token ids with
(src/bench/rng.rs:9-43): state += golden gamma, then the two-multiply mix;
`below` rejects draws above the largest multiple of the bound so that ids are
uniform. The first outputs of seed 0 are pinned in the tests (rng.rs:52-62)."""
from __future__ import annotations

from typing import List, Optional

_MASK = (1 << 64) - 1
GOLDEN_GAMMA = 0x9E3779B97F4A7C15
MAX_DRAW_COUNT = 64


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + GOLDEN_GAMMA) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def below(self, bound: int) -> Optional[int]:
        if bound <= 0:
            raise ValueError("bound must be positive")
        rejected = (_MASK % bound + 1) % bound
        max_accepted = _MASK - rejected
        for _ in range(MAX_DRAW_COUNT):
            draw = self.next_u64()
            if draw <= max_accepted:
                return draw % bound
        return None


def token_rows(rng: SplitMix64, rows: int, count: int, vocab_size: int) -> List[List[int]]:
    """`rows` sequences of `count` ids, drawn row after row (src/bench/mod.rs:203-241)."""
    out = []
    for _ in range(rows):
        row = []
        for _ in range(count):
            t = rng.below(vocab_size)
            if t is None:
                raise RuntimeError("random draw failed")
            row.append(t)
        out.append(row)
    return out
