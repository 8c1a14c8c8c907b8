"""What every part of a layer is, and the registries they are looked up in.

A layer is put together from parts: a mixer (attention here), a feed-forward,
norms, a position encoding inside the mixer, and a block that arranges them.
Each part takes its sizes and constants as parameters, names the tensors it
loads, and runs on a `StepContext`; none knows which model it is in. The
reference's counterparts are the structs of src/nn and src/models/llama, which
are wired for one model (src/models/llama/model.rs:47-52).

Interfaces
----------
Part (all kinds)
    expected_tensors(prefix) -> {tensor name: ExpectedTensor}
    load(prefix, fetch)            fetch(name) -> device tensor (stored dtype rule applied)
Norm
    add_norm(resid, delta, out)    resid += delta (float32, in place); out = norm(resid)
PositionEncoding
    inv_freq: float32 [rotary_dim / 2] on the device; rotary_dim; attention_factor;
    optionally pairing = "half" (default) | "interleaved"
Mixer
    cache_request() -> KVRequest | StateRequest | None
    forward(ctx, x, cache_view) -> y      x, y: [tokens, hidden] in the activation dtype
FeedForward
    forward(ctx, x) -> y
Block
    forward(ctx, resid, delta, cache_view) -> new delta (not yet added to resid)
Optional, any part
    replay_safe = True (class attribute): the part's forward launches the same
    kernels with the same arguments whatever the step's values are, i.e. it
    reads the step only through the device tensors of `ctx` (never
    `ctx.*_host`, which are None in a replayed step). Short prompt steps of a
    model whose parts all say so are captured once per bucket and replayed
    (engine/prompt.py); otherwise they are launched one by one.
    first_weight() -> the weight tensor its forward streams first, or None.
    `ctx.reads_after_part` holds the first weight of whatever runs after the
    part being called (the block sets it for its mixer and feed-forward, the
    model for the block); a part may hand it to its last product as
    `then_reads`, which single-token steps turn into an L2 prefetch. A part
    that ignores both is still correct.
    The norm between two parts as work of the projections around it (single-
    token steps): a norm may offer `sink(resid) -> ops.ResidualSink`; a part
    that sets `accepts_row_scaled = True` takes `x` as an `ops.RowScaled`
    (a norm's output that still lacks its row scale; `ops.plain(x)` gives the
    tensor); where both hold, the block puts the sink into
    `ctx.residual_sink` for the part in front, which may hand it to its last
    product (`Linear.forward(residual=...)`) and return what that returns. A
    part that ignores `ctx.residual_sink` is still correct: the norm then runs
    as a kernel of its own.

A new part is a class with these methods plus one `register_*` call; the
engine builds it from `PartSpec(kind, params)` as `cls(**params, dtype=...,
device=...)`.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor

Fetch = Callable[[str], torch.Tensor]


class Part:
    """Base of all parts: no tensors, nothing to load."""

    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {}

    def load(self, prefix: str, fetch: Fetch) -> None:
        return None

    def first_weight(self) -> Optional[torch.Tensor]:
        return None


def first_weight_of(part) -> Optional[torch.Tensor]:
    """`part.first_weight()` where the part offers it."""
    probe = getattr(part, "first_weight", None)
    return probe() if callable(probe) else None


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, Any] = {}

    def register(self, kind: str, cls=None, *, replace: bool = False):
        def put(c):
            if kind in self._classes and not replace:
                raise ValueError(f"{self.what} {kind!r} is already registered")
            self._classes[kind] = c
            return c
        return put if cls is None else put(cls)

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def kinds(self):
        return sorted(self._classes)

    def build(self, spec: PartSpec, **context):
        try:
            cls = self._classes[spec.kind]
        except KeyError:
            raise KeyError(f"no {self.what} named {spec.kind!r}; registered: {self.kinds()}") from None
        return cls(**spec.params, **context)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
