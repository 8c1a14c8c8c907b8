"""The arrangement of a layer's parts.

`pre_norm_residual` is the reference's decoder layer
(src/models/llama/model.rs:254-278):

    h = x + mixer(norm1(x));  x' = h + feed_forward(norm2(h))

The residual stream is float32 and each sum is made in the kernel that also
normalises for the next part, so a block receives the previous block's output
still un-added (`delta`) and returns its own the same way. In single-token
steps that kernel is the projection in front of the norm: the block offers the
norm's `sink` to the part in front through `ctx.residual_sink`, and a part
that used it returns an `ops.NormPending`, which the norm turns into the
`ops.RowScaled` input of the part behind it.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import LayerSpec
from ..weights.loader import ExpectedTensor
from .base import (FEED_FORWARDS, MIXERS, NORMS, Fetch, Part, first_weight_of,
                   register_block)


@register_block("pre_norm_residual")
class PreNormResidualBlock(Part):
    replay_safe = True  # forward reads nothing of the step on the host

    def __init__(self, layer: LayerSpec, *, dtype: torch.dtype, device: torch.device):
        ctx = dict(dtype=dtype, device=device)
        self.prefix = layer.prefix
        self.names = dict(layer.names)
        self.mixer = MIXERS.build(layer.mixer, **ctx)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, **ctx)
        self.mixer_norm = NORMS.build(layer.mixer_norm, **ctx)
        self.feed_forward_norm = NORMS.build(layer.feed_forward_norm, **ctx)

    def _named(self):
        p, n = self.prefix, self.names
        return ((self.mixer_norm, f"{p}.{n['mixer_norm']}"),
                (self.mixer, f"{p}.{n['mixer']}"),
                (self.feed_forward_norm, f"{p}.{n['feed_forward_norm']}"),
                (self.feed_forward, f"{p}.{n['feed_forward']}"))

    def expected_tensors(self, prefix: str = "") -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for part, name in self._named():
            out.update(part.expected_tensors(name))
        return out

    def load(self, prefix: str, fetch: Fetch) -> None:
        for part, name in self._named():
            part.load(name, fetch)

    def cache_request(self):
        return self.mixer.cache_request()

    def first_weight(self):
        return first_weight_of(self.mixer)

    def input_sink(self, resid: torch.Tensor):
        """The sink of this block's first norm, if its mixer takes the norm's
        output without its row scale; for whatever runs in front of the block."""
        return _sink_for(self.mixer_norm, self.mixer, resid)

    def forward(self, ctx, resid: torch.Tensor, delta, cache):
        after_block = getattr(ctx, "reads_after_part", None)  # what follows this block
        sink_after_block = getattr(ctx, "residual_sink", None)
        normed = self.mixer_norm.add_norm(resid, delta)
        ctx.reads_after_part = first_weight_of(self.feed_forward)
        ctx.residual_sink = _sink_for(self.feed_forward_norm, self.feed_forward, resid)
        mixed = self.mixer.forward(ctx, normed, cache)
        normed = self.feed_forward_norm.add_norm(resid, mixed)
        ctx.reads_after_part = after_block
        ctx.residual_sink = sink_after_block
        return self.feed_forward.forward(ctx, normed)


def _sink_for(norm, consumer, resid: torch.Tensor):
    """`norm.sink(resid)` where the norm offers one and `consumer` takes the
    norm's output as an `ops.RowScaled`; else None."""
    offer = getattr(norm, "sink", None)
    if not callable(offer) or not getattr(consumer, "accepts_row_scaled", False):
        return None
    return offer(resid)
