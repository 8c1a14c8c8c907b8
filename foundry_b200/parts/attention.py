"""Grouped-query attention over the cache, as a mixer.

q = n Wq^T, k = n Wk^T, v = n Wv^T (one fused product); q and k are rotated by
the position encoding; k and v are appended to the sequence's cache pages;
every token attends causally to its sequence's cache; o = attn Wo^T
(src/models/llama/attention.rs:72-131). Query head a reads key-value head
a // (heads // kv_heads) (src/nn/attention.rs:40-44); scores are scaled by
1/sqrt(head_dim) (attention.rs:56-58). Unlike the reference, heads x head_dim
need not equal the hidden size (it loads q_proj as [H, H], attention.rs:52).

The part takes head counts, head size, window and its position encoding as
parameters and asks the cache for keys and values of its shape; which layer
of which model it serves is not its business.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.store import KVRequest, KVView
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import ExpectedTensor
from .base import POSITION_ENCODINGS, Fetch, Part, register_mixer
from .linear import Linear


@register_mixer("gqa_attention")
class GQAAttention(Part):
    replay_safe = True  # forward reads nothing of the step on the host
    accepts_row_scaled = True  # the q/k/v product applies a deferred norm's row scale

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[PartSpec], window: Optional[int] = None, *,
                 dtype: torch.dtype, device: torch.device):
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.window = head_dim, window
        self.dtype, self.device = dtype, device
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        self.qkv = Linear(hidden_size, [("q_proj", self.q_size), ("k_proj", self.kv_size),
                                        ("v_proj", self.kv_size)], dtype=dtype, device=device)
        self.o = Linear(self.q_size, [("o_proj", hidden_size)], dtype=dtype, device=device)
        self.pairing = "half"
        if position_encoding is None:
            self.rotary_dim = 0
            self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
            self.angles_key = ("rotary angles", b"")
            factor = 1.0
        else:
            enc = POSITION_ENCODINGS.build(position_encoding, dtype=dtype, device=device)
            self.rotary_dim, self.inv_freq, factor = enc.rotary_dim, enc.inv_freq, enc.attention_factor
            self.pairing = getattr(enc, "pairing", "half")
            # layers whose encodings have the same frequencies share a step's angle table
            # (an encoding without a host copy of its frequencies keeps a table of its own)
            host = getattr(enc, "inv_freq_host", None)
            self.angles_key = ("rotary angles", host.tobytes() if host is not None else id(enc))
        self.scale = factor / math.sqrt(head_dim)

    # ----------------------------------------------------------------- setup
    def expected_tensors(self, prefix: str) -> Dict[str, ExpectedTensor]:
        return {**self.qkv.expected_tensors(prefix), **self.o.expected_tensors(prefix)}

    def load(self, prefix: str, fetch: Fetch) -> None:
        self.qkv.load(prefix, fetch)
        self.o.load(prefix, fetch)
        if self.rotary_dim and self.pairing == "half":
            # Store the rows of every query and key head so that the two features a
            # frequency turns are neighbours (2i, 2i + 1) instead of half a rotary width
            # apart: the product kernels then rotate in their epilogue by exchanging
            # values between neighbouring lanes. Scores are dot products over a head's
            # features, so any order serves as long as queries and keys share it; values
            # and the output projection are untouched.
            self.qkv.weight = self.qkv.weight.index_select(0, self._neighbour_order()).contiguous()
            self.pairing = "interleaved"

    def _neighbour_order(self) -> torch.Tensor:
        """Row order of the fused q/k/v matrix with rotation partners adjacent."""
        half = self.rotary_dim // 2
        within = []
        for i in range(half):
            within += [i, i + half]
        within += list(range(self.rotary_dim, self.head_dim))
        order = []
        for head in range(self.num_heads + self.num_kv_heads):
            order += [head * self.head_dim + e for e in within]
        order += list(range(len(order), len(order) + self.kv_size))  # the value heads as they are
        return torch.tensor(order, dtype=torch.long, device=self.qkv.weight.device)

    def cache_request(self) -> KVRequest:
        return KVRequest(self.num_kv_heads, self.head_dim, self.window)

    def first_weight(self):
        return self.qkv.weight

    def context_flops(self, token_counts, starts) -> float:
        """Operations of the scores and the weighted sums of one step: 4 per
        query head, head element and visible (query, key) pair."""
        pairs = 0.0
        for n, start in zip(token_counts, starts):
            for p in (start, start + n - 1):  # causal: the mean of the first and last query
                pairs += 0.5 * n * (min(p + 1, self.window) if self.window else p + 1)
        return 4.0 * self.num_heads * self.head_dim * pairs

    # ------------------------------------------------------------------- run
    def forward(self, ctx, x, cache: KVView):
        table = ctx.page_table(cache.group)
        if ops.qkv_rope_fusable(x, self.qkv.weight, self.rotary_dim, self.head_dim, cache.k):
            # a handful of tokens: projection, rotation and cache write in one kernel
            q = ops.gemm_skinny_rope(x, self.qkv.weight, ctx.positions, ctx.seq_of_token, table,
                                     self.inv_freq, self.rotary_dim, cache.k, cache.v,
                                     self.num_heads, self.num_kv_heads, self.head_dim,
                                     ring_pages=cache.group.ring_pages, write_cache=cache.writes,
                                     pairing=self.pairing)
        elif ops.qkv_rows_rope_fusable(x, self.qkv.weight, self.rotary_dim, self.head_dim, cache.k,
                                       self.pairing):
            # up to a few hundred tokens: the same on the tcgen05 product
            q = ops.gemm_rows_rope(x, self.qkv.weight, ctx.positions, ctx.seq_of_token, table,
                                   self.inv_freq, self.rotary_dim, cache.k, cache.v,
                                   self.num_heads, self.num_kv_heads, self.head_dim,
                                   ring_pages=cache.group.ring_pages, write_cache=cache.writes)
        elif ops.qkv_tc_rope_fusable(x, self.qkv.weight, self.rotary_dim, self.head_dim, cache.k,
                                     self.pairing):
            # a prompt: the same in the epilogue of the products whose rows are tokens,
            # with the step's angles from a table that the first layer of the step makes
            shared = getattr(ctx, "shared", None)
            cs = shared.get(self.angles_key) if shared is not None else None
            if cs is None:
                cs = ops.rope_table(ctx.positions, self.inv_freq)
                if shared is not None:
                    shared[self.angles_key] = cs
            q = ops.gemm_tc_rope(x, self.qkv.weight, cs, ctx.positions, ctx.seq_of_token, table,
                                 self.rotary_dim, cache.k, cache.v, self.num_heads,
                                 self.num_kv_heads, self.head_dim,
                                 ring_pages=cache.group.ring_pages, write_cache=cache.writes)
        else:
            # (a row-scaled input stays so: the tcgen05 products apply the scale)
            qkv = self.qkv.forward(x, allow_planes=True)  # a tensor or split-K planes
            q = ops.rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, table, self.inv_freq,
                                  self.rotary_dim, cache.k, cache.v, self.num_heads,
                                  self.num_kv_heads, self.head_dim,
                                  ring_pages=cache.group.ring_pages, write_cache=cache.writes,
                                  dtype=x.dtype, pairing=self.pairing)
        attn = torch.empty((x.shape[0], self.q_size), dtype=x.dtype, device=x.device)
        ops.attention(ctx, q, attn, table, cache.k, cache.v, self.num_heads, self.num_kv_heads,
                      self.head_dim, self.scale, window=cache.group.window,
                      ring_pages=cache.group.ring_pages, then_reads=self.o.weight)
        return self.o.forward(attn, allow_planes=True,
                              then_reads=getattr(ctx, "reads_after_part", None),
                              residual=getattr(ctx, "residual_sink", None))
