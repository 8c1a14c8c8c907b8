"""A model built from its description: parts, weights, and the forward pass
over a step's tokens.

Order of work (src/models/llama/model.rs:168-193 and 102-122): gather the
token embeddings; run the schedule's layers; keep only the rows whose logits
are wanted; final norm; output head (the embedding table when the description
names no separate head, model.rs:62). The residual stream is float32.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import CacheRequest, SequenceCache
from ..config.spec import ModelSpec
from ..kernels import ops
from ..parts import BLOCKS, NORMS
from ..parts.base import first_weight_of
from ..parts.linear import matmul_nt
from ..weights.loader import ExpectedTensor, check_against, load_tensor
from ..weights.safetensors_io import WeightFiles


def _build_blocks(spec: ModelSpec, dtype, device):
    return [BLOCKS.build(layer.block, layer=layer, dtype=dtype, device=device)
            for layer in spec.layers]


def expected_tensors(spec: ModelSpec) -> Dict[str, ExpectedTensor]:
    """Every tensor the model loads, by name, with its shape. Building the
    parts for this needs no GPU: no part touches the device before `load`."""
    model = Model(spec, torch.bfloat16, torch.device("meta"))
    return model.expected_tensors()


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.blocks = _build_blocks(spec, dtype, device)
        self.final_norm = NORMS.build(spec.final_norm, dtype=dtype, device=device)
        self.embedding: Optional[torch.Tensor] = None
        self.output_head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------- weights
    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        spec = self.spec
        out = {spec.embedding_name: ExpectedTensor((spec.vocab_size, spec.hidden_size))}
        for block in self.blocks:
            out.update(block.expected_tensors())
        out.update(self.final_norm.expected_tensors(spec.final_norm_prefix))
        if spec.output_head_name is not None:
            out[spec.output_head_name] = ExpectedTensor((spec.vocab_size, spec.hidden_size))
        return out

    def load(self, files: WeightFiles) -> None:
        """Check the folder against the model's list, then move every tensor
        to the device in its run dtype."""
        check_against(files, self.expected_tensors(), self.spec.ignorable_tensors)
        self._load_with(lambda name: load_tensor(files, name, self.dtype, self.device))

    def load_tensors(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take already materialised tensors (any device), by the same names."""
        from ..weights.loader import stored_to_run_dtype
        expected = self.expected_tensors()
        missing = [n for n in expected if n not in tensors]
        wrong = [(n, e.shape, tuple(tensors[n].shape)) for n, e in expected.items()
                 if n in tensors and tuple(tensors[n].shape) != tuple(e.shape)]
        if missing or wrong:
            from ..weights.loader import WeightsMismatch
            raise WeightsMismatch(missing, [], wrong, [])

        def fetch(name):
            t = tensors[name]
            return t.to(device=self.device, dtype=stored_to_run_dtype(t.dtype, self.dtype))
        self._load_with(fetch)

    def _load_with(self, fetch) -> None:
        spec = self.spec
        self.embedding = fetch(spec.embedding_name).contiguous()
        for block in self.blocks:
            block.load(block.prefix, fetch)
        self.final_norm.load(spec.final_norm_prefix, fetch)
        self.output_head = (self.embedding if spec.output_head_name is None
                            else fetch(spec.output_head_name).contiguous())
        if self.embedding.dtype != self.dtype or self.output_head.dtype != self.dtype:
            raise ops.KernelError(
                f"embedding / output head are stored in {self.embedding.dtype}; run with "
                f"--dtype float32 for a 32-bit weight file")

    def weight_bytes_read_per_step(self) -> int:
        """Bytes of weights a single-token step reads once: every tensor the
        model lists (`expected_tensors`), in the run dtype, except the embedding
        table when a separate output head exists (its rows are only gathered;
        a tied table is read whole as the head). A feed-forward that routes
        tokens to some of its weights reads fewer than this counts."""
        spec = self.spec
        size = torch.empty((), dtype=self.dtype).element_size()
        total = 0
        for name, want in self.expected_tensors().items():
            if name == spec.embedding_name and spec.output_head_name is not None:
                continue
            count = 1
            for d in want.shape:
                count *= int(d)
            total += count * size
        return total

    def replay_safe(self) -> bool:
        """Whether every part says that its forward reads nothing of the step
        on the host (`replay_safe = True`, see parts/base.py): only then may a
        step of this model be captured once and replayed."""
        for block in self.blocks:
            parts = [block] + [getattr(block, name, None) for name in
                               ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")]
            if not all(p is not None and getattr(p, "replay_safe", False) for p in parts):
                return False
        return bool(getattr(self.final_norm, "replay_safe", False))

    # --------------------------------------------------------------- cache
    def cache_requests(self) -> Dict[int, CacheRequest]:
        requests: Dict[int, CacheRequest] = {}
        for entry in self.spec.schedule:
            want = self.blocks[entry.layer].cache_request()
            if entry.cache in requests and requests[entry.cache] != want:
                raise ValueError(
                    f"cache entry {entry.cache} is used by layers that need different storage")
            requests[entry.cache] = want
        return requests

    # ------------------------------------------------------------- forward
    def forward(self, ctx, cache: SequenceCache) -> torch.Tensor:
        """Logits [wanted rows, vocab] in float32 for the step `ctx` describes."""
        spec = self.spec
        shared = getattr(ctx, "shared", None)
        if shared is not None:
            shared.clear()  # what an earlier step on this context left
        resid = torch.empty((ctx.n_tokens, spec.hidden_size), dtype=torch.float32,
                            device=self.device)
        ops.embed_gather(self.embedding, ctx.token_ids, resid)
        delta = None
        for i, entry in enumerate(spec.schedule):
            block = self.blocks[entry.layer]
            follower = (self.blocks[spec.schedule[i + 1].layer] if i + 1 < len(spec.schedule)
                        else None)
            ctx.reads_after_part = (first_weight_of(follower) if follower is not None
                                    else self.output_head if ctx.n_want else None)
            # the last block's result meets the final norm on the wanted rows only
            offer = getattr(follower, "input_sink", None)
            ctx.residual_sink = offer(resid) if callable(offer) else None
            delta = block.forward(ctx, resid, delta, cache.view(entry.cache, entry.writes_cache))
        ctx.reads_after_part = None
        ctx.residual_sink = None
        n = ctx.n_want
        logits = torch.empty((n, spec.vocab_size), dtype=torch.float32, device=self.device)
        if n == 0:
            return logits
        rows = torch.empty((n, spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.gather_rows(resid, ctx.want_rows, rows)
        rows_delta = None
        if isinstance(delta, ops.Planes):
            delta = delta.sum(self.dtype)
        if delta is not None:
            rows_delta = torch.empty((n, spec.hidden_size), dtype=delta.dtype, device=self.device)
            ops.gather_rows(delta, ctx.want_rows, rows_delta)
        normed = self.final_norm.add_norm(rows, rows_delta)
        return matmul_nt(normed, self.output_head, logits)
