"""Short prompt steps as replayed CUDA graphs.

A prompt step of the 3B model is some 230 kernel launches; from Python that is
4 to 5 ms of host time, more than the GPU needs for a prompt of up to a few
hundred tokens (the gain shrinks with the step: at 20 tokens the step takes
half the time, at 512 a few per cent less, and from about 1,000 tokens on the
buffers that a captured step keeps are no longer worth it). So steps of up to `PROMPT_GRAPH_TOKENS` tokens run like the
single-token steps (decode.py): padded up to a bucket (tokens, sequences,
page-table width, wanted rows), described by fixed device buffers that one copy
from pinned memory refreshes, captured once per bucket and replayed.

Padding tokens have sequence index -1 (the cache kernels skip them, attention
gives them no block), padding sequences have no tokens and length 0, padding
wanted rows point at row 0 and their logits are dropped: padding changes no
result. Longer steps are bound by the GPU and run as plain launches.

A captured step may not depend on host-side values of the step: the context of
a replayed step carries no host copies, and the attention's grid comes from a
bound that the bucket gives. Parts that read the host copies in their forward
(a part says so by not setting `replay_safe = True`) keep the model on plain
launches.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import PAGE
from ..kernels import ops
from .context import SequenceStep, StepContext, StepPlan, plan_step
from .decode import bucket_of
from .staging import StagingRing

# steps of more tokens than this run as plain launches (0: always plain)
PROMPT_GRAPH_TOKENS = int(os.environ.get("FOUNDRY_B200_PROMPT_GRAPH_TOKENS", "512"))
MAX_RUNNERS = 24  # buckets kept; the least recently used one goes first


def token_bucket(n: int) -> int:
    """16, 32, 64, 128, then multiples of 128: the boundaries at which the
    products change kernels (16, 128) are bucket boundaries too, so a padded
    step runs the kernels its plain form would."""
    if n <= 128:
        return max(16, bucket_of(n))
    return (n + 127) // 128 * 128


class PromptRunner:
    """Fixed buffers and the captured graph of one bucket."""

    def __init__(self, engine, tokens: int, seqs: int, width: int, want: int, long_queries: bool):
        self.engine = engine
        self.key = (tokens, seqs, width, want, long_queries)
        dev = engine.device
        groups = engine.cache.groups
        t, s = tokens, seqs
        # packed int32 fields, as in build_context
        sizes = [t, t, t, want, s, s + 1, s] + [s * width for _ in groups]
        offsets = [int(o) for o in np.cumsum([0] + sizes)]
        # steps may be queued ahead of the device (portions of a prompt whose logits
        # nobody waits for): the upload goes through a ring of pinned buffers
        self.fields = StagingRing(offsets[-1], torch.int32, dev)
        self.dev = self.fields.dev
        host_np = self.fields.values
        part = [self.dev[offsets[i]:offsets[i + 1]] for i in range(len(sizes))]
        self.h = [host_np[offsets[i]:offsets[i + 1]] for i in range(len(sizes))]
        self.h_tables = [self.h[7 + i].reshape(s, width) for i in range(len(groups))]
        self.ctx = StepContext(
            n_tokens=t, n_seqs=s, n_want=want, token_ids=part[0], positions=part[1],
            seq_of_token=part[2], want_rows=part[3], slots=part[4], cu_tokens=part[5],
            kv_lens=part[6], slots_host=None, cu_tokens_host=None, kv_lens_host=None,
            is_decode=False, max_q_len=t, max_kv_len=width * PAGE,
            # every sequence adds at most one partly filled block
            query_blocks_bound=(t + 63) // 64 + s, long_queries=long_queries)
        for i, group in enumerate(groups):
            self.ctx._tables[id(group)] = part[7 + i].view(s, width)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self.kernel_histogram: Dict[str, int] = {}
        self.logits: Optional[torch.Tensor] = None

    def fill(self, plan: StepPlan, scratch_slot: int) -> None:
        h = self.h
        T, S, W = int(plan.token_ids.size), len(plan.slots), len(plan.want_rows)
        h[0][:T] = plan.token_ids
        h[0][T:] = 0
        h[1][:T] = plan.positions
        h[1][T:] = 0
        h[2][:T] = plan.seq_of
        h[2][T:] = -1
        h[3][:W] = plan.want_rows
        h[3][W:] = 0
        h[4][:S] = plan.slots
        h[4][S:] = scratch_slot
        h[5][:S + 1] = plan.cu
        h[5][S + 1:] = T  # padding sequences: no tokens
        h[6][:S] = plan.kv_lens
        h[6][S:] = 0
        for table, (_, w, rows) in zip(self.h_tables, plan.tables):
            table[:S, :w] = np.asarray(rows, np.int32).reshape(S, w)
        self.fields.upload()

    def _body(self) -> None:
        with ops.scratch_owner(self.engine.scratch):
            self.logits = self.engine.model.forward(self.ctx, self.engine.cache)

    def run(self) -> torch.Tensor:
        """One step over the buffers' contents; logits [want bucket, vocab] in a
        buffer that the next step of this bucket reuses."""
        if self.graph is None:
            # as in DecodeRunner.run: this call's step runs plainly, then the same
            # work is captured for the later ones
            before = ops.launch_count()
            counted = ops.PROFILER.snapshot_counts()
            self._body()
            self.kernels_per_step = ops.launch_count() - before
            after = ops.PROFILER.snapshot_counts()
            self.kernel_histogram = {k: n - counted.get(k, 0) for k, n in after.items()
                                     if n != counted.get(k, 0)}
            plain_logits = self.logits
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self.engine.graph_pool(),
                                  capture_error_mode="relaxed"):
                self._body()
            ops.add_launches(-self.kernels_per_step)
            if ops.PROFILER.mode is not None:
                ops.PROFILER.add_counts({k: -n for k, n in self.kernel_histogram.items()})
            self.graph = graph
            self.logits.copy_(plain_logits)
            return self.logits
        self.graph.replay()
        ops.add_launches(self.kernels_per_step)
        if ops.PROFILER.mode is not None:
            ops.PROFILER.add_counts(self.kernel_histogram)
        return self.logits


def replay_safe(model) -> bool:
    """Whether every part of the model says that its forward reads nothing of
    the step on the host."""
    return model.replay_safe()


class PromptRunners:
    """The buckets of an engine, least recently used first out."""

    def __init__(self, engine):
        self.engine = engine
        self.enabled = replay_safe(engine.model)
        self._runners: Dict[Tuple[int, int, int, int, bool], PromptRunner] = {}

    def wants(self, steps: Sequence[SequenceStep]) -> bool:
        if not self.enabled or not self.engine.use_graphs or PROMPT_GRAPH_TOKENS <= 0:
            return False
        if ops.PROFILER.mode == "kernels":  # per-kernel timing needs plain launches
            return False
        return sum(len(s.tokens) for s in steps) <= PROMPT_GRAPH_TOKENS

    def step(self, steps: Sequence[SequenceStep]) -> torch.Tensor:
        engine = self.engine
        plan = plan_step(engine.cache, steps, engine.spec.vocab_size, engine.spec.max_positions)
        width = 8
        for _, w, _ in plan.tables:
            while width < w:
                width *= 2
        longest = max(plan.cu[i + 1] - plan.cu[i] for i in range(len(plan.slots)))
        key = (token_bucket(int(plan.token_ids.size)), bucket_of(len(plan.slots)), width,
               bucket_of(len(plan.want_rows)) if plan.want_rows else 0, longest >= 64)
        runner = self._runners.pop(key, None)
        if runner is None:
            if len(self._runners) >= MAX_RUNNERS:
                self._runners.pop(next(iter(self._runners)))
            runner = PromptRunner(engine, *key)
        self._runners[key] = runner  # most recently used last
        runner.fill(plan, engine.cache.scratch_slot)
        logits = runner.run()
        return logits[:len(plan.want_rows)].clone()

    def clear(self) -> None:
        self._runners.clear()
