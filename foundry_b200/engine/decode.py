"""Single-token steps as a replayed CUDA graph.

A decode step of the 3B model is some two hundred small kernels; launched one
by one from the host they cost more than they run. The reference pays that
price (about 1,780 dispatches a step, src/metal/stream.rs batches them 64 to
a command buffer). Here the step of a fixed number of rows is captured once
and replayed: the kernels read tokens, positions, lengths and page tables from
fixed device buffers that one small copy from pinned host memory refreshes
before each replay.

Rows are padded up to a bucket size (1, 2, 4, ...). A padding row has
sequence index -1: the cache kernels skip it and its logits are ignored, so
padding changes no result. The chosen token of each row is written where the
next step reads its input, so steps can follow one another without the host
seeing the tokens (`DecodeSession.step`), or with the host feeding and reading
them every step (`step_host`, which is what generation uses).

A host that reads every step's tokens before it decides on the next leaves the
device idle while it decides. `step_host(..., more=True)` therefore starts the
step after this one before it hands this one's tokens out, on the guess that
the same rows go on with exactly those tokens (which is what a generation loop
does until a row ends). The next call finds its step already running. If the
guess was wrong (another token, a row less) the step is taken back:
`cancel_ahead` gives up the one position it added to each sequence, and the
rows it wrote are written again by the step that is wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import PAGE
from ..kernels import ops
from ..sampling.params import SamplingParams
from .context import StepContext, lengths_are_unequal
from .staging import StagingRing


def bucket_of(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class DecodeRunner:
    """Fixed buffers and the captured graph for `bucket` rows and page tables
    `width` pages wide."""

    def __init__(self, engine, bucket: int, width: int, unequal: bool = False):
        self.engine, self.bucket, self.width, self.unequal = engine, bucket, width, unequal
        dev = engine.device
        groups = engine.cache.groups
        b = bucket
        # packed int32 fields: token ids | positions | seq_of_token | want_rows | slots |
        # cu_tokens | kv_lens | one page table per group
        sizes = [b, b, b, b, b, b + 1, b] + [b * width for _ in groups]
        offsets = [int(o) for o in np.cumsum([0] + sizes)]
        # the host may prepare steps ahead of the device: uploads go through a ring
        self.fields = StagingRing(offsets[-1], torch.int32, dev)
        self.dev = self.fields.dev
        self.host_np = self.fields.values
        part = [self.dev[offsets[i]:offsets[i + 1]] for i in range(len(sizes))]
        self.h = [self.host_np[offsets[i]:offsets[i + 1]] for i in range(len(sizes))]
        self.meta_start = offsets[1]  # everything after the token ids
        # A captured step must not depend on host-side values of the step, so its
        # context carries none. A model with a part that reads them (one that does
        # not set `replay_safe`) is never captured: its steps are launched plainly
        # and the session fills the host copies in before each one.
        self.capturable = engine.model.replay_safe()
        self.ctx = StepContext(
            n_tokens=b, n_seqs=b, n_want=b, token_ids=part[0], positions=part[1],
            seq_of_token=part[2], want_rows=part[3], slots=part[4], cu_tokens=part[5],
            kv_lens=part[6], slots_host=None, cu_tokens_host=None, kv_lens_host=None,
            is_decode=True, max_q_len=1, max_kv_len=width * PAGE, unequal_lengths=unequal)
        for i, group in enumerate(groups):
            self.ctx._tables[id(group)] = part[7 + i].view(b, width)
        self.h_tables = [self.h[7 + i].reshape(b, width) for i in range(len(groups))]
        self.row_sig: List[Optional[Tuple[int, int, int]]] = [None] * b
        self.h[3][:] = np.arange(b)  # every row's logits are wanted
        self.h[5][:] = np.arange(b + 1)
        # sampling inputs: temperature per row; random stream and step count per row
        self.temperature = torch.zeros(b, dtype=torch.float32, device=dev)
        self.temperature_value = 0.0
        self.sampling_fields = StagingRing(2 * b, torch.int64, dev)
        self.meta64 = self.sampling_fields.dev
        self.next_tokens = torch.zeros(b, dtype=torch.int32, device=dev)
        self.tokens_host = torch.zeros(b, dtype=torch.int32).pin_memory()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kernels_per_step = 0
        self.kernel_histogram: Dict[str, int] = {}
        self.logits: Optional[torch.Tensor] = None

    def _body(self) -> None:
        engine = self.engine
        with ops.scratch_owner(engine.scratch):
            self.logits = engine.model.forward(self.ctx, engine.cache)
        b = self.bucket
        ops.select_tokens(self.logits, self.next_tokens, self.temperature, self.meta64[:b],
                          self.meta64[b:])
        self.ctx.token_ids.copy_(self.next_tokens)

    def run(self) -> None:
        """One step over the buffers' current contents."""
        if not self.engine.use_graphs or not self.capturable:
            self._body()
            return
        if self.graph is None:
            # The first call runs plainly (it loads the kernels, sizes the
            # allocator and IS this call's step); then the same work is captured
            # for every later call. Capturing executes nothing.
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
            # "relaxed": torch's pinned-memory allocator may query an event of an
            # earlier host copy while the capture is open; that call touches
            # nothing of this capture and must not invalidate it
            with torch.cuda.graph(graph, pool=self.engine.graph_pool(),
                                  capture_error_mode="relaxed"):
                self._body()
            ops.add_launches(-self.kernels_per_step)  # recorded, not launched
            if ops.PROFILER.mode is not None:
                ops.PROFILER.add_counts({k: -n for k, n in self.kernel_histogram.items()})
            self.graph = graph
            # `self.logits` is now the graph's own buffer, which replays fill;
            # this call's logits are the plain run's
            self.logits.copy_(plain_logits)
            return
        self.graph.replay()
        ops.add_launches(self.kernels_per_step)
        if ops.PROFILER.mode is not None:
            ops.PROFILER.add_counts(self.kernel_histogram)


class DecodeSession:
    """Decode steps of a set of open sequences, row i being `slots[i]`.
    `keys[i]` names row i's random stream and `counts[i]` is how many tokens
    its sequence has generated (both only matter when sampling)."""

    def __init__(self, engine, slots: Sequence[int], sampling: SamplingParams = SamplingParams(),
                 keys: Optional[Sequence[int]] = None, counts: Optional[Sequence[int]] = None):
        from ..sampling.sampler import stream_key
        self.engine = engine
        self.slots = list(slots)
        self.sampling = sampling
        keys = list(keys) if keys is not None else list(range(len(slots)))
        self.keys = keys
        self.streams = [stream_key(sampling.seed, k) for k in keys]
        self.counts = list(counts) if counts is not None else [0] * len(slots)
        self.runner: Optional[DecodeRunner] = None
        self.h2d_bytes_per_step = 0
        self.d2h_bytes_per_step = 0
        self._ahead: Optional[dict] = None  # the step that was started on a guess
        self._read = torch.cuda.Event()     # behind the copy of a step's tokens to the host

    def _prepare(self) -> DecodeRunner:
        """Reserve one more token per sequence and refresh the host buffers."""
        engine, cache = self.engine, self.engine.cache
        n = len(self.slots)
        lengths = [cache.length(s) for s in self.slots]
        limit = engine.spec.max_positions
        for s, length in zip(self.slots, lengths):
            if length + 1 > limit:
                raise ValueError(f"slot {s} would pass the model's {limit} positions")
        cache.reserve({s: length + 1 for s, length in zip(self.slots, lengths)})
        need = 1
        for g in cache.groups:
            need = max(need, max(len(g.pages.pages(s)) for s in self.slots))
        bucket = bucket_of(n)
        unequal = lengths_are_unequal(lengths)
        runner = self.runner
        if runner is None or runner.bucket != bucket or runner.width < need \
                or runner.unequal != unequal:
            width = 8 if runner is None or runner.bucket != bucket else runner.width
            while width < need:
                width *= 2
            previous = runner
            runner = self.runner = engine.decode_runner(bucket, width, unequal)
            if previous is not None and previous is not runner and previous.bucket == bucket:
                # tokens that stay on the device (`step`) move on with the session
                runner.ctx.token_ids.copy_(previous.next_tokens)
        h = runner.h
        h[1][:n] = lengths
        h[1][n:] = 0
        h[2][:n] = np.arange(n)
        h[2][n:] = -1
        h[4][:n] = self.slots
        h[4][n:] = cache.scratch_slot
        h[6][:n] = lengths
        h[6][:n] += 1
        h[6][n:] = 0
        epoch = cache.table.epoch
        for i, s in enumerate(self.slots):
            count = sum(len(g.pages.pages(s)) for g in cache.groups)
            sig = (s, epoch[s], count)
            if runner.row_sig[i] != sig:
                runner.row_sig[i] = sig
                for table, group in zip(runner.h_tables, cache.groups):
                    pages = group.pages.pages(s)
                    table[i, :len(pages)] = pages
        for i in range(n, bucket):
            runner.row_sig[i] = None
        if not runner.capturable:  # plain launches: the parts may read the step on the host
            pad = bucket - n
            runner.ctx.slots_host = self.slots + [cache.scratch_slot] * pad
            runner.ctx.cu_tokens_host = list(range(bucket + 1))
            runner.ctx.kv_lens_host = [length + 1 for length in lengths] + [0] * pad
        return runner

    def _upload(self, runner: DecodeRunner, tokens: Optional[Sequence[int]]) -> None:
        n = len(self.slots)
        start = runner.meta_start
        if tokens is not None:
            runner.host_np[:n] = tokens
            runner.host_np[n:runner.bucket] = 0
            start = 0
        self.h2d_bytes_per_step = runner.fields.upload(start)
        temperature = float(self.sampling.temperature)
        if runner.temperature_value != temperature:
            runner.temperature.fill_(temperature)
            runner.temperature_value = temperature
        if temperature > 0.0:
            b = runner.bucket
            m = runner.sampling_fields.values
            m[:n] = self.streams
            m[b:b + n] = self.counts
            self.h2d_bytes_per_step += runner.sampling_fields.upload()

    def set_tokens(self, tokens: Sequence[int]) -> None:
        """Device-resident stepping (`step`) starts from these input tokens."""
        self.cancel_ahead()
        self._pending_tokens = list(tokens)

    def step(self) -> None:
        """One step whose input tokens are the previous step's choices, which
        stay on the device."""
        self.cancel_ahead()
        self._launch(getattr(self, "_pending_tokens", None))
        self._pending_tokens = None

    def _launch(self, tokens: Optional[Sequence[int]]) -> DecodeRunner:
        runner = self._prepare()
        self._upload(runner, tokens)
        runner.run()
        self.counts = [c + 1 for c in self.counts]
        return runner

    # ------------------------------------------------------- a step ahead
    def has_ahead(self) -> bool:
        return self._ahead is not None

    def _may_run_ahead(self) -> bool:
        """A step may be started on a guess if it can be taken back and cannot
        fail: no state of fixed size, a step that never reads the host, room in
        the model's positions and in the cache."""
        engine, cache = self.engine, self.engine.cache
        if cache.state or not engine.model.replay_safe() or not engine.use_graphs:
            return False
        lengths = [cache.length(s) for s in self.slots]
        if any(n + 1 > engine.spec.max_positions for n in lengths):
            return False
        return cache.table.can_grow({s: n + 1 for s, n in zip(self.slots, lengths)})

    def cancel_ahead(self) -> None:
        """Take back the step that was started on a guess, if there is one: every
        sequence that is still the one it was gives up the position the step
        added (a slot that was closed meanwhile, or closed and opened again,
        is left alone)."""
        ahead, self._ahead = self._ahead, None
        if ahead is None:
            return
        table = self.engine.cache.table
        for slot, epoch, length in ahead["slots"]:
            if table.slots.is_held(slot) and table.epoch[slot] == epoch \
                    and table.length[slot] == length + 1:
                self.engine.cache.forget_from(slot, length)
        self.counts = list(ahead["counts"])

    def step_host(self, tokens: Sequence[int], more: bool = False,
                  counts: Optional[Sequence[int]] = None) -> List[int]:
        """One step fed from the host; returns the chosen tokens on the host.
        `counts`: how many tokens each row has generated before this step
        (sampling only). `more`: the caller expects to come back with the same
        rows and the tokens returned here, so the step after this one is
        started before this one's tokens are handed out."""
        tokens = [int(t) for t in tokens]
        ahead = self._ahead
        if ahead is not None and (ahead["tokens"] != tokens or
                                  (counts is not None and list(counts) != ahead["counts"])):
            self.cancel_ahead()
            ahead = None
        self._ahead = None
        if ahead is None:
            if counts is not None:
                self.counts = list(counts)
            runner = self._launch(tokens)
        else:
            runner = self.runner  # the step for these tokens is already on its way
        n = len(self.slots)
        runner.tokens_host[:n].copy_(runner.next_tokens[:n], non_blocking=True)
        self._read.record()
        guess = None
        if more and self._may_run_ahead():
            table = self.engine.cache.table
            guess = {"slots": [(s, table.epoch[s], table.length[s]) for s in self.slots],
                     "counts": list(self.counts)}
            self._launch(None)  # its input tokens are where this step left them
        self._read.synchronize()
        ops.raise_on_device_failure()
        self.d2h_bytes_per_step = n * 4
        out = runner.tokens_host[:n].tolist()
        if guess is not None:
            guess["tokens"] = out
            self._ahead = guess
        return out

    def logits(self) -> torch.Tensor:
        """float32 logits [rows, vocab] of the last step (a buffer the next step
        reuses). Waits for the step and raises if one of its kernels gave up."""
        if self._ahead is not None:
            raise RuntimeError("a step was started ahead: its logits have replaced the last "
                               "step's (use step_host(..., more=False) where logits are read)")
        torch.cuda.current_stream().synchronize()
        ops.raise_on_device_failure()
        return self.runner.logits[:len(self.slots)]
