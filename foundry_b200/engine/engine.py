"""The engine: a loaded model, its cache, the step function and the loop.

`Engine.step` is the one step function: a batch of sequences, each bringing
its next tokens (a whole prompt, a chunk, or one token), run as one packed
batch from the cache, returning float32 logits at the wanted places only.
The reference's counterpart is `CausalLm::forward` + `Decoder`
(src/models/mod.rs:19-27, src/generate/mod.rs:92-205), which takes equal
lengths and one shared position.
"""
from __future__ import annotations

import itertools
import weakref
from typing import List, Optional, Sequence

import torch

from ..cache.store import SequenceCache
from ..config import load_model_config
from ..config.spec import ModelSpec
from ..sampling import Sampler, SamplingParams
from ..weights.safetensors_io import WeightFiles
from . import generate as loop
from ..cache.pages import CacheFull
from .context import SequenceStep, build_context, check_steps
from .prompt import PromptRunners
from .decode import DecodeRunner, DecodeSession
from .model import Model
from ..kernels import ops

_ENGINE_NUMBERS = itertools.count()
_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "f32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r}: choose bfloat16 or float32") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(
            f"the engine runs on CUDA devices only (asked for {device}, CUDA available: "
            f"{torch.cuda.is_available()}); there is no CPU path")
    return device


class Engine:
    def __init__(self, spec: ModelSpec, config, dtype=torch.bfloat16, device="cuda:0",
                 max_tokens: int = 8192, max_slots: int = 256):
        self.device = require_cuda(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        self.spec, self.config = spec, config
        self.model = Model(spec, self.dtype, self.device)
        self._cache_args = (max_tokens, max_slots)
        self.cache: Optional[SequenceCache] = None
        self.sampler = Sampler(self.device)
        self.use_graphs = True  # replay decode steps as CUDA graphs
        self._runners = {}
        self._graph_pool = None
        self._session = None
        self._prompts = None  # graphs of short prompt steps, made at the first one
        # scratch memory that kernels share between their CTAs is this engine's own
        self.scratch = ("engine", next(_ENGINE_NUMBERS))
        weakref.finalize(self, ops.release_scratch, self.scratch)

    # ---------------------------------------------------------------- load
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0",
                    max_tokens: int = 8192, max_slots: int = 256) -> "Engine":
        """config.json picks the architecture; model.safetensors gives the weights."""
        arch, config = load_model_config(model_dir)
        engine = cls(arch.build_spec(config), config, dtype, device, max_tokens, max_slots)
        engine.model.load(WeightFiles.open(model_dir))
        engine._make_cache()
        return engine

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", device="cuda:0",
                    max_tokens: int = 8192, max_slots: int = 256, std: float = 0.02,
                    norm_std: float = 0.0) -> "Engine":
        """Random weights made on the device (no folder): for measurements at
        sizes whose files would take long to write. `config` is a decoded
        config.json document, or a typed configuration that can write one
        (`to_json`); the architecture is the one the document names."""
        from collections.abc import Mapping
        from ..config.registry import resolve_architecture
        from ..weights.random_init import random_tensors
        import foundry_b200.models  # noqa: F401
        if isinstance(config, Mapping):
            arch = resolve_architecture(config)
            config = arch.parse_config(config)
        else:
            arch = resolve_architecture(config.to_json())
        engine = cls(arch.build_spec(config), config, dtype, device, max_tokens, max_slots)
        expected = engine.model.expected_tensors()
        store = torch.bfloat16 if engine.dtype == torch.bfloat16 else torch.float32
        # one tensor at a time: the float32 draw of a large matrix is freed at once
        tensors = {}
        for name, want in expected.items():
            tensors.update(random_tensors({name: want}, seed, dtype=store, std=std,
                                          norm_std=norm_std, device=str(engine.device)))
        engine.model.load_tensors(tensors)
        engine._make_cache()
        return engine

    def _make_cache(self) -> None:
        max_tokens, max_slots = self._cache_args
        self.cache = SequenceCache(self.model.cache_requests(), max_tokens, max_slots, self.dtype,
                                   self.device)

    # ------------------------------------------------------- StepBackend
    def open_sequence(self) -> int:
        return self.cache.open_sequence()

    def close_sequence(self, slot: int) -> None:
        self.cache.close_sequence(slot)

    def _settle(self) -> None:
        """Take back a decode step that the engine's session started on a guess
        (`DecodeSession.step_host(more=True)`), before anything else runs."""
        if self._session is not None:
            self._session.cancel_ahead()

    def free_slots(self) -> int:
        return self.cache.table.slots.free

    def free_tokens(self) -> int:
        return self.cache.free_tokens()

    def capacity_tokens(self) -> int:
        return self.cache.max_tokens

    def max_positions(self) -> int:
        return self.spec.max_positions

    # ---------------------------------------------------------------- step
    def step(self, steps: Sequence[SequenceStep]) -> torch.Tensor:
        """Run the given tokens from the cache; float32 logits [wanted, vocab]
        in the order of `steps` and of each `want`."""
        if self._is_decode(steps):
            return self._decode(steps, SamplingParams(), None, None)[1].logits().clone()
        self._settle()
        limit = self.cache.step_token_limit()
        if limit is not None and any(len(s.tokens) > limit for s in steps):
            return self._step_in_portions(steps, limit)
        if self._prompts is None:
            self._prompts = PromptRunners(self)
        if self._prompts.wants(steps):
            logits = self._prompts.step(steps)
        else:
            ctx = build_context(self.cache, steps, self.spec.vocab_size, self.device,
                                self.spec.max_positions)
            with ops.scratch_owner(self.scratch):
                logits = self.model.forward(ctx, self.cache)
        if logits.shape[0]:
            # logits leave the engine: wait for them, and let none out after a
            # kernel gave up on a bounded wait
            torch.cuda.current_stream().synchronize()
            ops.raise_on_device_failure()
        return logits

    def _step_in_portions(self, steps: Sequence[SequenceStep], limit: int) -> torch.Tensor:
        """A step in rounds of at most `limit` tokens per sequence, for models
        with a windowed cache group (see `SequenceCache.step_token_limit`): the
        logits come back as one step's would, in the order of `steps` and of
        each `want`. The whole step is validated first, so that a refused step
        changes nothing."""
        plan_check = [SequenceStep(s.slot, list(s.tokens), list(s.want)) for s in steps]
        growth = check_steps(self.cache, plan_check, self.spec.vocab_size, self.spec.max_positions)
        if not self.cache.table.can_grow(growth):
            raise CacheFull("the step needs more pages than are free")
        rows = {}  # (sequence of the step, index into its `want`) -> logits row
        longest = max(len(s.tokens) for s in plan_check)
        for start in range(0, longest, limit):
            portion, keys = [], []
            for i, s in enumerate(plan_check):
                if start >= len(s.tokens):
                    continue
                chunk = s.tokens[start:start + limit]
                wanted = [(k, w - start) for k, w in enumerate(s.want)
                          if start <= w < start + len(chunk)]
                portion.append(SequenceStep(s.slot, chunk, [w for _, w in wanted]))
                keys.extend((i, k) for k, _ in wanted)
            logits = self.step(portion)
            for row, key in zip(logits, keys):
                rows[key] = row
        ordered = [rows[(i, k)] for i, s in enumerate(plan_check) for k in range(len(s.want))]
        if not ordered:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        return torch.stack(ordered)

    def step_select(self, steps: Sequence[SequenceStep], params: SamplingParams,
                    keys: Sequence[int], counts: Sequence[int], more: bool = False) -> List[int]:
        """A step whose wanted logits are turned into tokens on the device;
        only the token ids cross to the host. `more`: the caller expects to
        come back with the same sequences, each with the token returned here
        (a generation loop whose rows all go on unless a stop token ends one);
        single-token steps then start the next step before they return."""
        if self._is_decode(steps):
            return self._decode(steps, params, keys, counts, more)[0]
        logits = self.step(steps)
        tokens = self.sampler.select(logits, params, keys, counts)
        return tokens.tolist()

    @staticmethod
    def _is_decode(steps: Sequence[SequenceStep]) -> bool:
        return len(steps) > 0 and all(len(s.tokens) == 1 and list(s.want) == [0] for s in steps)

    def _decode(self, steps, params, keys, counts, more: bool = False):
        """One token per sequence, through a `DecodeSession` (fixed buffers,
        replayed graph); returns (host tokens, the session)."""
        slots = [s.slot for s in steps]
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        for s in steps:
            if not self.cache.table.slots.is_held(s.slot):
                raise ValueError(f"slot {s.slot} is not open")
            if not 0 <= int(s.tokens[0]) < self.spec.vocab_size:
                raise ValueError(f"token id {s.tokens[0]} is outside the vocabulary of "
                                 f"{self.spec.vocab_size}")
        keys = list(range(len(slots))) if keys is None else list(keys)
        session = self._session
        if session is None or session.slots != slots or session.sampling != params \
                or session.keys != keys:
            self._settle()
            session = self._session = DecodeSession(self, slots, params, keys, counts)
        tokens = session.step_host([int(s.tokens[0]) for s in steps], more, counts)
        return tokens, session

    # -------------------------------------------------------------- decode
    def decode_session(self, slots: Sequence[int], sampling: SamplingParams = SamplingParams(),
                       keys: Optional[Sequence[int]] = None,
                       counts: Optional[Sequence[int]] = None) -> "DecodeSession":
        self._settle()
        return DecodeSession(self, slots, sampling, keys, counts)

    def decode_runner(self, bucket: int, width: int, unequal: bool = False) -> "DecodeRunner":
        """The captured step for `bucket` rows, page tables `width` pages wide, and
        sequences of about equal or of unequal lengths (the attention shares its
        work differently)."""
        key = (bucket, width) if not unequal else (bucket, width, "unequal")
        if key not in self._runners:
            self._runners[key] = DecodeRunner(self, bucket, width, unequal)
        return self._runners[key]

    def graph_pool(self):
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # ------------------------------------------------------------ generate
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_token_id: Optional[Sequence[int]] = None,
                 sampling: SamplingParams = SamplingParams(), max_batch: Optional[int] = None,
                 ignore_eos: bool = False) -> loop.Generation:
        stops = self.spec.eos_token_ids if eos_token_id is None else tuple(eos_token_id)
        return loop.generate(self, prompts, max_new_tokens, stops, sampling, max_batch, ignore_eos)
