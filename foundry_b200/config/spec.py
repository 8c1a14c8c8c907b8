"""What an architecture hands to the engine: a description made of data.

An architecture turns its typed configuration into a `ModelSpec`: for every
layer the names and parameters of its parts (mixer, feed-forward, norms, block
arrangement), and the order in which layers run. Nothing below this file knows
a model's name; parts are looked up by `PartSpec.kind` in the part registries
(foundry_b200/parts/registry.py).

The reference hard-wires one arrangement (src/models/llama/model.rs:254-278:
norm, attention, add, norm, MLP, add; the same for every layer, each layer run
once in index order, model.rs:180-192). Here that arrangement is one value of
this data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part by registry name with its sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward.

    `prefix` is the layer's tensor-name prefix in the weight files
    (`model.layers.3`); parts append their own names to it.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    # tensor-name component of each part under `prefix`, e.g. mixer -> "self_attn"
    names: Mapping[str, str] = field(default_factory=lambda: {
        "mixer": "mixer", "feed_forward": "feed_forward",
        "mixer_norm": "mixer_norm", "feed_forward_norm": "feed_forward_norm"})


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    `layer` indexes `ModelSpec.layers` (a layer may be named by several
    entries: its weights are then shared). `cache` names the cache entry the
    run's mixer uses; `writes_cache = False` makes the mixer read what another
    run wrote there instead of appending its own keys and values.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    output_head_name: Optional[str]  # None: the output head is the embedding table
    eos_token_ids: Tuple[int, ...] = ()
    ignorable_tensors: Tuple[str, ...] = ()  # fnmatch patterns that may be present unused

    def cache_entry_count(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)

    def validate(self) -> None:
        writers: Dict[int, int] = {}
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{position}] names layer {entry.layer}, "
                                 f"the model has {len(self.layers)}")
            if entry.cache < 0:
                raise ValueError(f"schedule[{position}] names cache entry {entry.cache}")
            if entry.writes_cache:
                if entry.cache in writers:
                    raise ValueError(
                        f"cache entry {entry.cache} is written by schedule[{writers[entry.cache]}] "
                        f"and schedule[{position}]")
                writers[entry.cache] = position
        for position, entry in enumerate(self.schedule):
            if not entry.writes_cache:
                if entry.cache not in writers or writers[entry.cache] > position:
                    raise ValueError(
                        f"schedule[{position}] reads cache entry {entry.cache} before a run wrote it")


def default_schedule(layer_count: int) -> Tuple[ScheduleEntry, ...]:
    """Each layer once, in order, with a cache entry of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(layer_count))
