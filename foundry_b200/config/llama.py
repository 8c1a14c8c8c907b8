"""Typed configuration of the Llama dense decoder, read from config.json.

Every size and constant of the model comes from here; no other file holds one.
The key set and the validation order follow the reference
(src/models/llama/config.rs:38-201). Differences, all widening:

* `head_dim` need not satisfy heads x head_dim == hidden_size
  (the reference rejects that at config.rs:141-155);
* `tie_word_embeddings = false` is accepted (rejected at config.rs:177-180);
* keys a real model folder may omit get the conventional defaults
  (`num_key_value_heads`, `tie_word_embeddings`, `rope_theta`, `eos_token_id`);
* keys the reference ignores (`hidden_act`, `attention_bias`, `mlp_bias`,
  `pretraining_tp`) are read and rejected when they ask for a path that does
  not exist.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from . import errors
from .files import decode_json, read_config_json

MODEL_TYPE = "llama"  # src/models/llama/config.rs:11
ROPE_TYPE_LLAMA3 = "llama3"  # src/models/llama/config.rs:12


@dataclass(frozen=True)
class Llama3RopeScaling:
    """Frequency-dependent RoPE scaling (src/models/llama/config.rs:30-36)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_json(self) -> dict:
        return {
            "rope_type": ROPE_TYPE_LLAMA3,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    max_position_embeddings: int
    vocab_size: int
    tie_word_embeddings: bool
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architectures: Tuple[str, ...] = ("LlamaForCausalLM",)
    model_type: str = MODEL_TYPE
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ read
    @classmethod
    def open(cls, directory: str) -> "LlamaConfig":
        """Read `<directory>/config.json` (src/models/llama/config.rs:82-104)."""
        return cls.parse(read_config_json(directory))

    @classmethod
    def parse(cls, source) -> "LlamaConfig":
        """Build from JSON text, bytes or an already decoded mapping."""
        doc = decode_json(source)
        req = _Reader(doc)
        model_type = req.string("model_type")
        if model_type != MODEL_TYPE:
            raise errors.ModelType(f"model_type is {model_type!r}, expected {MODEL_TYPE!r}")
        hidden = req.positive("hidden_size")
        inter = req.positive("intermediate_size")
        layers = req.positive("num_hidden_layers")
        heads = req.positive("num_attention_heads")
        kv_heads = req.non_negative("num_key_value_heads", default=heads)
        eps = req.number("rms_norm_eps")
        max_pos = req.positive("max_position_embeddings")
        vocab = req.positive("vocab_size")
        theta = req.number("rope_theta", default=10000.0)
        tie = req.boolean("tie_word_embeddings", default=False)
        head_dim = req.optional_int("head_dim")
        if head_dim is None:
            if hidden % heads != 0:
                raise errors.HeadDimInvalid(
                    f"head_dim is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}"
                )
            head_dim = hidden // heads
        if head_dim <= 0 or head_dim % 2 != 0:
            raise errors.HeadDimInvalid(f"head_dim {head_dim} is not a positive even number")
        if kv_heads == 0 or heads % kv_heads != 0:
            raise errors.HeadRatio(
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}"
            )
        scaling = _parse_rope_scaling(doc.get("rope_scaling"))
        if not (eps > 0.0):
            raise errors.ConfigJson(f"rms_norm_eps must be positive, got {eps}")
        if not (theta > 0.0):
            raise errors.ConfigJson(f"rope_theta must be positive, got {theta}")
        _reject_unsupported(doc)
        eos = _parse_token_ids(doc.get("eos_token_id"), "eos_token_id")
        bos = req.optional_int("bos_token_id")
        archs = doc.get("architectures") or ["LlamaForCausalLM"]
        if not isinstance(archs, list) or not all(isinstance(a, str) for a in archs):
            raise errors.ConfigJson("architectures must be a list of strings")
        known = {f for f in cls.__dataclass_fields__}  # type: ignore[attr-defined]
        extra = {k: v for k, v in doc.items() if k not in known}
        return cls(
            hidden_size=hidden,
            intermediate_size=inter,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(eps),
            rope_theta=float(theta),
            rope_scaling=scaling,
            max_position_embeddings=max_pos,
            vocab_size=vocab,
            tie_word_embeddings=tie,
            eos_token_id=eos,
            bos_token_id=bos,
            torch_dtype=doc.get("torch_dtype") if isinstance(doc.get("torch_dtype"), str) else None,
            architectures=tuple(archs),
            extra=extra,
        )

    # ----------------------------------------------------------------- write
    def to_json(self) -> dict:
        """The config.json that `parse` reads back to an equal object."""
        doc = {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_json(),
            "max_position_embeddings": self.max_position_embeddings,
            "vocab_size": self.vocab_size,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.eos_token_id:
            doc["eos_token_id"] = (
                self.eos_token_id[0] if len(self.eos_token_id) == 1 else list(self.eos_token_id)
            )
        if self.bos_token_id is not None:
            doc["bos_token_id"] = self.bos_token_id
        if self.torch_dtype is not None:
            doc["torch_dtype"] = self.torch_dtype
        return doc

    # ------------------------------------------------------------ arithmetic
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameter_count(self) -> int:
        """Stored parameters (a tied output head counts once)."""
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = h * (self.q_size + 2 * self.kv_size) + self.q_size * h + 3 * h * i + 2 * h
        total = v * h + self.num_hidden_layers * per_layer + h
        if not self.tie_word_embeddings:
            total += v * h
        return total


# ---------------------------------------------------------------- helpers


class _Reader:
    """Typed access to the decoded document; a missing or mistyped required
    key is `ConfigJson`, as serde reports it in the reference."""

    def __init__(self, doc: Mapping[str, Any]):
        self.doc = doc

    def _get(self, key, default):
        if key not in self.doc or self.doc[key] is None:
            if default is _MISSING:
                raise errors.ConfigJson(f"config.json lacks the required key {key!r}")
            return default
        return self.doc[key]

    def string(self, key, default=None):
        value = self._get(key, _MISSING if default is None else default)
        if not isinstance(value, str):
            raise errors.ConfigJson(f"{key} must be a string")
        return value

    def _int(self, key, default):
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, int):
            raise errors.ConfigJson(f"{key} must be an integer, got {value!r}")
        return value

    def positive(self, key, default=None):
        value = self._int(key, _MISSING if default is None else default)
        if value <= 0:
            raise errors.ConfigJson(f"{key} must be positive, got {value}")
        return value

    def non_negative(self, key, default=None):
        value = self._int(key, _MISSING if default is None else default)
        if value < 0:
            raise errors.ConfigJson(f"{key} must not be negative, got {value}")
        return value

    def optional_int(self, key):
        if key not in self.doc or self.doc[key] is None:
            return None
        return self._int(key, _MISSING)

    def number(self, key, default=None):
        value = self._get(key, _MISSING if default is None else default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise errors.ConfigJson(f"{key} must be a number, got {value!r}")
        return float(value)

    def boolean(self, key, default=None):
        value = self._get(key, _MISSING if default is None else default)
        if not isinstance(value, bool):
            raise errors.ConfigJson(f"{key} must be true or false, got {value!r}")
        return value


_MISSING = object()


def _parse_rope_scaling(raw) -> Optional[Llama3RopeScaling]:
    """`rope_scaling` absent or null means unscaled frequencies
    (src/models/llama/config.rs:49, 168-176). The older key `type` is read as
    `rope_type`; `default` also means unscaled."""
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise errors.ConfigJson("rope_scaling must be an object or null")
    rope_type = raw.get("rope_type", raw.get("type"))
    if rope_type == "default":
        return None
    if rope_type != ROPE_TYPE_LLAMA3:
        raise errors.RopeType(f"rope_scaling.rope_type is {rope_type!r}; only 'llama3' is built")
    reader = _Reader(raw)
    scaling = Llama3RopeScaling(
        factor=reader.number("factor"),
        low_freq_factor=reader.number("low_freq_factor"),
        high_freq_factor=reader.number("high_freq_factor"),
        original_max_position_embeddings=reader.positive("original_max_position_embeddings"),
    )
    if scaling.factor <= 0 or scaling.low_freq_factor <= 0:
        raise errors.ConfigJson("rope_scaling factors must be positive")
    if scaling.high_freq_factor == scaling.low_freq_factor:
        raise errors.ConfigJson("rope_scaling high_freq_factor equals low_freq_factor")
    return scaling


def _parse_token_ids(raw, key) -> Tuple[int, ...]:
    """An integer or a list of them (src/models/llama/config.rs:65-79);
    absent means the model never stops by itself."""
    if raw is None:
        return ()
    items = raw if isinstance(raw, list) else [raw]
    for item in items:
        if isinstance(item, bool) or not isinstance(item, int) or item < 0:
            raise errors.ConfigJson(f"{key} must hold non-negative integers, got {item!r}")
    return tuple(items)


def _reject_unsupported(doc: Mapping[str, Any]) -> None:
    act = doc.get("hidden_act", "silu")
    if act != "silu":
        raise errors.UnsupportedOption(f"hidden_act {act!r}: only 'silu' is built")
    for key in ("attention_bias", "mlp_bias"):
        if doc.get(key, False):
            raise errors.UnsupportedOption(f"{key} = true: projections carry no bias here")
    if doc.get("pretraining_tp", 1) not in (1, None):
        raise errors.UnsupportedOption("pretraining_tp other than 1 is not built")
