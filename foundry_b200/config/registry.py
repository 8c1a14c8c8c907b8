"""One registry from an architecture's name to its configuration and model.

The reference dispatches with a single hard check, `model_type == "llama"`
(src/models/llama/config.rs:208-215), and `src/models/mod.rs:1` declares the
single module. Here config.json's `architectures[0]` (falling back to
`model_type`) is looked up in a table, so that another architecture is one
`register_architecture` call and no edit of the engine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping

from . import errors
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str  # config.json `architectures[0]`
    model_type: str  # config.json `model_type`
    parse_config: Callable[[Mapping[str, Any]], Any]  # decoded json -> typed config
    build_spec: Callable[[Any], ModelSpec]  # typed config -> description of the model


_BY_NAME: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> Architecture:
    if arch.name in _BY_NAME and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _BY_NAME[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _BY_NAME.pop(name, None)


def registered_architectures() -> List[str]:
    return sorted(_BY_NAME)


def resolve_architecture(doc: Mapping[str, Any]) -> Architecture:
    """Pick the architecture a decoded config.json names."""
    import foundry_b200.models  # noqa: F401  (registers the built-in architectures)
    archs = doc.get("architectures")
    if isinstance(archs, list):
        for name in archs:
            if name in _BY_NAME:
                return _BY_NAME[name]
    model_type = doc.get("model_type")
    if not isinstance(archs, list) or not archs:
        for arch in _BY_NAME.values():
            if arch.model_type == model_type:
                return arch
    raise errors.UnknownArchitecture(
        f"config.json names architectures={archs!r}, model_type={model_type!r}; "
        f"registered: {registered_architectures()}")
