"""Typed configurations, the description an architecture produces, and the
registry from architecture name to both."""
from . import errors
from .errors import ConfigError
from .files import CONFIG_FILE, read_config_json
from .llama import Llama3RopeScaling, LlamaConfig
from .registry import (Architecture, register_architecture, registered_architectures,
                       resolve_architecture, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule


def load_model_config(directory: str):
    """Read `<directory>/config.json` and return `(architecture, typed config)`;
    the model class is chosen by the file, never by the caller."""
    import foundry_b200.models  # noqa: F401  (registers the built-in architectures)

    doc = read_config_json(directory)
    arch = resolve_architecture(doc)
    return arch, arch.parse_config(doc)


__all__ = [
    "errors", "ConfigError", "CONFIG_FILE", "Llama3RopeScaling", "LlamaConfig", "read_config_json",
    "Architecture", "register_architecture", "registered_architectures", "resolve_architecture",
    "unregister_architecture", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
    "default_schedule", "load_model_config",
]
