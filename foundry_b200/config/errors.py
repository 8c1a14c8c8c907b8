"""Configuration errors.

The names follow the reference's `LlamaConfigError` variants
(src/models/llama/error.rs:5-30) so that a caller switching engines meets the
same failure classes; two reference variants are gone because the limits they
guard are lifted here (`HiddenSizeMismatch`: heads x head_dim may differ from
the hidden size; `UntiedEmbeddings`: a separate output head is supported).
"""


class ConfigError(ValueError):
    """Base class of every configuration failure."""


class ConfigRead(ConfigError):
    """config.json is missing or unreadable (src/models/llama/config.rs:84-92)."""


class ConfigTooLarge(ConfigError):
    """config.json is larger than 1 MiB (src/models/llama/config.rs:93-102)."""


class ConfigJson(ConfigError):
    """Not JSON, or a required key is absent or of the wrong type
    (src/models/llama/config.rs:203-206)."""


class ModelType(ConfigError):
    """`model_type` is not the one the architecture expects
    (src/models/llama/config.rs:208-215)."""


class HeadRatio(ConfigError):
    """Attention heads are not a multiple of key-value heads
    (src/models/llama/config.rs:156-167)."""


class HeadDimInvalid(ConfigError):
    """Head size is not a positive even number
    (src/models/llama/rotary_emb.rs:140-146)."""


class RopeType(ConfigError):
    """`rope_scaling.rope_type` is not one this architecture implements
    (src/models/llama/config.rs:168-176)."""


class UnsupportedOption(ConfigError):
    """A key asks for a code path that does not exist (biases, another
    activation): the reference has no such path either (src/nn/linear.rs:9-11,
    src/models/llama/mlp.rs:56)."""


class UnknownArchitecture(ConfigError):
    """No registered architecture matches config.json."""
