"""The Llama dense decoder as data: config.json -> `ModelSpec`.

Per layer (src/models/llama/model.rs:254-278): RMSNorm -> grouped-query
attention with rotary positions -> residual add -> RMSNorm -> SwiGLU -> residual
add; then a final RMSNorm and the output head (model.rs:117-122, 192), which is
the embedding table when `tie_word_embeddings` is set (model.rs:62). Tensor
names are the Hugging Face ones the reference loads (model.rs:144, 153, 158,
230-245; attention.rs:50-55; mlp.rs:34-38).
"""
from __future__ import annotations

from ..config.llama import MODEL_TYPE, LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule

ARCHITECTURE = "LlamaForCausalLM"
# tensor-name components under `model.layers.<i>` (src/models/llama/model.rs:226-245)
HF_NAMES = {"mixer": "self_attn", "feed_forward": "mlp", "mixer_norm": "input_layernorm",
            "feed_forward_norm": "post_attention_layernorm"}


def build_llama_spec(config: LlamaConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"size": config.hidden_size, "eps": config.rms_norm_eps})
    if config.rope_scaling is None:
        rope = PartSpec("rope", {"head_dim": config.head_dim, "theta": config.rope_theta})
    else:
        s = config.rope_scaling
        rope = PartSpec("rope_llama3", {
            "head_dim": config.head_dim,
            "theta": config.rope_theta,
            "factor": s.factor,
            "low_freq_factor": s.low_freq_factor,
            "high_freq_factor": s.high_freq_factor,
            "original_max_position_embeddings": s.original_max_position_embeddings,
        })
    mixer = PartSpec("gqa_attention", {
        "hidden_size": config.hidden_size,
        "num_heads": config.num_attention_heads,
        "num_kv_heads": config.num_key_value_heads,
        "head_dim": config.head_dim,
        "position_encoding": rope,
        "window": None,
    })
    feed_forward = PartSpec("swiglu", {
        "hidden_size": config.hidden_size,
        "intermediate_size": config.intermediate_size,
    })
    block = PartSpec("pre_norm_residual", {})
    layers = tuple(
        LayerSpec(
            prefix=f"model.layers.{i}",
            block=block,
            mixer=mixer,
            feed_forward=feed_forward,
            mixer_norm=norm,
            feed_forward_norm=norm,
            names=HF_NAMES,
        )
        for i in range(config.num_hidden_layers)
    )
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        layers=layers,
        schedule=default_schedule(config.num_hidden_layers),
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_prefix="model.norm",
        output_head_name=None if config.tie_word_embeddings else "lm_head.weight",
        eos_token_ids=config.eos_token_id,
        ignorable_tensors=(
            ("lm_head.weight",) if config.tie_word_embeddings else ()
        ) + ("*.rotary_emb.inv_freq",),
    )
    spec.validate()
    return spec


LLAMA = register_architecture(Architecture(
    name=ARCHITECTURE,
    model_type=MODEL_TYPE,
    parse_config=LlamaConfig.parse,
    build_spec=build_llama_spec,
), replace=True)
