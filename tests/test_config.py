"""Configuration and registry: what is read, what is defaulted, what is refused.

The 3B literal is the key set of a published Llama 3.2 config.json, as the
reference's own parse test uses it (src/models/llama/config.rs:230-264); the
expectations on defaults and rejections follow config.rs:320-451.
"""
import json

import pytest

import tiny
from foundry_b200.config import (LlamaConfig, errors, load_model_config, register_architecture,
                                 registered_architectures, resolve_architecture,
                                 unregister_architecture, Architecture)
from foundry_b200.models.llama import build_llama_spec

LLAMA_3B = {
    "architectures": ["LlamaForCausalLM"], "attention_bias": False, "attention_dropout": 0.0,
    "bos_token_id": 128000, "eos_token_id": [128001, 128008, 128009], "head_dim": 128,
    "hidden_act": "silu", "hidden_size": 3072, "initializer_range": 0.02,
    "intermediate_size": 8192, "max_position_embeddings": 131072, "mlp_bias": False,
    "model_type": "llama", "num_attention_heads": 24, "num_hidden_layers": 28,
    "num_key_value_heads": 8, "pretraining_tp": 1, "rms_norm_eps": 1e-05,
    "rope_scaling": {"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "rope_theta": 500000.0, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
    "transformers_version": "4.45.0.dev0", "use_cache": True, "vocab_size": 128256,
}


def test_the_3b_config_parses_to_its_sizes():
    c = LlamaConfig.parse(json.dumps(LLAMA_3B))
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (3072, 8192, 28)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (24, 8, 128)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 500000.0
    assert c.rope_scaling.factor == 32.0 and c.rope_scaling.original_max_position_embeddings == 8192
    assert c.eos_token_id == (128001, 128008, 128009) and c.bos_token_id == 128000
    assert c.tie_word_embeddings and c.vocab_size == 128256
    # the parameter count of the published model (benchmarks/*/report.json:8-9)
    assert c.parameter_count() == 3_212_749_824


def test_defaults_for_keys_a_folder_may_omit():
    doc = {k: v for k, v in tiny.CONFIGS["tiny_a"].items()
           if k not in ("head_dim", "rope_scaling", "num_key_value_heads", "tie_word_embeddings",
                        "rope_theta", "eos_token_id")}
    c = LlamaConfig.parse(doc)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_scaling is None
    assert c.tie_word_embeddings is False and c.rope_theta == 10000.0 and c.eos_token_id == ()


def test_a_single_stop_token_becomes_a_list():
    assert LlamaConfig.parse(tiny.CONFIGS["tiny_a"]).eos_token_id == (7,)
    assert LlamaConfig.parse(tiny.CONFIGS["tiny_b"]).eos_token_id == (3, 5)


def test_head_dim_need_not_divide_the_hidden_size():
    c = LlamaConfig.parse(tiny.CONFIGS["tiny_b"])
    assert c.num_attention_heads * c.head_dim == 192 != c.hidden_size


def test_round_trip_through_json():
    for doc in (LLAMA_3B, tiny.CONFIGS["tiny_a"], tiny.CONFIGS["tiny_b"]):
        c = LlamaConfig.parse(doc)
        assert LlamaConfig.parse(json.dumps(c.to_json())) == c


@pytest.mark.parametrize("change, error", [
    ({"model_type": "mistral"}, errors.ModelType),
    ({"num_key_value_heads": 3}, errors.HeadRatio),
    ({"num_key_value_heads": 0}, errors.HeadRatio),
    ({"head_dim": 15}, errors.HeadDimInvalid),
    ({"head_dim": 0}, errors.HeadDimInvalid),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, errors.RopeType),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, errors.ConfigJson),
    ({"hidden_act": "gelu"}, errors.UnsupportedOption),
    ({"attention_bias": True}, errors.UnsupportedOption),
    ({"mlp_bias": True}, errors.UnsupportedOption),
    ({"hidden_size": "64"}, errors.ConfigJson),
    ({"vocab_size": 0}, errors.ConfigJson),
    ({"rms_norm_eps": 0.0}, errors.ConfigJson),
    ({"eos_token_id": -1}, errors.ConfigJson),
])
def test_rejections(change, error):
    with pytest.raises(error):
        LlamaConfig.parse({**tiny.CONFIGS["tiny_a"], **change})


@pytest.mark.parametrize("key", ["model_type", "hidden_size", "intermediate_size",
                                 "num_hidden_layers", "num_attention_heads", "rms_norm_eps",
                                 "max_position_embeddings", "vocab_size"])
def test_a_missing_required_key_is_named(key):
    doc = {k: v for k, v in tiny.CONFIGS["tiny_a"].items() if k != key}
    with pytest.raises(errors.ConfigJson, match=key):
        LlamaConfig.parse(doc)


def test_not_json_and_not_an_object():
    with pytest.raises(errors.ConfigJson):
        LlamaConfig.parse(b"{not json")
    with pytest.raises(errors.ConfigJson):
        LlamaConfig.parse("[1, 2]")


def test_open_reads_the_folder_and_limits_the_size(tmp_path):
    with pytest.raises(errors.ConfigRead):
        LlamaConfig.open(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tiny.CONFIGS["tiny_b"]))
    assert LlamaConfig.open(str(tmp_path)).hidden_size == 96
    (tmp_path / "config.json").write_text(" " * (1024 * 1024 + 1))
    with pytest.raises(errors.ConfigTooLarge):
        LlamaConfig.open(str(tmp_path))


def test_registry_picks_the_model_by_config(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps(tiny.CONFIGS["tiny_a"]))
    arch, config = load_model_config(str(tmp_path))
    assert arch.name == "LlamaForCausalLM" and config.hidden_size == 64
    # without `architectures`, model_type decides
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(errors.UnknownArchitecture, match="LlamaForCausalLM"):
        resolve_architecture({"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2"})


def test_another_architecture_is_one_registration():
    arch = Architecture("ToyForCausalLM", "toy", LlamaConfig.parse, build_llama_spec)
    register_architecture(arch)
    try:
        with pytest.raises(ValueError):
            register_architecture(arch)
        assert resolve_architecture({"architectures": ["ToyForCausalLM"]}) is arch
    finally:
        unregister_architecture("ToyForCausalLM")


def test_the_description_is_data():
    spec = build_llama_spec(LlamaConfig.parse(tiny.CONFIGS["tiny_b"]))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].mixer.kind == "gqa_attention"
    assert spec.layers[0].mixer.params["position_encoding"].kind == "rope_llama3"
    assert spec.layers[1].feed_forward.params["intermediate_size"] == 256
    assert spec.output_head_name == "lm_head.weight"
    tied = build_llama_spec(LlamaConfig.parse(tiny.CONFIGS["tiny_a"]))
    assert tied.output_head_name is None and tied.layers[0].mixer.params["position_encoding"].kind == "rope"


def test_schedule_validation():
    from dataclasses import replace
    from foundry_b200.config import ScheduleEntry
    spec = build_llama_spec(LlamaConfig.parse(tiny.CONFIGS["tiny_a"]))
    # a layer named twice, the second run reading the first run's cache
    replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1),
                            ScheduleEntry(0, 0, writes_cache=False))).validate()
    with pytest.raises(ValueError, match="before"):
        replace(spec, schedule=(ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1))).validate()
    with pytest.raises(ValueError, match="written by"):
        replace(spec, schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0))).validate()
    with pytest.raises(ValueError, match="names layer"):
        replace(spec, schedule=(ScheduleEntry(5, 0),)).validate()
