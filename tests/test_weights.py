"""Weights: the safetensors reader and writer, the one error that lists all
that is wrong with a folder, dtype rules, and the random-weights mode.
File-level cases follow the reference's own (src/weights/mod.rs:410-975)."""
import json
import os
import struct

import pytest
import torch
from safetensors.torch import load_file, save_file as st_save

import tiny
from foundry_b200.config import LlamaConfig
from foundry_b200.engine.model import expected_tensors
from foundry_b200.models.llama import build_llama_spec
from foundry_b200.weights import (WeightFiles, WeightsMismatch, check_against,
                                  save_file, stored_to_run_dtype, write_model_folder)
from foundry_b200.weights import safetensors_io as sio
from foundry_b200.weights.random_init import random_tensors


def spec_of(name):
    return build_llama_spec(LlamaConfig.parse(tiny.CONFIGS[name]))


def test_written_files_are_read_by_the_safetensors_package_and_back(tmp_path):
    tensors = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(6, dtype=torch.int32),
               "c": torch.randn(4), "empty": torch.zeros(0, 2)}
    path = str(tmp_path / "model.safetensors")
    save_file(tensors, path, metadata={"format": "pt"})
    theirs = load_file(path)
    ours = WeightFiles.open(str(tmp_path))
    assert sorted(ours.names()) == sorted(tensors)
    for name, t in tensors.items():
        assert torch.equal(theirs[name], t) and torch.equal(ours.tensor(name), t)
        assert ours.tensor(name).dtype == t.dtype
    assert ours.numel() == sum(t.numel() for t in tensors.values())
    # and a file their writer made
    st_save({"x": torch.ones(2, 2)}, str(tmp_path / "model.safetensors"))
    assert torch.equal(WeightFiles.open(str(tmp_path)).tensor("x"), torch.ones(2, 2))


def test_sharded_folder_and_its_index_checks(tmp_path):
    save_file({"a": torch.ones(2)}, str(tmp_path / "s1.safetensors"))
    save_file({"b": torch.zeros(3)}, str(tmp_path / "s2.safetensors"))
    index = {"metadata": {"total_size": 20}, "weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}
    (tmp_path / sio.INDEX_FILE).write_text(json.dumps(index))
    files = WeightFiles.open(str(tmp_path))
    assert sorted(files.names()) == ["a", "b"] and files.nbytes() == 20
    index["weight_map"]["a"] = "s2.safetensors"
    (tmp_path / sio.INDEX_FILE).write_text(json.dumps(index))
    with pytest.raises(sio.IndexMismatch):
        WeightFiles.open(str(tmp_path))
    index["weight_map"] = {"a": "../s1.safetensors"}
    (tmp_path / sio.INDEX_FILE).write_text(json.dumps(index))
    with pytest.raises(sio.InvalidShardName):
        WeightFiles.open(str(tmp_path))
    index = {"metadata": {"total_size": 21}, "weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}
    (tmp_path / sio.INDEX_FILE).write_text(json.dumps(index))
    with pytest.raises(sio.ByteCountMismatch):
        WeightFiles.open(str(tmp_path))
    save_file({"a": torch.ones(2)}, str(tmp_path / "s2.safetensors"))
    index = {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}
    (tmp_path / sio.INDEX_FILE).write_text(json.dumps(index))
    with pytest.raises(sio.DuplicateTensor):
        WeightFiles.open(str(tmp_path))


def _raw(tmp_path, header: dict, data: bytes = b""):
    raw = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(raw)) + raw + data)
    return str(tmp_path)


def test_malformed_files(tmp_path):
    (tmp_path / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(sio.InvalidHeader):
        WeightFiles.open(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(sio.InvalidHeader):
        WeightFiles.open(str(tmp_path))
    with pytest.raises(sio.UnknownDType):
        WeightFiles.open(_raw(tmp_path, {"x": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}, b"\0"))
    with pytest.raises(sio.ByteCountMismatch):
        WeightFiles.open(_raw(tmp_path, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(sio.InvalidHeader):  # ends beyond the file
        WeightFiles.open(_raw(tmp_path, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4))
    with pytest.raises(sio.InvalidShape):
        WeightFiles.open(_raw(tmp_path, {"x": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 0]}}))
    with pytest.raises(sio.ShardOpen):
        WeightFiles.open(str(tmp_path / "nowhere"))
    files = WeightFiles.open(_raw(tmp_path, {"__metadata__": {"k": "v"}}))
    assert files.names() == []
    with pytest.raises(sio.TensorNotFound):
        files.tensor("x")


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    spec = spec_of("tiny_a")
    want = expected_tensors(spec)
    tensors = random_tensors(want, 0)
    del tensors["model.norm.weight"]
    del tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64).bfloat16()
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64).bfloat16()
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.float16)
    tensors["lm_head.weight"] = torch.zeros(256, 64).bfloat16()  # tied: may be present, unused
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsMismatch) as info:
        check_against(WeightFiles.open(str(tmp_path)), want, spec.ignorable_tensors)
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    assert e.wrong_dtype == [("model.layers.1.input_layernorm.weight", "F16")]
    for needle in ("missing", "unexpected", "wrong shape", "wrong dtype", "q_proj.bias",
                   "model.norm.weight", "[32, 64]"):
        assert needle in str(e)


def test_an_untied_model_needs_its_head(tmp_path):
    spec = spec_of("tiny_b")
    tensors = random_tensors(expected_tensors(spec), 1)
    del tensors["lm_head.weight"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsMismatch, match="lm_head.weight"):
        check_against(WeightFiles.open(str(tmp_path)), expected_tensors(spec), spec.ignorable_tensors)


def test_the_expected_list_is_the_hugging_face_one():
    names = set(expected_tensors(spec_of("tiny_b")))
    assert len(names) == 2 + 1 + 3 * 9
    for n in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight",
              "model.layers.2.self_attn.q_proj.weight", "model.layers.0.mlp.down_proj.weight",
              "model.layers.1.post_attention_layernorm.weight"):
        assert n in names
    e = expected_tensors(spec_of("tiny_b"))
    assert e["model.layers.0.self_attn.q_proj.weight"].shape == (192, 96)
    assert e["model.layers.0.self_attn.o_proj.weight"].shape == (96, 192)
    assert e["model.layers.0.self_attn.k_proj.weight"].shape == (96, 96)


def test_dtype_rules():
    bf, f32 = torch.bfloat16, torch.float32
    assert stored_to_run_dtype(bf, bf) == bf
    assert stored_to_run_dtype(f32, bf) == f32  # a tensor stored in 32 bits stays so
    assert stored_to_run_dtype(bf, f32) == f32 and stored_to_run_dtype(f32, f32) == f32
    assert stored_to_run_dtype(torch.int64, bf) == torch.int32


def test_random_weights_mode_is_deterministic_and_per_tensor(tmp_path):
    a = write_model_folder(str(tmp_path / "a"), LlamaConfig.parse(tiny.CONFIGS["tiny_a"]), 0)
    b = write_model_folder(str(tmp_path / "b"), LlamaConfig.parse(tiny.CONFIGS["tiny_a"]), 0)
    c = write_model_folder(str(tmp_path / "c"), LlamaConfig.parse(tiny.CONFIGS["tiny_a"]), 1)
    fa, fb_, fc = (load_file(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert all(torch.equal(fa[k], fb_[k]) for k in fa)
    assert not torch.equal(fa["model.embed_tokens.weight"], fc["model.embed_tokens.weight"])
    assert fa["model.embed_tokens.weight"].dtype == torch.bfloat16
    w = fa["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = fa["model.norm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.03 < float(n.std()) < 0.2
    assert LlamaConfig.open(a) == LlamaConfig.parse(tiny.CONFIGS["tiny_a"])
    check_against(WeightFiles.open(a), expected_tensors(spec_of("tiny_a")), ())
