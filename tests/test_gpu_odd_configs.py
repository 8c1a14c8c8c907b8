"""Configurations with awkward sizes, each replayed in three cuttings against
the plain model in both dtypes: head sizes in steps of 16 that the tensor-core
attention does not build (48, 80, 96), one kv head for all heads, as many kv
heads as heads, widths, feed-forward widths and vocabularies that are odd or
no multiple of 8 (which sends products to the CUDA-core kernel), a single
layer, a large eps, partial last pages."""
import pytest

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "rope_scaling": None,
        "max_position_embeddings": 256}
ODD = {
    "head48_mqa": dict(num_hidden_layers=2, hidden_size=80, num_attention_heads=5,
                       num_key_value_heads=1, head_dim=48, intermediate_size=200, vocab_size=301,
                       rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True),
    "head80_mha": dict(num_hidden_layers=1, hidden_size=100, num_attention_heads=3,
                       num_key_value_heads=3, head_dim=80, intermediate_size=177, vocab_size=515,
                       rms_norm_eps=1e-3, rope_theta=777.0, tie_word_embeddings=False),
    "head96_wide_group": dict(num_hidden_layers=2, hidden_size=72, num_attention_heads=8,
                              num_key_value_heads=2, head_dim=96, intermediate_size=90,
                              vocab_size=1000, rms_norm_eps=1e-6, rope_theta=1e6,
                              tie_word_embeddings=True,
                              rope_scaling={"rope_type": "llama3", "factor": 4.0,
                                            "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                                            "original_max_position_embeddings": 32}),
    "head64_group8": dict(num_hidden_layers=2, hidden_size=264, num_attention_heads=8,
                          num_key_value_heads=1, head_dim=64, intermediate_size=136,
                          vocab_size=777, rms_norm_eps=1e-5, rope_theta=50000.0,
                          tie_word_embeddings=False),
    "head128_small": dict(num_hidden_layers=1, hidden_size=48, num_attention_heads=2,
                          num_key_value_heads=2, head_dim=128, intermediate_size=24, vocab_size=97,
                          rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True),
}
LENGTHS = [1, 2, 63, 64, 65, 130, 200]
# Standard deviation of the random weights: wide enough that attention is far from
# uniform, not so wide that scores reach tens and bfloat16 rounding of q and k alone
# moves the softmax by several percent (which the width-264 configuration does at 0.1).
STD = {"head64_group8": 0.05}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_configurations_in_three_cuttings(tmp_path, name, dtype):
    import foundry_b200 as fb
    from foundry_b200.config import LlamaConfig
    from test_gpu_replay import run_batches, run_tail_one_by_one, run_whole
    cfg_doc = {**BASE, **ODD[name]}
    folder = fb.write_model_folder(str(tmp_path / name), LlamaConfig.parse(cfg_doc), 21,
                                   std=STD.get(name, 0.1))
    cfg, w = plain.read_model(folder)
    requests = [tiny.random_tokens(500 + i, n, cfg["vocab_size"]) for i, n in enumerate(LENGTHS)]
    expected = [plain.forward(cfg, w, r).numpy() for r in requests]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=8)
    for i, (r, e) in enumerate(zip(requests, expected)):
        tiny.assert_logits_close(run_whole(engine, r), e, dtype, f"{name} whole {i}")
        tiny.assert_logits_close(run_tail_one_by_one(engine, r), e, dtype, f"{name} tail {i}")
    for batch_size, share in ((3, 0.5), (7, 0.2)):
        got = run_batches(engine, requests, batch_size, share)
        for i, e in enumerate(expected):
            tiny.assert_logits_close(got[i], e, dtype, f"{name} batch {batch_size} request {i}")
