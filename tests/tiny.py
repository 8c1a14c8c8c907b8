"""The tiny configurations the tests run, and helpers shared by test files.

Tiny A and Tiny B differ in every size and option: layer count, width, head
count and grouping, head size, feed-forward width (176 is no power of two),
vocabulary, eps, theta, frequency scaling, tied or separate output head.
Tiny B's 16 frequencies fall into all three bands of the llama3 scaling.
"""
import numpy as np
import torch

CONFIGS = {
    "tiny_a": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
        "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256,
        "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
        "tie_word_embeddings": True, "max_position_embeddings": 128, "eos_token_id": 7,
    },
    "tiny_b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6,
        "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 256, "vocab_size": 384,
        "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
        "tie_word_embeddings": False, "max_position_embeddings": 256, "eos_token_id": [3, 5],
    },
}
SEEDS = {"tiny_a": 0, "tiny_b": 1}
# Wider weights than N(0, 0.02) make attention and logits far from uniform, so
# that a wrong key, position or row shows in the logits instead of averaging out.
STD = 0.08


def write_folder(folder: str, name: str, std: float = STD, dtype=torch.bfloat16) -> str:
    from foundry_b200.config import LlamaConfig
    from foundry_b200.weights import write_model_folder
    return write_model_folder(folder, LlamaConfig.parse(CONFIGS[name]), SEEDS[name], std=std,
                              dtype=dtype)


def random_tokens(seed: int, length: int, vocab: int):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=length)]


def close_fraction(actual: np.ndarray, expected: np.ndarray, atol: float, rtol: float) -> float:
    """Share of elements with |a - e| <= atol + rtol * max(|a|, |e|): the
    reference's element rule (src/eval/compare.rs:26-35)."""
    bound = atol + rtol * np.maximum(np.abs(actual), np.abs(expected))
    return float(np.mean(np.abs(actual - expected) <= bound))


def assert_logits_close(actual, expected, dtype: str, what: str = ""):
    """float32: every element within a summation-order bound of the float64
    plain model. bfloat16: the reference's element rule for 16-bit engines
    (src/eval/compare.rs:8-9, 51-91: rtol 1e-2, >= 99.9 % of elements close,
    nothing non-finite). Its atol of 1e-2 (src/models/llama/model.rs:362-368) is
    for activations of order one; logits here reach several units because the
    test weights are wide, so atol is 1e-2 times the logit scale. A wrong key,
    position or cache row moves logits by tens of percent of that scale."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    assert np.isfinite(actual).all(), f"{what}: non-finite logits"
    if not actual.size:
        return
    err = np.abs(actual - expected).max()
    scale = max(1.0, float(np.abs(expected).max()))
    if dtype == "float32":
        assert err <= 2e-5 * scale, f"{what}: max |diff| {err:.3e} (scale {scale:.2f})"
    else:
        frac = close_fraction(actual, expected, atol=1e-2 * scale, rtol=1e-2)
        assert frac >= 0.999, f"{what}: only {frac:.5f} of elements close, max |diff| {err:.3e}"
        assert err <= 5e-2 * scale, f"{what}: max |diff| {err:.3e} (scale {scale:.2f})"
