"""The benchmark configuration's layer sizes (hidden 3072, 24 heads over 8 kv
heads of size 128, feed-forward 8192, vocabulary 128256, llama3 scaling with
factor 32) against the plain model, on the unequal batch the benchmark
configuration names (lengths 3, 500 and 2048), then two single-token steps.

Two layers instead of 28: the float64 plain model runs on the CPU and a full
depth would take many minutes; every kernel still meets its real widths, head
size and vocabulary. Logits are compared at a spread of positions of each
sequence (the output head over all 2,551 rows would dominate the CPU time).
"""
import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
    "hidden_size": 3072, "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 8192, "vocab_size": 128256, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LENGTHS = (3, 500, 2048)


def plain_logits_at(cfg, w, tokens, rows):
    """The plain model's logits at chosen positions of one whole sequence."""
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    positions = list(range(len(tokens)))
    for i in range(cfg["num_hidden_layers"]):
        x = plain.decoder_layer(x, w, i, cfg, positions)
    x = plain.rms_norm(x[rows], w["model.norm.weight"], cfg["rms_norm_eps"])
    return (x @ w["model.embed_tokens.weight"].T).numpy()


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    import foundry_b200 as fb
    from foundry_b200.config import LlamaConfig
    folder = str(tmp_path_factory.mktemp("wide") / "model")
    # N(0, 0.02) weights, norm weights 1 + N(0, 0.1)
    fb.write_model_folder(folder, LlamaConfig.parse(CONFIG), 2, std=0.02)
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(11)
    seqs = [[int(t) for t in rng.integers(0, 128000, size=n + 2)] for n in LENGTHS]
    rows = [sorted({0, n // 3, n - 2, n - 1, n, n + 1} & set(range(n + 2))) for n in LENGTHS]
    want = [plain_logits_at(cfg, w, s, r) for s, r in zip(seqs, rows)]
    return folder, seqs, rows, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_widths_on_an_unequal_batch(wide, dtype):
    import foundry_b200 as fb
    from foundry_b200.engine import SequenceStep
    folder, seqs, rows, want = wide
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=4096, max_slots=4)
    slots = [engine.open_sequence() for _ in seqs]
    # prompts of 3, 500 and 2048 tokens in one step, logits at the chosen places
    steps = [SequenceStep(s, q[:n], [r for r in rw if r < n])
             for s, q, n, rw in zip(slots, seqs, LENGTHS, rows)]
    got = engine.step(steps).cpu().numpy()
    at = 0
    pieces = [[] for _ in seqs]
    for i, (n, rw) in enumerate(zip(LENGTHS, rows)):
        k = len([r for r in rw if r < n])
        pieces[i].append(got[at:at + k])
        at += k
    # then two single-token steps of all three sequences
    for extra in range(2):
        out = engine.step([SequenceStep(s, [q[n + extra]], [0])
                           for s, q, n in zip(slots, seqs, LENGTHS)]).cpu().numpy()
        for i in range(len(seqs)):
            pieces[i].append(out[i:i + 1])
    for i, w in enumerate(want):
        g = np.concatenate(pieces[i])
        assert g.shape == w.shape
        assert np.isfinite(g).all()
        scale = max(1.0, float(np.abs(w).max()))
        err = float(np.abs(g - w).max())
        if dtype == "float32":
            # sums of up to 8,192 float32 products, a few products deep: a summation-order
            # bound of 1e-4 of the logit scale
            assert err <= 1e-4 * scale, f"sequence {i}: max |diff| {err:.3e} (scale {scale:.2f})"
        else:
            close = np.abs(g - w) <= 1e-2 * scale + 1e-2 * np.maximum(np.abs(g), np.abs(w))
            assert close.mean() >= 0.999, f"sequence {i}: {close.mean():.5f} close, max {err:.3e}"
            assert err <= 5e-2 * scale, f"sequence {i}: max |diff| {err:.3e} (scale {scale:.2f})"
    from foundry_b200.kernels import ops
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("streams", [3, 12])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_equal_plainly_launched_steps(wide, dtype, streams):
    """Single-token steps replayed as a graph run their kernels back to back, so
    that dependent launches really overlap; launched one by one they do not.
    Both must give the same logits, bit for bit, step after step. Three streams
    take the products' 8-token form, twelve the 16-token form."""
    import foundry_b200 as fb
    from foundry_b200.engine import SequenceStep
    folder, seqs, _, _ = wide
    # streams of at least 48 tokens
    seqs = [seqs[1], seqs[2], seqs[2][100:]] + [seqs[2][150 * i:] for i in range(1, streams - 2)]
    results = []
    for graphs in (True, False):
        engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=4096, max_slots=streams + 1)
        engine.use_graphs = graphs
        slots = [engine.open_sequence() for _ in seqs]
        engine.step([SequenceStep(s, q[:40], []) for s, q in zip(slots, seqs)])
        rows = []
        for i in range(8):
            rows.append(engine.step([SequenceStep(s, [q[40 + i]], [0])
                                     for s, q in zip(slots, seqs)]).clone())
        results.append(torch.stack(rows))
    assert torch.equal(results[0], results[1])
