"""The layer sizes of the three benchmark configurations against the plain
model, two layers deep:

  3B  hidden 3072, 24 heads over 8 kv heads of 128, feed-forward 8192, tied head
  1B  hidden 2048, 32 heads over 8 kv heads of 64,  feed-forward 8192, tied head
  8B  hidden 4096, 32 heads over 8 kv heads of 128, feed-forward 14336, separate head

all with vocabulary 128256 and llama3 frequency scaling. 3B runs the unequal
batch its configuration names (3, 500 and 2048 tokens), then two single-token
steps. 1B and 8B run an unequal batch, a step in which one prompt goes on by
70 tokens while the others bring one (keys before the first query, at head
sizes 64 and 128), single-token steps of 4 sequences, then 20 more sequences
join for single-token steps of 24 (the 17 to 128 row products and the decode
attention's plan at these widths).

Two layers instead of 16 / 28 / 32: the float64 plain model runs on the CPU;
every kernel still meets its real widths, head size and vocabulary. The plain
side keeps the embedding and the head in 16 bits and widens what it uses, and
logits are compared at chosen places only.
"""
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu


def config(hidden, heads, head_dim, intermediate, factor, tied):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": 8,
        "head_dim": head_dim, "intermediate_size": intermediate, "vocab_size": 128256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "tie_word_embeddings": tied, "max_position_embeddings": 131072,
    }


CONFIGS = {
    "3b": config(3072, 24, 128, 8192, 32.0, True),
    "1b": config(2048, 32, 64, 8192, 32.0, True),
    "8b": config(4096, 32, 128, 14336, 8.0, False),
}
CONFIG = CONFIGS["3b"]
LENGTHS = (3, 500, 2048)


class WidenedOnUse(dict):
    """Tensors kept as stored and widened to float64 each time one is read."""

    def __getitem__(self, name):
        return dict.__getitem__(self, name).to(torch.float64)


class PlainWide:
    """The plain model for wide matrices: layer weights in float64 (or, with
    `widen_on_use`, as stored and widened when a layer reads them: 28 layers in
    float64 would be 22 GB), the embedding and the head as stored (rows widened
    when used)."""

    def __init__(self, folder, widen_on_use=False):
        from safetensors import safe_open
        with open(os.path.join(folder, "config.json")) as handle:
            self.cfg = json.load(handle)
        self.w, self.table = (WidenedOnUse() if widen_on_use else {}), {}
        with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as handle:
            for name in handle.keys():
                t = handle.get_tensor(name)
                if name in ("model.embed_tokens.weight", "lm_head.weight"):
                    self.table[name] = t
                elif widen_on_use:
                    dict.__setitem__(self.w, name, t)
                else:
                    self.w[name] = t.to(torch.float64)

    def logits_at(self, tokens, rows):
        """Logits at positions `rows` of one whole sequence."""
        cfg = self.cfg
        x = self.table["model.embed_tokens.weight"][torch.as_tensor(tokens)].to(torch.float64)
        positions = list(range(len(tokens)))
        for i in range(cfg["num_hidden_layers"]):
            x = plain.decoder_layer(x, self.w, i, cfg, positions)
        x = plain.rms_norm(x[rows], self.w["model.norm.weight"], cfg["rms_norm_eps"])
        head = self.table["model.embed_tokens.weight" if cfg["tie_word_embeddings"]
                          else "lm_head.weight"]
        out = [x @ head[at:at + 16384].to(torch.float64).T for at in range(0, head.shape[0], 16384)]
        return torch.cat(out, 1).numpy()


def assert_close(got, want, dtype, what):
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max())
    if dtype == "float32":
        # sums of up to 14,336 float32 products, a few products deep: a summation-order
        # bound of 1e-4 of the logit scale
        assert err <= 1e-4 * scale, f"{what}: max |diff| {err:.3e} (scale {scale:.2f})"
    else:
        close = np.abs(got - want) <= 1e-2 * scale + 1e-2 * np.maximum(np.abs(got), np.abs(want))
        assert close.mean() >= 0.999, f"{what}: {close.mean():.5f} close, max {err:.3e}"
        assert err <= 5e-2 * scale, f"{what}: max |diff| {err:.3e} (scale {scale:.2f})"


def write_folder(tmp_path_factory, name, layers=2):
    import foundry_b200 as fb
    from foundry_b200.config import LlamaConfig
    folder = str(tmp_path_factory.mktemp(f"wide_{name}") / "model")
    # N(0, 0.02) weights, norm weights 1 + N(0, 0.1); drawn on the GPU (seconds, not minutes)
    fb.write_model_folder(folder, LlamaConfig.parse({**CONFIGS[name], "num_hidden_layers": layers}),
                          2, std=0.02, device="cuda:0")
    return folder


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    folder = write_folder(tmp_path_factory, "3b")
    model = PlainWide(folder)
    rng = np.random.default_rng(11)
    seqs = [[int(t) for t in rng.integers(0, 128000, size=n + 2)] for n in LENGTHS]
    rows = [sorted({0, n // 3, n - 2, n - 1, n, n + 1} & set(range(n + 2))) for n in LENGTHS]
    want = [model.logits_at(s, r) for s, r in zip(seqs, rows)]
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
        assert_close(np.concatenate(pieces[i]), w, dtype, f"sequence {i}")
    from foundry_b200.kernels import ops
    assert ops.gemm_tc_status() == 0


@pytest.mark.slow
def test_the_benchmark_model_at_its_full_depth_in_float32(tmp_path_factory):
    """All 28 layers of the 3B configuration in 32 bits on the unequal batch's
    two short sequences (3 and 500 tokens in one step): what 28 layers make of
    the float32 kernels' rounding, against the float64 plain model. The 2,048-
    token sequence stays with the two-layer test: 28 layers of it in float64 on
    the CPU would take many minutes."""
    import foundry_b200 as fb
    from foundry_b200.engine import SequenceStep
    folder = write_folder(tmp_path_factory, "3b", layers=28)
    model = PlainWide(folder, widen_on_use=True)
    rng = np.random.default_rng(13)
    seqs = [[int(t) for t in rng.integers(0, 128000, size=n)] for n in (3, 500)]
    rows = [[0, 2], [0, 250, 499]]
    want = [model.logits_at(s, r) for s, r in zip(seqs, rows)]
    del model
    engine = fb.Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_slots=2)
    slots = [engine.open_sequence() for _ in seqs]
    got = engine.step([SequenceStep(s, q, r) for s, q, r in zip(slots, seqs, rows)]).cpu().numpy()
    at = 0
    for i, w in enumerate(want):
        g = got[at:at + len(rows[i])]
        at += len(rows[i])
        scale = max(1.0, float(np.abs(w).max()))
        err = float(np.abs(g - w).max())
        assert np.isfinite(g).all()
        # 28 layers of float32 sums against float64: within 1e-3 of the logit scale
        assert err <= 1e-3 * scale, f"sequence {i}: max |diff| {err:.3e} (scale {scale:.2f})"


# ------------------------------------------------------------------ 1B and 8B
FIRST = (3, 150, 400, 130)  # prompt tokens of the first four sequences
MORE, LATE = 70, 20  # the fourth prompt goes on by MORE tokens; LATE sequences join later
SINGLE_4, SINGLE_24 = 3, 2  # single-token steps with 4 and with 24 sequences


@pytest.fixture(scope="module", params=["1b", "8b"])
def twin(request, tmp_path_factory):
    """(name, folder, sequences, {sequence: (rows, plain logits there)})."""
    name = request.param
    folder = write_folder(tmp_path_factory, name)
    model = PlainWide(folder)
    rng = np.random.default_rng(5)
    total = [n + 1 + SINGLE_4 + SINGLE_24 for n in FIRST]
    total[3] += MORE - 1
    late = [int(n) for n in rng.integers(2, 40, size=LATE)]
    total += [n + SINGLE_24 for n in late]
    seqs = [[int(t) for t in rng.integers(0, 128000, size=n)] for n in total]
    want = {}
    for i, s in enumerate(seqs):
        if i < 4:
            first = FIRST[i]
            rows = sorted({0, first // 2, first - 1} | set(range(first, len(s))))
        else:
            rows = [late[i - 4] - 1] + list(range(late[i - 4], len(s)))
        want[i] = (rows, model.logits_at(s, rows))
    return name, folder, seqs, late, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_other_benchmark_widths(twin, dtype):
    import foundry_b200 as fb
    from foundry_b200.engine import SequenceStep
    from foundry_b200.kernels import ops
    name, folder, seqs, late, want = twin
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=4096, max_slots=24)
    got = {i: [] for i in range(len(seqs))}
    at = [0] * len(seqs)  # tokens of each sequence in the cache
    slots = [engine.open_sequence() for _ in range(4)]

    def run(entries):
        """entries: (sequence, token count, wanted places); appends the logits."""
        out = engine.step([SequenceStep(slots[i], seqs[i][at[i]:at[i] + n], w)
                           for i, n, w in entries]).cpu().numpy()
        row = 0
        for i, n, w in entries:
            got[i].append(out[row:row + len(w)])
            row += len(w)
            at[i] += n

    run([(i, FIRST[i], sorted({0, FIRST[i] // 2, FIRST[i] - 1})) for i in range(4)])
    # one prompt goes on by MORE tokens while the other three bring one token each
    run([(0, 1, [0]), (1, 1, [0]), (2, 1, [0]), (3, MORE, list(range(MORE)))])
    for _ in range(SINGLE_4):
        run([(i, 1, [0]) for i in range(4)])
    slots += [engine.open_sequence() for _ in range(LATE)]
    run([(4 + j, n, [n - 1]) for j, n in enumerate(late)])
    for _ in range(SINGLE_24):
        run([(i, 1, [0]) for i in range(len(seqs))])
    assert max(key[0] for key in engine._runners) == 32  # 24 rows ran in the 32-row bucket
    for i, (rows, logits) in want.items():
        assert_close(np.concatenate(got[i]), logits, dtype, f"{name} sequence {i}")
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
