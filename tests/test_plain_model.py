"""The plain implementation checked against itself, on the CPU.

Nothing of the reference can be run on this machine (Rust, Metal only), so the
plain model rests on the reference's formulas. Two checks guard its own code:

* a second statement of one decoder layer, written again from the cited lines
  with scalar loops in numpy (no matrix products, no broadcasting tricks, no
  code shared with `plain_llama`), must give the same numbers;
* the plain model run token by token over explicit lists of keys and values
  (what a cache does) must give the logits of its whole-sequence run.
"""
import math

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("plain")
    return {name: plain.read_model(tiny.write_folder(str(root / name), name)) for name in tiny.CONFIGS}


def loop_layer(x, w, i, cfg, positions):
    """One decoder layer with scalar loops (src/models/llama/model.rs:254-278)."""
    S, H = x.shape
    A, K = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or H // A
    eps = cfg["rms_norm_eps"]
    p = f"model.layers.{i}"

    def get(name):
        return w[name].numpy()

    def norm(rows, weight):  # src/nn/norm.rs:31-51
        out = np.zeros_like(rows)
        for s in range(rows.shape[0]):
            total = 0.0
            for h in range(H):
                total += rows[s, h] * rows[s, h]
            r = 1.0 / math.sqrt(total * (1.0 / H) + eps)
            for h in range(H):
                out[s, h] = rows[s, h] * r * weight[h]
        return out

    def project(rows, weight):  # y = x W^T, src/nn/linear.rs:19-36
        out = np.zeros((rows.shape[0], weight.shape[0]))
        for s in range(rows.shape[0]):
            for o in range(weight.shape[0]):
                out[s, o] = float(np.dot(weight[o], rows[s]))  # one output element at a time
        return out

    # frequencies, src/models/llama/rotary_emb.rs:135-183, in 32-bit
    f32 = np.float32
    scaling = cfg.get("rope_scaling")
    freqs = []
    for j in range(D // 2):
        f = f32(1.0) / f32(np.power(f32(cfg["rope_theta"]), f32(2 * j) / f32(D), dtype=f32))
        if scaling:
            ctx = f32(scaling["original_max_position_embeddings"])
            wavelen = f32(2.0 * math.pi) / f
            low_wl = ctx / f32(scaling["low_freq_factor"])
            high_wl = ctx / f32(scaling["high_freq_factor"])
            g = f / f32(scaling["factor"]) if wavelen > low_wl else f
            if high_wl <= wavelen <= low_wl:
                smooth = (ctx / wavelen - f32(scaling["low_freq_factor"])) / \
                    (f32(scaling["high_freq_factor"]) - f32(scaling["low_freq_factor"]))
                g = (f32(1.0) - smooth) * g / f32(scaling["factor"]) + smooth * g
            f = f32(g)
        freqs.append(f32(f))

    def rotate(heads, s):  # element j pairs with j + D/2, rotary_emb.rs:62-85
        out = np.zeros_like(heads)
        for h in range(heads.shape[0]):
            for j in range(D // 2):
                angle = float(f32(positions[s]) * freqs[j])  # a 32-bit product
                c, sn = math.cos(angle), math.sin(angle)
                a, b = heads[h, j], heads[h, j + D // 2]
                out[h, j] = a * c - b * sn
                out[h, j + D // 2] = b * c + a * sn
        return out

    n1 = norm(x, get(f"{p}.input_layernorm.weight"))
    q = project(n1, get(f"{p}.self_attn.q_proj.weight")).reshape(S, A, D)
    k = project(n1, get(f"{p}.self_attn.k_proj.weight")).reshape(S, K, D)
    v = project(n1, get(f"{p}.self_attn.v_proj.weight")).reshape(S, K, D)
    for s in range(S):
        q[s], k[s] = rotate(q[s], s), rotate(k[s], s)
    attn = np.zeros((S, A, D))
    for s in range(S):
        for a in range(A):
            kv = a // (A // K)  # src/nn/attention.rs:40-44
            scores = []
            for j in range(S):
                if positions[j] <= positions[s]:  # src/nn/masking.rs:76-92
                    scores.append((j, float(np.dot(q[s, a], k[j, kv])) * (1.0 / math.sqrt(D))))
            top = max(sc for _, sc in scores)
            weights = [(j, math.exp(sc - top)) for j, sc in scores]  # src/nn/activation.rs:30-40
            total = sum(e for _, e in weights)
            for j, e in weights:
                attn[s, a] += (e / total) * v[j, kv]
    h = x + project(attn.reshape(S, A * D), get(f"{p}.self_attn.o_proj.weight"))
    n2 = norm(h, get(f"{p}.post_attention_layernorm.weight"))
    gate = project(n2, get(f"{p}.mlp.gate_proj.weight"))
    up = project(n2, get(f"{p}.mlp.up_proj.weight"))
    act = np.zeros_like(gate)
    for s in range(S):
        for c in range(gate.shape[1]):
            act[s, c] = gate[s, c] / (1.0 + math.exp(-gate[s, c])) * up[s, c]  # activation.rs:18-27
    return h + project(act, get(f"{p}.mlp.down_proj.weight"))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_a_second_statement_of_a_decoder_layer_agrees(models, name):
    cfg, w = models[name]
    rng = np.random.default_rng(3)
    S = 9
    x = torch.from_numpy(rng.normal(size=(S, cfg["hidden_size"])))
    positions = list(range(4, 4 + S))  # not starting at 0: the angles matter
    for layer in range(cfg["num_hidden_layers"]):
        want = plain.decoder_layer(x, w, layer, cfg, positions).numpy()
        got = loop_layer(x.numpy(), w, layer, cfg, positions)
        assert np.abs(got - want).max() <= 1e-11 * max(1.0, np.abs(want).max())


def forward_token_by_token(cfg, w, tokens):
    """The plain model with explicit key and value lists per layer: one token a
    step, queries of the new token only, everything else from the lists."""
    A, K = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = plain.head_dim_of(cfg)
    eps = cfg["rms_norm_eps"]
    keys = [[] for _ in range(cfg["num_hidden_layers"])]
    values = [[] for _ in range(cfg["num_hidden_layers"])]
    rows = []
    for pos, token in enumerate(tokens):
        x = w["model.embed_tokens.weight"][token][None, :]
        cos, sin = plain.rotary_tables(cfg, [pos])
        for i in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{i}"
            n = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)
            q = plain.apply_rotary((n @ w[f"{p}.self_attn.q_proj.weight"].T).reshape(1, A, D), cos, sin)
            k = plain.apply_rotary((n @ w[f"{p}.self_attn.k_proj.weight"].T).reshape(1, K, D), cos, sin)
            keys[i].append(k[0])
            values[i].append((n @ w[f"{p}.self_attn.v_proj.weight"].T).reshape(K, D))
            ks, vs = torch.stack(keys[i]), torch.stack(values[i])  # [pos + 1, K, D]
            out = torch.empty(A, D, dtype=torch.float64)
            for a in range(A):
                scores = (ks[:, a // (A // K)] @ q[0, a]) / math.sqrt(D)
                out[a] = torch.softmax(scores, 0) @ vs[:, a // (A // K)]
            h = x + out.reshape(1, A * D) @ w[f"{p}.self_attn.o_proj.weight"].T
            x = h + plain.mlp(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w,
                              f"{p}.mlp")
        x = plain.rms_norm(x, w["model.norm.weight"], eps)
        head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
        rows.append(x @ head.T)
    return torch.cat(rows)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_the_plain_model_token_by_token_equals_its_whole_run(models, name):
    cfg, w = models[name]
    tokens = tiny.random_tokens(12, 70, cfg["vocab_size"])  # over a page boundary of the engine
    whole = plain.forward(cfg, w, tokens)
    stepped = forward_token_by_token(cfg, w, tokens)
    assert float((whole - stepped).abs().max()) <= 1e-10 * max(1.0, float(whole.abs().max()))


def test_greedy_generation_and_sampling_helpers(models):
    cfg, w = models["tiny_a"]
    prompt = [5, 17, 3]
    out = plain.greedy_generate(cfg, w, prompt, 4)
    seq = list(prompt)
    for t in out:  # each token is the first index of the largest logit of the run so far
        row = plain.forward(cfg, w, seq)[-1]
        assert t == int(torch.argmax(row)) and row[t] == row.max()
        seq.append(t)
    assert plain.argmax_first(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    stop = out[1]
    assert plain.greedy_generate(cfg, w, prompt, 4, eos=[stop]) == out[:out.index(stop) + 1]
    u = [plain.sample_uniform(1, 2, 3, t) for t in range(1000)]
    assert 0.0 < min(u) and max(u) < 1.0 and 0.45 < sum(u) / len(u) < 0.55
    assert plain.sample_uniform(1, 2, 3, 4) != plain.sample_uniform(1, 2, 4, 4)
