"""A plain, slow Llama: whole sequences, no cache, no batching, float64.

This file rests on the reference's formulas, not on its code run here: the
reference (stratorys/foundry) is Rust with a Metal-only device backend
(src/lib.rs:4-5, src/cli/mod.rs:193-197), there is no Rust toolchain on this
machine, and it has no CPU device to run its model on; so its model code can
be neither compiled nor executed here. Each function restates one part from
the cited lines. It shares no code with `foundry_b200`: it reads config.json
with `json`, the weights with the `safetensors` package, and computes with
torch on the CPU.

Storage rounding is not imitated: weights are widened to float64 as stored and
nothing is rounded afterwards. The one deliberate 32-bit step is the rotary
angle, which the reference forms as a 32-bit product of a 32-bit position and a
32-bit frequency (rotary_emb.rs:113-133); its rounding is part of the model.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
from safetensors import safe_open

F64 = torch.float64


# ------------------------------------------------------------------ loading
def read_model(folder: str):
    """(config dict, {tensor name: float64 tensor})."""
    with open(os.path.join(folder, "config.json")) as handle:
        cfg = json.load(handle)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(F64)
    return cfg, weights


def head_dim_of(cfg) -> int:
    # src/models/llama/config.rs:141-143: head_dim, else hidden_size / heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# --------------------------------------------------------- position encoding
def inv_freq(cfg) -> np.ndarray:
    """src/models/llama/rotary_emb.rs:135-183, every operation in 32-bit."""
    f32 = np.float32
    d = head_dim_of(cfg)
    theta = f32(cfg.get("rope_theta", 10000.0))
    out = []
    scaling = cfg.get("rope_scaling")
    for dim_index in range(0, d, 2):
        f = f32(1.0) / np.power(theta, f32(dim_index) / f32(d), dtype=f32)  # :150-153
        if scaling:
            ctx = f32(scaling["original_max_position_embeddings"])  # :166-167
            factor = f32(scaling["factor"])
            low, high = f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"])
            wavelen_low, wavelen_high = ctx / low, ctx / high  # :168-169
            wavelen = f32(2.0 * math.pi) / f  # :170
            scaled = f / factor if wavelen > wavelen_low else f  # :171-175
            smooth = (ctx / wavelen - low) / (high - low)  # :176-177
            if wavelen_high <= wavelen <= wavelen_low:  # :178-182
                f = (f32(1.0) - smooth) * scaled / factor + smooth * scaled
            else:
                f = scaled
        out.append(f32(f))
    return np.asarray(out, dtype=f32)


def rotary_tables(cfg, positions: Sequence[int]):
    """cos, sin of shape [S, D]: the D/2 frequencies repeated twice
    (rotary_emb.rs:113-133); angle = f32(position) * f32(inv_freq) in 32-bit."""
    f = inv_freq(cfg)
    pos = np.asarray(positions, dtype=np.float32)[:, None]
    angle = (pos * f[None, :]).astype(np.float32)  # one 32-bit rounding
    angle = np.concatenate([angle, angle], axis=1).astype(np.float64)
    return torch.from_numpy(np.cos(angle)), torch.from_numpy(np.sin(angle))


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[..., D/2:], x[..., :D/2]) (rotary_emb.rs:76-85)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x * cos + rotate_half(x) * sin, x: [S, heads, D] (rotary_emb.rs:62-74)."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


# ---------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w (src/nn/norm.rs:31-51)."""
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) * (1.0 / x.shape[-1]) + eps)
    return x * scale * weight


# ----------------------------------------------------------------- attention
def attention(x, w, prefix, cfg, positions, window: Optional[int] = None):
    """src/models/llama/attention.rs:72-131 with src/nn/attention.rs:23-60."""
    S = x.shape[0]
    A, K, D = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    q = (x @ w[f"{prefix}.q_proj.weight"].T).reshape(S, A, D)  # attention.rs:88-95
    k = (x @ w[f"{prefix}.k_proj.weight"].T).reshape(S, K, D)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).reshape(S, K, D)
    cos, sin = rotary_tables(cfg, positions)
    q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)  # attention.rs:104-105
    scale = 1.0 / math.sqrt(D)  # attention.rs:56-58
    group = A // K
    out = torch.empty(S, A, D, dtype=F64)
    pos = torch.as_tensor(list(positions))
    visible = pos[None, :] <= pos[:, None]  # key <= query (src/nn/masking.rs:76-92)
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    for a in range(A):
        kv = a // group  # src/nn/attention.rs:40-44
        scores = (q[:, a, :] @ k[:, kv, :].T) * scale  # nn/attention.rs:45-55
        scores = scores.masked_fill(~visible, float("-inf"))
        scores = scores - scores.max(-1, keepdim=True).values  # src/nn/activation.rs:35-39
        p = torch.exp(scores)
        p = p / p.sum(-1, keepdim=True)
        out[:, a, :] = p @ v[:, kv, :]  # nn/attention.rs:56-59
    return out.reshape(S, A * D) @ w[f"{prefix}.o_proj.weight"].T  # attention.rs:121-131


# ---------------------------------------------------------------- feed-forward
def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (src/nn/activation.rs:18-27)."""
    return x / (1.0 + torch.exp(-x))


def mlp(x, w, prefix):
    """down(silu(gate(x)) * up(x)) (src/models/llama/mlp.rs:49-58)."""
    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return (silu(gate) * up) @ w[f"{prefix}.down_proj.weight"].T


# --------------------------------------------------------------------- model
def decoder_layer(x, w, i, cfg, positions):
    """src/models/llama/model.rs:254-278."""
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    h = x + attention(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn",
                      cfg, positions)
    return h + mlp(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")


def forward(cfg, w, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [S, vocab] of one whole sequence starting at position 0
    (src/models/llama/model.rs:168-193, 102-122)."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]  # src/nn/linear.rs:54-69
    positions = list(range(len(tokens)))  # src/nn/masking.rs:11-23 with past = 0
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]  # model.rs:62 (tied); a separate head otherwise
    return x @ head.T


# ---------------------------------------------------------------- generation
def argmax_first(row: torch.Tensor) -> int:
    """Largest value, lowest index among equals
    (src/metal/kernels/reduce.metal:42-78)."""
    best = row.max()
    return int(torch.nonzero(row == best)[0, 0])


def greedy_generate(cfg, w, prompt: Sequence[int], max_new_tokens: int,
                    eos: Sequence[int] = ()) -> List[int]:
    """Greedy decoding by running the whole sequence again for every token
    (the loop of src/generate/mod.rs:45-90 without its cache)."""
    seq = list(prompt)
    new: List[int] = []
    for _ in range(max_new_tokens):
        token = argmax_first(forward(cfg, w, seq)[-1])
        new.append(token)
        seq.append(token)
        if token in eos:
            break
    return new


# ------------------------------------------------------------------ sampling
_GOLDEN = 0x9E3779B97F4A7C15
_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    """SplitMix64's output function (constants as in src/bench/rng.rs:3-5, 21-27)."""
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def sample_uniform(seed: int, key: int, step: int, token: int) -> float:
    """The uniform in (0, 1) that temperature sampling draws for one token id;
    written with Python integers, independently of the library's host code."""
    z = _mix((seed + _GOLDEN * (key + 1)) & _MASK)
    z = _mix((z + _GOLDEN * (step + 1)) & _MASK)
    z = _mix((z + _GOLDEN * (token + 1)) & _MASK)
    return ((z >> 40) + 0.5) / 16777216.0


def sample_scores(logits: torch.Tensor, temperature: float, seed: int, key: int,
                  step: int) -> torch.Tensor:
    """logit / T + Gumbel noise, float64; its argmax is the sampled token."""
    u = torch.tensor([sample_uniform(seed, key, step, i) for i in range(logits.shape[-1])],
                     dtype=F64)
    return logits.to(F64) / temperature - torch.log(-torch.log(u))
