"""Named configurations for measurements with random weights: the config.json
documents of the model sizes the benchmarks quote, so that `foundry bench
--config NAME --random-weights SEED` needs no model folder. These are data for
the command line and for bench.py; no part or kernel reads them."""
from __future__ import annotations

from typing import Dict


def _llama(layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, factor, tied,
           theta=500000.0, eps=1e-5, original=8192, max_positions=131072) -> Dict:
    scaling = None if factor is None else {
        "rope_type": "llama3", "factor": float(factor), "low_freq_factor": 1.0,
        "high_freq_factor": 4.0, "original_max_position_embeddings": original}
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "num_hidden_layers": layers, "hidden_size": hidden, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "head_dim": head_dim,
            "intermediate_size": intermediate, "vocab_size": vocab, "rms_norm_eps": eps,
            "rope_theta": theta, "rope_scaling": scaling, "tie_word_embeddings": tied,
            "max_position_embeddings": max_positions}


PRESETS: Dict[str, Dict] = {
    "llama-3.2-1b": _llama(16, 2048, 32, 8, 64, 8192, 128256, 32.0, True),
    "llama-3.2-3b": _llama(28, 3072, 24, 8, 128, 8192, 128256, 32.0, True),
    "llama-3.1-8b": _llama(32, 4096, 32, 8, 128, 14336, 128256, 8.0, False),
    "tiny-a": _llama(2, 64, 4, 2, 16, 176, 256, None, True, theta=10000.0, max_positions=128),
    "tiny-b": _llama(3, 96, 6, 3, 32, 256, 384, 8.0, False, eps=1e-6, original=64,
                     max_positions=256),
}


def preset(name: str) -> Dict:
    try:
        return dict(PRESETS[name])
    except KeyError:
        raise ValueError(f"no configuration named {name!r}; known: {sorted(PRESETS)}") from None
