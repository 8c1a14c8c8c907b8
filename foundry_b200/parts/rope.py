"""Rotary position encodings: the frequency vector is the part.

The rotation itself runs inside the mixer's kernel, which takes the inverse
frequencies, the rotary width and the pairing as parameters (`pairing = "half"`:
frequency i turns elements i and i + width/2, the reference's; "interleaved":
elements 2i and 2i + 1); a variant of the encoding is another frequency vector
and, if it pairs otherwise, another `pairing` attribute.

inv_freq[j] = 1 / theta^(2j / D), j = 0 .. D/2, in 32-bit
(src/models/llama/rotary_emb.rs:135-160). The "llama3" scaling
(rotary_emb.rs:162-183) leaves short wavelengths as they are, divides long
ones by `factor`, and blends between the two bands:

    wavelen = 2*pi / f;  low_wl = ctx / low_freq_factor;  high_wl = ctx / high_freq_factor
    f' = f / factor if wavelen > low_wl else f
    smooth = (ctx / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    f'' = (1 - smooth) * f' / factor + smooth * f'   if high_wl <= wavelen <= low_wl else f'
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import Part, register_position_encoding

F = np.float32


def plain_inv_freq(head_dim: int, theta: float) -> np.ndarray:
    if head_dim <= 0 or head_dim % 2:
        raise ValueError(f"rotary width {head_dim} is not a positive even number")
    exponents = np.arange(0, head_dim, 2, dtype=F) / F(head_dim)
    return (F(1.0) / np.power(F(theta), exponents, dtype=F)).astype(F)


def llama3_inv_freq(head_dim: int, theta: float, factor: float, low_freq_factor: float,
                    high_freq_factor: float, original_max_position_embeddings: int) -> np.ndarray:
    f = plain_inv_freq(head_dim, theta)
    ctx = F(original_max_position_embeddings)
    factor, low, high = F(factor), F(low_freq_factor), F(high_freq_factor)
    low_wl, high_wl = ctx / low, ctx / high
    wavelen = F(2.0 * math.pi) / f
    scaled = np.where(wavelen > low_wl, f / factor, f).astype(F)
    smooth = ((ctx / wavelen - low) / (high - low)).astype(F)
    medium = (wavelen >= high_wl) & (wavelen <= low_wl)
    blended = ((F(1.0) - smooth) * scaled / factor + smooth * scaled).astype(F)
    return np.where(medium, blended, scaled).astype(F)


class _Rotary(Part):
    attention_factor = 1.0
    pairing = "half"  # src/models/llama/rotary_emb.rs:76-85 (rotate_half)

    def _finish(self, inv_freq: np.ndarray, device: torch.device) -> None:
        self.rotary_dim = 2 * int(inv_freq.shape[0])
        self.inv_freq_host = inv_freq
        self.inv_freq = torch.from_numpy(inv_freq.copy()).to(device)


@register_position_encoding("rope")
class Rope(_Rotary):
    def __init__(self, head_dim: int, theta: float, *, dtype=None, device=None):
        self._finish(plain_inv_freq(head_dim, theta), device)


@register_position_encoding("rope_llama3")
class RopeLlama3(_Rotary):
    def __init__(self, head_dim: int, theta: float, factor: float, low_freq_factor: float,
                 high_freq_factor: float, original_max_position_embeddings: int, *,
                 dtype=None, device=None):
        self._finish(llama3_inv_freq(head_dim, theta, factor, low_freq_factor, high_freq_factor,
                                     original_max_position_embeddings), device)
