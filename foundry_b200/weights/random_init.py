"""Random-weights mode: a model folder from a configuration and a seed.

The reference only ever loads published checkpoints; it has no random mode.
This one writes what the loader reads: `config.json` and `model.safetensors`
with the architecture's own tensor names, so tests and benchmarks run the same
load path as a real folder.

Each tensor has its own stream, keyed by (seed, tensor name): adding a tensor
or changing the order leaves the others as they were.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Mapping, Optional

import torch

from ..config.files import CONFIG_FILE
from .safetensors_io import SINGLE_FILE, save_file


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & (2**63 - 1)


def random_tensors(expected: Mapping[str, "ExpectedTensor"], seed: int, *,
                   dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                   norm_std: float = 0.1, device: str = "cpu",
                   is_norm: Optional[Callable[[str], bool]] = None) -> Dict[str, torch.Tensor]:
    """Matrices ~ N(0, std); vectors (norm weights) ~ 1 + N(0, norm_std)."""
    out: Dict[str, torch.Tensor] = {}
    for name, want in expected.items():
        gen = torch.Generator(device=device)
        gen.manual_seed(tensor_seed(seed, name))
        norm = is_norm(name) if is_norm is not None else len(want.shape) == 1
        if want.integer:
            out[name] = torch.zeros(want.shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(want.shape, generator=gen, dtype=torch.float32, device=device)
        t = 1.0 + norm_std * t if norm else std * t
        out[name] = t.to(dtype)
    return out


def write_model_folder(directory: str, config, seed: int, *,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                       norm_std: float = 0.1, device: str = "cpu") -> str:
    """Write `config.json` and `model.safetensors` for `config`
    (a typed configuration of a registered architecture) and return the folder.
    `device`: where the numbers are drawn (a CUDA device draws billions of them
    in seconds; its stream differs from the CPU's for the same seed)."""
    from ..config.registry import resolve_architecture
    from ..engine.model import expected_tensors
    import foundry_b200.models  # noqa: F401

    doc = config.to_json()
    arch = resolve_architecture(doc)
    spec = arch.build_spec(config)
    os.makedirs(directory, exist_ok=True)
    tensors = {}
    for name, want in expected_tensors(spec).items():  # one at a time: the draw is freed at once
        drawn = random_tensors({name: want}, seed, dtype=dtype, std=std, norm_std=norm_std,
                               device=device)
        tensors[name] = drawn[name].cpu()
    save_file(tensors, os.path.join(directory, SINGLE_FILE), metadata={"format": "pt"})
    with open(os.path.join(directory, CONFIG_FILE), "w") as handle:
        json.dump(doc, handle, indent=2)
        handle.write("\n")
    return directory
