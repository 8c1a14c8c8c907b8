"""From a model folder's tensors to the tensors a model asks for, by name.

The reference fetches each tensor by its Hugging Face name and fails on the
first one that is absent, not bf16 or of another shape
(src/models/llama/weights.rs:17-55: `TensorNotFound`, `TensorDTypeMismatch`,
`TensorShapeMismatch`). Here the whole folder is checked against the whole
list first, and ONE error names everything that is missing, unexpected or
mis-shaped, so a wrong folder is diagnosed in one run.

Storage rule: floating tensors stored in 16 bits are kept in bfloat16 when the
engine runs in bfloat16; a tensor stored in 32 bits stays in 32 bits; integer
tables become int32 (range-checked); a float32 engine widens everything to
float32, which is exact for bfloat16 values.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import List, Mapping, Sequence, Tuple

import torch

from .safetensors_io import WeightFiles, WeightsError


@dataclass(frozen=True)
class ExpectedTensor:
    shape: Tuple[int, ...]
    integer: bool = False  # an integer table rather than a floating tensor


class WeightsMismatch(WeightsError):
    """The folder's tensors are not the ones the model needs."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing: List[str] = list(missing)
        self.unexpected: List[str] = list(unexpected)
        self.wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = list(wrong_shape)
        self.wrong_dtype: List[Tuple[str, str]] = list(wrong_dtype)
        lines = ["the weight files do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT_OK = ("BF16", "F32")
_INT_OK = ("I64", "I32", "I16", "I8", "U8", "U32")


def check_against(files: WeightFiles, expected: Mapping[str, ExpectedTensor],
                  ignorable: Sequence[str] = ()) -> None:
    """Raise `WeightsMismatch` unless the folder holds exactly the expected
    tensors (plus ignorable ones) with the expected shapes and a usable dtype."""
    missing, unexpected, wrong_shape, wrong_dtype = [], [], [], []
    for name, want in expected.items():
        if name not in files:
            missing.append(name)
            continue
        entry = files.entry(name)
        if tuple(entry.shape) != tuple(want.shape):
            wrong_shape.append((name, tuple(want.shape), tuple(entry.shape)))
        ok = _INT_OK if want.integer else _FLOAT_OK
        if entry.dtype not in ok:
            wrong_dtype.append((name, entry.dtype))
    for name in files.names():
        if name not in expected and not any(fnmatch.fnmatchcase(name, p) for p in ignorable):
            unexpected.append(name)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsMismatch(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)


def stored_to_run_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor has on the device (see the module docstring)."""
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_tensor(files: WeightFiles, name: str, run_dtype: torch.dtype,
                device: torch.device) -> torch.Tensor:
    host = files.tensor(name)
    target = stored_to_run_dtype(host.dtype, run_dtype)
    if target == torch.int32 and host.dtype != torch.int32:
        if host.numel() and (int(host.max()) > 2**31 - 1 or int(host.min()) < -2**31):
            raise WeightsError(f"integer table {name!r} does not fit in int32")
    return host.to(device=device, dtype=target)
