"""Reading and writing safetensors files, by tensor name.

The container is the one the reference reads (src/weights/mod.rs:76-99,
281-336): an 8-byte little-endian header length, a JSON header that maps each
tensor name to `{dtype, shape, data_offsets}` (the `__metadata__` entry is not
a tensor), then the raw little-endian data. A folder holds either
`model.safetensors` or `model.safetensors.index.json` with a `weight_map` from
tensor name to shard file (src/weights/mod.rs:215-258). The file-level checks
carry the reference's names (src/weights/error.rs:1-41).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import torch

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"
MAX_INDEX_BYTES = 100 * 1024 * 1024  # src/weights/mod.rs:35
MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
    "U32": (torch.int32, 4),  # read as bits; the loader range-checks integer tables
}
_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
          torch.float64: "F64", torch.int64: "I64", torch.int32: "I32", torch.int16: "I16",
          torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}


class WeightsError(ValueError):
    """A weight file or folder is malformed."""


class IndexRead(WeightsError): pass
class IndexTooLarge(WeightsError): pass
class IndexJson(WeightsError): pass
class ShardOpen(WeightsError): pass
class InvalidShardName(WeightsError): pass
class InvalidHeader(WeightsError): pass
class UnknownDType(WeightsError): pass
class InvalidShape(WeightsError): pass
class DuplicateTensor(WeightsError): pass
class IndexMismatch(WeightsError): pass
class ByteCountMismatch(WeightsError): pass
class TensorNotFound(WeightsError, KeyError): pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str  # safetensors dtype string
    shape: Tuple[int, ...]
    shard: str  # path of the file that holds it
    begin: int  # absolute byte offsets in that file
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.begin

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


def parse_header(path: str) -> Tuple[Dict[str, TensorEntry], Dict[str, str]]:
    """Read one file's header and validate every entry against the file size."""
    try:
        size = os.stat(path).st_size
        with open(path, "rb") as handle:
            prefix = handle.read(8)
            if len(prefix) != 8:
                raise InvalidHeader(f"{path}: shorter than the 8-byte header length")
            (header_len,) = struct.unpack("<Q", prefix)
            if header_len > MAX_HEADER_BYTES or 8 + header_len > size:
                raise InvalidHeader(f"{path}: header length {header_len} exceeds the file")
            raw = handle.read(header_len)
    except OSError as exc:
        raise ShardOpen(f"cannot open {path}: {exc}") from exc
    try:
        header = json.loads(raw)
    except ValueError as exc:
        raise InvalidHeader(f"{path}: header is not JSON: {exc}") from exc
    if not isinstance(header, dict):
        raise InvalidHeader(f"{path}: header is not a JSON object")
    metadata = header.pop("__metadata__", None) or {}
    data_start = 8 + header_len
    entries: Dict[str, TensorEntry] = {}
    for name, info in header.items():
        try:
            dtype, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError) as exc:
            raise InvalidHeader(f"{path}: entry {name!r} is malformed") from exc
        if dtype not in _DTYPES:
            raise UnknownDType(f"{path}: tensor {name!r} has dtype {dtype!r}")
        if any((not isinstance(d, int)) or d < 0 for d in shape):
            raise InvalidShape(f"{path}: tensor {name!r} has shape {list(shape)}")
        numel = 1
        for d in shape:
            numel *= d
        if not (isinstance(begin, int) and isinstance(end, int) and 0 <= begin <= end):
            raise InvalidHeader(f"{path}: tensor {name!r} has offsets {info['data_offsets']}")
        if end - begin != numel * _DTYPES[dtype][1]:
            raise ByteCountMismatch(
                f"{path}: tensor {name!r} of shape {list(shape)} and dtype {dtype} spans "
                f"{end - begin} bytes")
        if data_start + end > size:
            raise InvalidHeader(f"{path}: tensor {name!r} ends beyond the file")
        entries[name] = TensorEntry(name, dtype, shape, path, data_start + begin, data_start + end)
    return entries, metadata


class WeightFiles:
    """The tensors of a model folder, looked up by name
    (src/weights/mod.rs:112-118)."""

    def __init__(self, entries: Dict[str, TensorEntry]):
        self._entries = entries

    @classmethod
    def open(cls, directory: str) -> "WeightFiles":
        index_path = os.path.join(directory, INDEX_FILE)
        if os.path.exists(index_path):
            return cls._open_sharded(directory, index_path)
        entries, _ = parse_header(os.path.join(directory, SINGLE_FILE))
        return cls(entries)

    @classmethod
    def _open_sharded(cls, directory: str, index_path: str) -> "WeightFiles":
        try:
            if os.stat(index_path).st_size > MAX_INDEX_BYTES:
                raise IndexTooLarge(f"{index_path} exceeds {MAX_INDEX_BYTES} bytes")
            with open(index_path, "rb") as handle:
                raw = handle.read()
        except OSError as exc:
            raise IndexRead(f"cannot read {index_path}: {exc}") from exc
        try:
            index = json.loads(raw)
            weight_map = index["weight_map"]
            if not isinstance(weight_map, dict):
                raise TypeError("weight_map is not an object")
        except (ValueError, KeyError, TypeError) as exc:
            raise IndexJson(f"{index_path}: {exc}") from exc
        entries: Dict[str, TensorEntry] = {}
        for shard in sorted(set(weight_map.values())):
            # a shard is named by a plain file name (src/weights/mod.rs:251-258)
            if not isinstance(shard, str) or not shard or os.path.basename(shard) != shard \
                    or shard in (".", ".."):
                raise InvalidShardName(f"{index_path}: shard name {shard!r}")
            shard_entries, _ = parse_header(os.path.join(directory, shard))
            for name, entry in shard_entries.items():
                if name in entries:
                    raise DuplicateTensor(f"tensor {name!r} is in {entries[name].shard} and {shard}")
                entries[name] = entry
        for name, shard in weight_map.items():
            held = entries.get(name)
            if held is None or os.path.basename(held.shard) != shard:
                raise IndexMismatch(f"{index_path}: {name!r} is not in shard {shard!r}")
        total = (index.get("metadata") or {}).get("total_size")
        if total is not None and total != sum(e.nbytes for e in entries.values()):
            raise ByteCountMismatch(
                f"{index_path}: total_size {total} differs from the tensors' "
                f"{sum(e.nbytes for e in entries.values())} bytes")
        return cls(entries)

    def names(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def entry(self, name: str) -> TensorEntry:
        try:
            return self._entries[name]
        except KeyError:
            raise TensorNotFound(f"no tensor named {name!r}") from None

    def nbytes(self) -> int:
        return sum(e.nbytes for e in self._entries.values())

    def numel(self) -> int:
        return sum(e.numel for e in self._entries.values())

    def tensor(self, name: str, *, pin: bool = False) -> torch.Tensor:
        """A host copy of the tensor, in the dtype the file stores."""
        entry = self.entry(name)
        raw = torch.empty(entry.nbytes, dtype=torch.uint8, pin_memory=pin)
        if entry.nbytes:
            with open(entry.shard, "rb") as handle:
                handle.seek(entry.begin)
                got = handle.readinto(memoryview(raw.numpy()).cast("B"))
            if got != entry.nbytes:
                raise InvalidHeader(f"{entry.shard}: short read of tensor {name!r}")
        return raw.view(entry.torch_dtype).reshape(entry.shape)


def save_file(tensors: Mapping[str, torch.Tensor], path: str,
              metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write one safetensors file; tensors are laid out in name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise UnknownDType(f"tensor {name!r} has dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as handle:
        handle.write(struct.pack("<Q", len(raw)))
        handle.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                handle.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
