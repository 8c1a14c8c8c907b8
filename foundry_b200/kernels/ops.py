"""Python faces of the CUDA launchers: torch tensors in, checked, pointers out.

Each function checks device, dtype, contiguity and the sizes the kernel
assumes, then calls the `extern "C"` launcher on the current CUDA stream.
Nothing here computes: a tensor that is not on a CUDA device is an error, not
a reason to compute elsewhere.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import os as _os

import torch

from . import library

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; equals FB_PAGE in csrc/common.cuh

_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_ll, c_float, c_ull = (ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                                         ctypes.c_float, ctypes.c_ulonglong)

_SIGNATURES = {
    "fb_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "fb_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_float, c_void_p, c_int,
                       c_int, c_int, c_void_p],
    "fb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "fb_gather_rows": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "fb_cast": [c_void_p, c_int, c_void_p, c_int, c_ll, c_void_p],
    "fb_rope_kv_write": [c_void_p, c_int, c_ll, c_int, c_ll, c_void_p, c_int, c_ll, c_void_p,
                         c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_ll, c_ll,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "fb_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int,
                     c_int, c_void_p],
    "fb_attention_simt": [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p,
                          c_int, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_float, c_void_p],
    "fb_sum_planes": [c_void_p, c_int, c_ll, c_ll, c_void_p, c_int, c_void_p],
    "fb_gemm_tc": [c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_ll, c_int,
                   c_int, c_int, c_ll, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_int,
                   c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_ll, c_void_p,
                   c_void_p, c_ll, c_void_p, c_int, c_void_p],
    "fb_gemm_tc_rope": [c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_ll,
                        c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                        c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_ll,
                        c_ll, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p],
    "fb_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "fb_gemm_tc_status": [c_void_p],
    "fb_gemm_tc_pair_status": [c_void_p],
    "fb_gemm_skinny": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_int,
                       c_int, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p, c_int, c_int, c_int,
                       c_float, c_void_p],
    "fb_gemm_skinny_residual": [c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_void_p,
                                c_ll, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_ll,
                                c_int, c_void_p],
    "fb_apply_row_scale": [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                           c_ll, c_int, c_int, c_void_p],
    "fb_gemm_skinny_rope": [c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p,
                            c_void_p, c_int, c_void_p, c_int, c_void_p, c_ll, c_void_p, c_void_p,
                            c_ll, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_ll,
                            c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "fb_attention_prefill": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_void_p],
    "fb_attention_prefill_tc": [c_void_p, c_ll, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                c_int, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_float, c_void_p],
    "fb_attention_tc_status": [c_void_p],
    "fb_attention_decode": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int, c_float,
                            c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_ll, c_int, c_void_p],
    "fb_gemm_rows": [c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_int,
                     c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_ll, c_void_p,
                     c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                     c_void_p, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int,
                     c_int, c_int, c_int, c_void_p],
    "fb_gemm_rows_status": [c_void_p],
    "fb_row_scales": [c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p],
    "fb_select_tokens": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_int, c_void_p, c_void_p, c_void_p],
}

_FUNCS = {}


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported a failure."""


def _fn(name: str):
    fn = _FUNCS.get(name)
    if fn is None:
        lib = library.load()
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise library.KernelLibraryError(f"the kernel library lacks {name}") from None
        fn.argtypes = _SIGNATURES[name]
        fn.restype = ctypes.c_int
        _FUNCS[name] = fn
    return fn


_COUNT = [0]


class Profiler:
    """Dispatch counts, and in `kernels` mode GPU time, per kernel: the
    reference's `DeviceProfile` (src/nn/profile.rs:15-28). `steps` mode only
    counts and leaves execution unchanged; `kernels` mode brackets every launch
    with CUDA events, so it needs plain launches (no graph replay) and perturbs
    wall times. Product kernels are keyed with their shape, as the reference
    keys its matmul (src/metal/args.rs:196-204)."""

    def __init__(self):
        self.mode = None
        self._counts = {}
        self._events = []
        self._alloc0 = None

    def start(self, mode) -> None:
        if mode not in (None, "steps", "kernels"):
            raise ValueError(f"profile mode {mode!r}: choose steps or kernels")
        self.mode = mode
        self.take()

    def count(self, key: str, times: int = 1) -> None:
        self._counts[key] = self._counts.get(key, 0) + times

    def snapshot_counts(self):
        return dict(self._counts)

    def add_counts(self, counts) -> None:
        for key, n in counts.items():
            self.count(key, n)

    def take(self) -> dict:
        """The profile since the last `take`, and a fresh start."""
        kernels = {k: {"dispatch_count": n} for k, n in sorted(self._counts.items())}
        if self._events:
            torch.cuda.synchronize()
            for key, a, b in self._events:
                entry = kernels.setdefault(key, {"dispatch_count": 0})
                entry["gpu_ns"] = entry.get("gpu_ns", 0.0) + a.elapsed_time(b) * 1e6
        stats = torch.cuda.memory_stats() if torch.cuda.is_available() else {}
        now = (stats.get("allocation.all.allocated", 0), stats.get("allocated_bytes.all.allocated", 0))
        before = self._alloc0 or now
        self._alloc0 = now
        self._counts, self._events = {}, []
        busy = sum(k["gpu_ns"] for k in kernels.values() if "gpu_ns" in k) if self.mode == "kernels" else None
        return {"kernels": kernels, "allocation_count": now[0] - before[0],
                "allocated_bytes": now[1] - before[1], "gpu_busy_ns": busy}


PROFILER = Profiler()


def launch_count() -> int:
    """Kernels of this library launched so far (graph replays included)."""
    return _COUNT[0]


def add_launches(n: int) -> None:
    _COUNT[0] += n



def _call(name: str, *args, tag=None) -> None:
    """Launch `name`. `tag` is (format, values...) naming the shape for the
    profiler; it is formatted only when a profile is being taken."""
    _COUNT[0] += 1
    prof = PROFILER
    if prof.mode is not None:
        key = name[3:] + (" " + tag[0].format(*tag[1:]) if tag else "")
        prof.count(key)
        if prof.mode == "kernels" and not torch.cuda.is_current_stream_capturing():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            code = _fn(name)(*args)
            b.record()
            prof._events.append((key, a, b))
            if code != 0:
                message = library.load().fb_last_error().decode(errors="replace")
                raise KernelError(f"{name}: {message}")
            return
    code = _fn(name)(*args)
    if code != 0:
        message = library.load().fb_last_error().decode(errors="replace")
        raise KernelError(f"{name}: {message}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle. This is called once per launch: the raw
    getter costs a fraction of a microsecond, `torch.cuda.current_stream()` ten."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def code_of(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} has no kernel") from None


def _dev(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA devices only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    return t.data_ptr()


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride of a 2-d tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-d with contiguous rows, got strides {t.stride()}")
    return t.stride(0)


class Planes:
    """Partial results of a split-K product: float32 [splits, rows, cols] whose
    sum over the first axis is the product. Consumers (the residual-add-norm
    kernel, the rotary kernel) sum them in plane order while they read."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor

    @property
    def shape(self):
        return self.tensor.shape[1:]

    @property
    def count(self) -> int:
        return self.tensor.shape[0]

    def sum(self, dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(self.shape, dtype=dtype, device=self.tensor.device)
        return sum_planes(self.tensor, out)


class ResidualSink:
    """What a part's last projection may do instead of returning its result:
    add it to the float32 residual rows `resid` and prepare the input of the
    norm with weight `gamma` and `eps` that follows (see `gemm_bf16`)."""

    def __init__(self, resid: torch.Tensor, gamma: torch.Tensor, eps: float):
        self.resid, self.gamma, self.eps = resid, gamma, float(eps)


class RowScaled:
    """A norm's output that still lacks its row scale: `values` [T, H] bfloat16
    hold resid * gamma, and token t's scale is
    1 / sqrt(sum_c shares[c, t] / H + eps). The weight-streaming products
    multiply their results by it (the product is linear in the scale);
    `materialize` gives the plain tensor for anything else."""

    def __init__(self, values: torch.Tensor, shares: torch.Tensor, eps: float):
        self.values, self.shares, self.eps = values, shares, float(eps)
        self._scales = None

    @property
    def shape(self):
        return self.values.shape

    @property
    def dtype(self):
        return self.values.dtype

    @property
    def device(self):
        return self.values.device

    def scale_args(self):
        """(shares, count, stride, dim, eps) as the kernels take them."""
        return (self.shares.data_ptr(), self.shares.shape[0], self.shares.stride(0),
                self.values.shape[1], self.eps)

    def scales_args(self):
        """The same for kernels that take the tokens' scales themselves (a count
        of 0): one small kernel adds the shares up once, where the epilogues of
        a product of many rows would do it again for every tile."""
        if self._scales is None:
            T = self.values.shape[0]
            self._scales = torch.empty(T, dtype=torch.float32, device=self.values.device)
            _call("fb_row_scales", self.shares.data_ptr(), self.shares.shape[0],
                  self.shares.stride(0), self.values.shape[1], self.eps, self._scales.data_ptr(),
                  T, _stream())
        return (self._scales.data_ptr(), 0, 0, self.values.shape[1], self.eps)

    def materialize(self) -> torch.Tensor:
        T, H = self.values.shape
        out = torch.empty_like(self.values)
        _call("fb_apply_row_scale", _dev(self.values, "values", torch.bfloat16), H,
              *self.scale_args(), out.data_ptr(), H, T, H, _stream())
        return out


class NormPending:
    """The result of a projection that took a `ResidualSink`: the sum is already
    in `sink.resid`; the norm that `sink` named turns this into a `RowScaled`."""

    def __init__(self, sink: ResidualSink, values: torch.Tensor, shares: torch.Tensor):
        self.sink, self.values, self.shares = sink, values, shares


_NO_SCALE = (0, 0, 0, 0, 0.0)
MAX_SCALE_SHARES = 384  # FB_SKINNY_MAX_SHARES in csrc/gemm_skinny.cu


def _scale_of(x):
    """(scale arguments, tensor) of a weight-streaming product's input."""
    if not isinstance(x, RowScaled):
        return _NO_SCALE, x
    if x.shares.shape[0] > MAX_SCALE_SHARES:  # more than the kernel stages: apply it here
        return _NO_SCALE, x.materialize()
    return x.scale_args(), x.values


def plain(x):
    """`x` as a tensor: a `RowScaled` gets its scale applied."""
    return x.materialize() if isinstance(x, RowScaled) else x


# ------------------------------------------------------------------ embedding
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t,:] = table[ids[t],:] as float32; `out` is [T, H] float32."""
    V, H = table.shape
    T = ids.numel()
    if out.shape != (T, H):
        raise KernelError(f"embed_gather: out is {tuple(out.shape)}, expected {(T, H)}")
    _call("fb_embed_gather", _dev(table, "table"), code_of(table.dtype),
          _dev(ids, "ids", torch.int32), _dev(out, "out", torch.float32), T, H, V, _stream())
    return out


# ------------------------------------------------------ residual + RMS norm
def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """resid += delta (a tensor, split-K `Planes`, or None), in place, float32;
    out = rmsnorm(resid) * weight. With `out=None` only the sum is made. A
    `NormPending` delta (the sum was made by the projection) comes back as the
    `RowScaled` input of the next projection, and no kernel runs."""
    T, H = resid.shape
    if isinstance(delta, NormPending):
        sink = delta.sink
        if sink.resid.data_ptr() != resid.data_ptr() or sink.gamma.data_ptr() != weight.data_ptr() \
                or sink.eps != float(eps):
            raise KernelError("add_rmsnorm: the projection before this norm prepared its input "
                              "for another residual or another norm")
        return RowScaled(delta.values, delta.shares, eps)
    planes, plane_stride = 1, 0
    if isinstance(delta, Planes):
        planes, plane_stride = delta.count, T * H
        delta = delta.tensor
        if tuple(delta.shape[1:]) != (T, H) or not delta.is_contiguous():
            raise KernelError(f"add_rmsnorm: planes are {tuple(delta.shape)}, resid {(T, H)}")
    elif delta is not None and delta.shape != resid.shape:
        raise KernelError(f"add_rmsnorm: delta is {tuple(delta.shape)}, resid {tuple(resid.shape)}")
    if out is not None and out.shape != resid.shape:
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, resid {tuple(resid.shape)}")
    if weight.shape != (H,):
        raise KernelError(f"add_rmsnorm: weight is {tuple(weight.shape)}, expected {(H,)}")
    _call("fb_add_rmsnorm", _dev(resid, "resid", torch.float32),
          0 if delta is None else _dev(delta, "delta"),
          F32 if delta is None else code_of(delta.dtype), planes, plane_stride,
          _dev(weight, "weight", torch.float32), float(eps),
          0 if out is None else _dev(out, "out"),
          F32 if out is None else code_of(out.dtype), T, H, _stream())
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out[t,i] = silu(gate) * up, with gate i / up i in columns i / I+i, or in
    columns 2i / 2i+1 when `interleaved`."""
    T, two_i = gate_up.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} / out {tuple(out.shape)}")
    _call("fb_silu_mul", _dev(gate_up, "gate_up"), _dev(out, "out"), code_of(out.dtype), T,
          two_i // 2, 1 if interleaved else 0, _stream())
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    n, H = out.shape
    if src.shape[1] != H or rows.numel() != n or src.dtype != out.dtype:
        raise KernelError("gather_rows: shapes or dtypes differ")
    _call("fb_gather_rows", _dev(src, "src"), code_of(src.dtype), _dev(rows, "rows", torch.int32),
          _dev(out, "out"), n, H, _stream())
    return out


def cast(src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if src.numel() != out.numel():
        raise KernelError("cast: element counts differ")
    _call("fb_cast", _dev(src, "src"), code_of(src.dtype), _dev(out, "out"), code_of(out.dtype),
          src.numel(), _stream())
    return out


# ------------------------------------------------------------ rope + cache
def rope_kv_write(qkv, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int, ring_pages: int = 0,
                  write_cache: bool = True, q_out: Optional[torch.Tensor] = None,
                  dtype: Optional[torch.dtype] = None, pairing: str = "half") -> torch.Tensor:
    """Rotate the query heads of the fused projection output; rotate the key
    heads into the cache pages and copy the value heads there. `pairing`:
    frequency i turns elements (i, i + rotary_dim / 2) ("half") or (2i, 2i + 1)
    ("interleaved") of the rotary part. `qkv` is a
    tensor (queries are then rotated in place unless `q_out` is given) or
    split-K `Planes`, which are summed on the way (`q_out` of `dtype` is made).
    `k_cache`/`v_cache` are one cache entry's views [pages, kv_heads, PAGE,
    head_dim]. Returns the [T, heads * head_dim] (possibly strided) queries."""
    planes, plane_stride = 1, 0
    if isinstance(qkv, Planes):
        src = qkv.tensor
        planes = qkv.count
        T, width = qkv.shape
        plane_stride, src_stride = T * width, width
        dtype = dtype or (k_cache.dtype if k_cache is not None else torch.bfloat16)
        if q_out is None:
            q_out = torch.empty((T, num_heads * head_dim), dtype=dtype, device=src.device)
    else:
        src = qkv
        T = qkv.shape[0]
        src_stride = _rows(qkv, "qkv")
        dtype = qkv.dtype
        if q_out is None:
            q_out = qkv[:, :num_heads * head_dim]
    if positions.numel() != T or seq_of_token.numel() != T:
        raise KernelError("rope_kv_write: positions / seq_of_token do not cover the tokens")
    if inv_freq.numel() * 2 != rotary_dim:
        raise KernelError("rope_kv_write: inv_freq does not hold rotary_dim / 2 entries")
    page_stride = head_stride = 0
    kp = vp = 0
    if write_cache:
        _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, dtype)
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        kp, vp = k_cache.data_ptr(), v_cache.data_ptr()
    _call("fb_rope_kv_write", _dev(src, "qkv", contiguous=False), code_of(src.dtype), src_stride,
          planes, plane_stride, _dev(q_out, "q_out", dtype, contiguous=False), code_of(dtype),
          _rows(q_out, "q_out"), _dev(positions, "positions", torch.int32),
          _dev(seq_of_token, "seq_of_token", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1],
          _dev(inv_freq, "inv_freq", torch.float32), rotary_dim, kp, vp, page_stride, head_stride,
          ring_pages, T, num_heads, num_kv_heads, head_dim, 1 if write_cache else 0,
          _pairing_code(pairing), _stream())
    return q_out


PAIRINGS = {"half": 0, "interleaved": 1}


def _pairing_code(pairing: str) -> int:
    try:
        return PAIRINGS[pairing]
    except KeyError:
        raise KernelError(f"rotation pairing {pairing!r}: choose one of {sorted(PAIRINGS)}") from None


def _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, dtype) -> None:
    for name, c in (("k_cache", k_cache), ("v_cache", v_cache)):
        if c is None or not c.is_cuda or c.dtype != dtype:
            raise KernelError(f"{name} must be a CUDA tensor of dtype {dtype}")
        if c.dim() != 4 or c.shape[1:] != (num_kv_heads, PAGE, head_dim):
            raise KernelError(f"{name} is {tuple(c.shape)}, expected "
                              f"[pages, {num_kv_heads}, {PAGE}, {head_dim}]")
        if c.stride(3) != 1 or c.stride(2) != head_dim:
            raise KernelError(f"{name}: the rows of a page must be contiguous")
    if k_cache.stride() != v_cache.stride():
        raise KernelError("k_cache and v_cache differ in layout")


# ------------------------------------------------------------------- products
def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M,N] = x[M,K] @ w[N,K]^T with 32-bit FFMA accumulation."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or x.dtype != w.dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}, "
                          f"out {tuple(out.shape)}")
    _call("fb_gemm_simt", _dev(x, "x", contiguous=False), _dev(w, "w", contiguous=False),
          _dev(out, "out", contiguous=False), M, N, K, _rows(x, "x"), _rows(w, "w"),
          _rows(out, "out"), code_of(x.dtype), code_of(out.dtype), _stream(),
          tag=("m{} k{} n{}", M, K, N))
    return out


_SM_OF_DEVICE = {}


def sm_count() -> int:
    """SMs of the current device (asked once per device): the plans below size
    their grids to cover the SMs once."""
    device = torch.cuda.current_device()
    count = _SM_OF_DEVICE.get(device)
    if count is None:
        count = _SM_OF_DEVICE[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


# many token rows: one CTA per SM walks the tiles, two accumulators in tensor memory
PERSISTENT = _os.environ.get("FOUNDRY_B200_PERSISTENT", "1") != "0"
# two SMs on one 256-row tile (tcgen05 cta_group::2) for more than 128 token rows
PAIRED = _os.environ.get("FOUNDRY_B200_PAIRED", "1") != "0"
# up to this many token rows the one-tile product is considered beside the paired one
ONE_TILE_ROWS = int(_os.environ.get("FOUNDRY_B200_ONE_TILE_ROWS", "768"))


# The paired product shares the K of a thin last round's tiles among CTA pairs
# (float32 partial tiles in a workspace, summed by the warp that delivers last).
PAIR_TAIL_SHARES = _os.environ.get("FOUNDRY_B200_PAIR_TAIL_SHARES", "1") != "0"
PAIR_SHARE_MIN_KBLOCKS = 0  # K blocks of 64 a share keeps at least (0: the launcher's 32)
_PAIR_SCRATCH = {}
_SCRATCH_OWNER = threading.local()


class scratch_owner:
    """Within this block, kernels that need scratch memory between their CTAs
    (the paired product's shares, decode attention's arrival counters) take the
    scratch that belongs to `owner` (any hashable name): an engine runs its
    steps inside one, so two engines on two streams never meet in one buffer.
    Outside any block the scratch is the device's common one; calls that share a
    scratch must follow one another on one stream."""

    def __init__(self, owner):
        self.owner = owner

    def __enter__(self):
        self.previous = getattr(_SCRATCH_OWNER, "key", None)
        _SCRATCH_OWNER.key = self.owner
        return self

    def __exit__(self, *exc):
        _SCRATCH_OWNER.key = self.previous
        return False


def release_scratch(owner) -> None:
    """Forget the scratch of an owner that is gone."""
    for table in (_PAIR_SCRATCH, _COUNTERS):
        for key in [k for k in table if k[1] == owner]:
            del table[key]


def _scratch_key(device):
    index = device.index if device.index is not None else torch.cuda.current_device()
    return index, getattr(_SCRATCH_OWNER, "key", None)


def _pair_scratch(device):
    """(float32 workspace for the partial tiles of one round: 74 tiles of
    256 x 256; zeroed int32 counters, 8 per tile), one pair per device and
    scratch owner."""
    key = _scratch_key(device)
    got = _PAIR_SCRATCH.get(key)
    if got is None:
        if torch.cuda.is_current_stream_capturing():
            # memory made during a capture belongs to that graph; this must outlive it
            raise KernelError("the paired product's workspace must be made before a stream "
                              "capture: run the step once before capturing it")
        got = _PAIR_SCRATCH[key] = (
            torch.empty((sm_count() // 2) * 256 * 256, dtype=torch.float32, device=device),
            torch.zeros((sm_count() // 2) * 8, dtype=torch.int32, device=device))
    return got


def gemm_tc(a, b: torch.Tensor, out: Optional[torch.Tensor], stride_a: int, stride_b: int,
            bn: int, splits: int = 1, split_stride: int = 0, epilogue: int = 0,
            constant_operand: int = 0, persistent: int = 0,
            sink: Optional[ResidualSink] = None, sink_out=None) -> None:
    """Tensor-core product D[i,j] = sum_k a[i,k] b[j,k] written to
    out[i*stride_a + j*stride_b (+ split*split_stride)]; see csrc/gemm_tcgen05.cu.
    With tokens as the rows of `a` (stride_b == 1, one split): `a` may be a
    `RowScaled`, and `sink` (with `sink_out` = (values, shares)) makes the
    epilogue add into the residual rows in front of a norm instead of storing."""
    scale = _NO_SCALE
    if isinstance(a, RowScaled):
        scale, a = a.scales_args(), a.values
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    sink_args = (0, 0, 0, 0, 0, 0, 0)
    if sink is not None:
        values, shares = sink_out
        sink_args = (_dev(sink.resid, "resid", torch.float32, contiguous=False),
                     _rows(sink.resid, "resid"), _dev(sink.gamma, "gamma", torch.float32),
                     values.data_ptr(), values.stride(0), shares.data_ptr(), shares.stride(0))
        epilogue, out = 2, values  # `out` only names a buffer for the argument checks
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm_tc writes float32 or bfloat16, not {out.dtype}")
    scratch = (0, 0, 0, 0)
    if int(persistent) == 2 and PAIR_TAIL_SHARES:
        work, counters = _pair_scratch(a.device)
        scratch = (work.data_ptr(), work.numel() * 4, counters.data_ptr(), counters.numel())
    _call("fb_gemm_tc", _dev(a, "a", contiguous=False), _rows(a, "a"), a.shape[0],
          _dev(b, "b", contiguous=False), _rows(b, "b"), b.shape[0], a.shape[1],
          _dev(out, "out", contiguous=False), stride_a, stride_b,
          1 if out.dtype == torch.float32 else 0, bn, splits, split_stride, epilogue,
          constant_operand, int(persistent), *scratch, PAIR_SHARE_MIN_KBLOCKS, *scale, *sink_args,
          _stream(),
          tag=("a{} b{} k{} tile{} splits{}", a.shape[0], b.shape[0], a.shape[1], bn, splits))


# Bytes of the next kernel's weights that a single-token-step kernel asks into
# L2 while it finishes (0 switches the hints off).
L2_PREFETCH_BYTES = int(float(_os.environ.get("FOUNDRY_B200_L2_PREFETCH_MB", "8")) * (1 << 20))


def _prefetch_range(then_reads: Optional[torch.Tensor]):
    """(address, bytes) of the start of `then_reads` to bring into L2, or (0, 0)."""
    if then_reads is None or L2_PREFETCH_BYTES <= 0 or not then_reads.is_cuda:
        return 0, 0
    size = min(then_reads.numel() * then_reads.element_size(), L2_PREFETCH_BYTES) // 16 * 16
    if not then_reads.is_contiguous() or then_reads.data_ptr() % 16 or size <= 0:
        return 0, 0
    return then_reads.data_ptr(), size


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0,
                then_reads: Optional[torch.Tensor] = None, ksplit: int = 1,
                warps: int = 0) -> torch.Tensor:
    """Up to 16 token rows: the weight-streaming kernel (csrc/gemm_skinny.cu).
    epilogue 1: `w` rows are (gate, up) pairs and out is [M, N/2] = SiLU(gate)*up.
    `then_reads`: the weights the step streams after this product; the kernel's
    blocks ask for their start to be brought into L2 as they finish.
    `ksplit` > 1: K is shared by that many CTAs per row group and `out` is
    float32 planes [ksplit, M, N]. `warps`: 4, 8 or 16 per CTA (0: the
    launcher's choice)."""
    scale, x = _scale_of(x)
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny takes bfloat16 operands")
    want = (M, N // 2) if epilogue else (M, N)
    if ksplit > 1:
        want = (ksplit, *want)
        if out.dtype != torch.float32 or not out.is_contiguous():
            raise KernelError("gemm_skinny: K shares are written as contiguous float32 planes")
    if tuple(out.shape) != want or w.shape[1] != K:
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _call("fb_gemm_skinny", _dev(x, "x", contiguous=False), _rows(x, "x"),
          _dev(w, "w", contiguous=False), _rows(w, "w"), _dev(out, "out", contiguous=False),
          _rows(out, "out") if ksplit == 1 else N, 1 if out.dtype == torch.float32 else 0,
          M, N, K, epilogue,
          *_prefetch_range(then_reads), ksplit, M * N if ksplit > 1 else 0, warps, *scale,
          _stream(), tag=("m{} k{} n{}", M, K, N))
    return out


def gemm_skinny_residual(x: torch.Tensor, w: torch.Tensor, sink: ResidualSink,
                         then_reads: Optional[torch.Tensor] = None, warps: int = 0) -> NormPending:
    """Up to 16 token rows in front of a norm: sink.resid += x w^T in the
    product's epilogue, which also leaves resid * gamma in bfloat16 and each
    CTA's share of the rows' sums of squares for the product behind the norm."""
    M, K = x.shape
    N = w.shape[0]
    resid = sink.resid
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_skinny_residual: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)}")
    if tuple(resid.shape) != (M, N) or tuple(sink.gamma.shape) != (N,):
        raise KernelError(f"gemm_skinny_residual: resid {tuple(resid.shape)}, gamma "
                          f"{tuple(sink.gamma.shape)} for a product of {(M, N)}")
    values = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    shares = torch.empty(((N + 15) // 16, 16), dtype=torch.float32, device=x.device)
    _call("fb_gemm_skinny_residual", _dev(x, "x", contiguous=False), _rows(x, "x"),
          _dev(w, "w", contiguous=False), _rows(w, "w"), M, N, K,
          _dev(resid, "resid", torch.float32, contiguous=False), _rows(resid, "resid"),
          _dev(sink.gamma, "gamma", torch.float32), values.data_ptr(), N, shares.data_ptr(), 16,
          *_prefetch_range(then_reads), warps, _stream(), tag=("m{} k{} n{}", M, K, N))
    return NormPending(sink, values, shares)


def qkv_rows_rope_fusable(x, w: torch.Tensor, rotary_dim: int, head_dim: int,
                          k_cache: Optional[torch.Tensor], pairing: str) -> bool:
    """Whether `gemm_rows_rope` takes this projection: 17 to 256 bfloat16 token
    rows and a rotation of adjacent features."""
    return (FUSE_QKV_ROPE and rows_usable(x, w) and pairing == "interleaved"
            and rotary_dim % 4 == 0 and head_dim % 4 == 0
            and (k_cache is None or k_cache.dtype == torch.bfloat16))


def qkv_rope_fusable(x: torch.Tensor, w: torch.Tensor, rotary_dim: int, head_dim: int,
                     k_cache: Optional[torch.Tensor]) -> bool:
    """Whether `gemm_skinny_rope` takes this projection: bfloat16, few token
    rows, and a rotation whose pairs fall into the kernel's 8-row halves."""
    if isinstance(x, RowScaled):
        x = x.values
    return (FUSE_QKV_ROPE and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and 0 < x.shape[0] <= SKINNY_ROWS and _tc_usable(x, w, x)
            and rotary_dim % 16 == 0 and head_dim % 16 == 0
            and (k_cache is None or k_cache.dtype == torch.bfloat16))


def gemm_skinny_rope(x: torch.Tensor, w: torch.Tensor, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, page_table: torch.Tensor, inv_freq: torch.Tensor,
                     rotary_dim: int, k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                     head_dim: int, ring_pages: int = 0, write_cache: bool = True,
                     then_reads: Optional[torch.Tensor] = None,
                     pairing: str = "half") -> torch.Tensor:
    """The fused q/k/v projection of up to 16 tokens, rotated and stored by the
    product's epilogue: returns the rotated queries [T, heads * head_dim]; the
    rotated keys and the values go into the cache pages (`rope_kv_write` has
    the meaning of the arguments). `w` is [(heads + 2 kv_heads) * head_dim, K].
    The attention behind it may have its blocks placed early only for contexts
    of up to `ROPE_TRIGGER_PAGES` pages: measured on the 3B decode step, that
    gained 1 to 2 % at 512 and 3,072 tokens of context and lost 11 % at 8 K and
    16 K."""
    scale, x = _scale_of(x)
    T, K = x.shape
    if w.shape != ((num_heads + 2 * num_kv_heads) * head_dim, K):
        raise KernelError(f"gemm_skinny_rope: w is {tuple(w.shape)} for {num_heads}+2x{num_kv_heads} "
                          f"heads of {head_dim} and K={K}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny_rope takes bfloat16 operands")
    if positions.numel() != T or seq_of_token.numel() != T:
        raise KernelError("gemm_skinny_rope: positions / seq_of_token do not cover the tokens")
    if inv_freq.numel() * 2 != rotary_dim:
        raise KernelError("gemm_skinny_rope: inv_freq does not hold rotary_dim / 2 entries")
    q_out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    page_stride = head_stride = kp = vp = 0
    if write_cache:
        _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        kp, vp = k_cache.data_ptr(), v_cache.data_ptr()
    _call("fb_gemm_skinny_rope", _dev(x, "x", contiguous=False), _rows(x, "x"),
          _dev(w, "w", contiguous=False), _rows(w, "w"), T, K,
          _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1],
          _dev(inv_freq, "inv_freq", torch.float32) if rotary_dim else 0, rotary_dim,
          q_out.data_ptr(), q_out.stride(0), kp, vp, page_stride, head_stride, ring_pages,
          num_heads, num_kv_heads, head_dim, 1 if write_cache else 0, _pairing_code(pairing),
          *_prefetch_range(then_reads), skinny_plan(w.shape[0], K, False)[1],
          1 if page_table.shape[1] <= ROPE_TRIGGER_PAGES else 0, *scale, _stream(),
          tag=("m{} k{} n{}", T, K, w.shape[0]))
    return q_out


# ----------------------------------------------- 17 .. 256 token rows (tcgen05)
# Token rows up to which the product that shares a weight tile's K among the CTAs
# of a cluster and sums in the kernel is taken (csrc/gemm_rows_tcgen05.cu);
# ROWS_MAX = 0 keeps the one-tile product with float32 planes. Up to 64 rows this
# kernel makes the decode step faster; at 128 rows it has only three shared-memory
# stages and the one-tile product stays ahead. The kernel itself takes up to 256 rows.
# ROWS_SPLITS overrides the CTAs per weight tile (0: the launcher's choice).
ROWS_SPLITS = int(_os.environ.get("FOUNDRY_B200_ROWS_SPLITS", "0"))
ROWS_MAX = int(_os.environ.get("FOUNDRY_B200_ROWS_MAX", "64"))
def rows_usable(x, w) -> bool:
    """Whether the few-rows tcgen05 product takes this projection."""
    values = x.values if isinstance(x, RowScaled) else x
    return (SKINNY_ROWS < values.shape[0] <= ROWS_MAX and values.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and _tc_usable(values, w, values))


def _gemm_rows(x, w, epilogue: int, out=None, sink: Optional[ResidualSink] = None,
               sink_out=None, rope=None) -> None:
    """The launcher's face; `x` may be a `RowScaled`."""
    scale = _NO_SCALE
    if isinstance(x, RowScaled):
        scale, x = x.scale_args(), x.values
    M, K = x.shape
    N = w.shape[0]
    out_args = (0, 0, 0)
    if out is not None:
        out_args = (_dev(out, "out", contiguous=False), _rows(out, "out"),
                    1 if out.dtype == torch.float32 else 0)
    sink_args = (0, 0, 0, 0, 0, 0, 0)
    if sink is not None:
        values, shares = sink_out
        sink_args = (_dev(sink.resid, "resid", torch.float32, contiguous=False),
                     _rows(sink.resid, "resid"), _dev(sink.gamma, "gamma", torch.float32),
                     values.data_ptr(), values.stride(0), shares.data_ptr(), shares.stride(0))
    rope_args = (0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0)
    if rope is not None:
        rope_args = rope
    _call("fb_gemm_rows", _dev(x, "x", torch.bfloat16, contiguous=False), _rows(x, "x"), M,
          _dev(w, "w", torch.bfloat16, contiguous=False), _rows(w, "w"), N, K, *out_args, epilogue,
          *scale, *sink_args, *rope_args, ROWS_SPLITS, _stream(),
          tag=("m{} k{} n{} e{}", M, K, N, epilogue))


def gemm_rows(x, w: torch.Tensor, out: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, silu_mul: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for 17 to 256 token rows (any count up to
    256 works); with `silu_mul` the weight rows are (gate, up) pairs and out is
    [M, N / 2]. `x` may be a `RowScaled`."""
    M, N = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype or torch.bfloat16,
                          device=w.device)
    if tuple(out.shape) != (M, N // 2 if silu_mul else N) or out.stride(1) != 1:
        raise KernelError(f"gemm_rows: out is {tuple(out.shape)} for x {tuple(x.shape)}, w {tuple(w.shape)}")
    _gemm_rows(x, w, 1 if silu_mul else 0, out=out)
    return out


def gemm_rows_residual(x: torch.Tensor, w: torch.Tensor, sink: ResidualSink) -> NormPending:
    """The same product in front of a norm: sink.resid += x w^T in the epilogue,
    which also leaves resid * gamma in bfloat16 and each weight tile's share of
    the rows' sums of squares (see `gemm_skinny_residual`)."""
    M, N = x.shape[0], w.shape[0]
    if tuple(sink.resid.shape) != (M, N) or tuple(sink.gamma.shape) != (N,):
        raise KernelError(f"gemm_rows_residual: resid {tuple(sink.resid.shape)}, gamma "
                          f"{tuple(sink.gamma.shape)} for a product of {(M, N)}")
    values = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
    shares = torch.empty(((N + 127) // 128, (M + 31) // 32 * 32), dtype=torch.float32, device=w.device)
    _gemm_rows(x, w, 2, sink=sink, sink_out=(values, shares))
    return NormPending(sink, values, shares)


def gemm_rows_rope(x, w: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                   page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   num_heads: int, num_kv_heads: int, head_dim: int, ring_pages: int = 0,
                   write_cache: bool = True) -> torch.Tensor:
    """The fused q/k/v projection of 17 to 256 tokens, rotated and stored by the
    product's epilogue (see `gemm_skinny_rope`). The rotation pairs ADJACENT
    features (frequency i turns features 2i and 2i + 1 of a head): the caller's
    weight rows are laid out for the "interleaved" pairing."""
    M, K = x.shape
    rows = (num_heads + 2 * num_kv_heads) * head_dim
    if w.shape != (rows, K):
        raise KernelError(f"gemm_rows_rope: w is {tuple(w.shape)} for {num_heads}+2x{num_kv_heads} "
                          f"heads of {head_dim} and K={K}")
    if positions.numel() != M or seq_of_token.numel() != M or inv_freq.numel() * 2 != rotary_dim:
        raise KernelError("gemm_rows_rope: positions / seq_of_token / inv_freq do not fit")
    q_out = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=w.device)
    kp = vp = page_stride = head_stride = 0
    if write_cache:
        _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        kp, vp = k_cache.data_ptr(), v_cache.data_ptr()
    else:
        w = w[:num_heads * head_dim]  # keys and values are another layer's: not computed
    rope = (_dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
            _dev(page_table, "page_table", torch.int32), page_table.shape[1],
            _dev(inv_freq, "inv_freq", torch.float32) if rotary_dim else 0, rotary_dim,
            q_out.data_ptr(), q_out.stride(0), kp, vp, page_stride, head_stride, ring_pages,
            num_heads, num_kv_heads, head_dim)
    _gemm_rows(x, w, 3, rope=rope)
    return q_out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [frequencies, tokens, 2]: cos and sin of position * frequency, the
    angle a 32-bit product as in the rotary kernels. One table serves every layer
    of a step whose encodings share the frequencies."""
    T, half = positions.numel(), inv_freq.numel()
    cs = torch.empty((half, T, 2), dtype=torch.float32, device=positions.device)
    _call("fb_rope_table", _dev(positions, "positions", torch.int32),
          _dev(inv_freq, "inv_freq", torch.float32) if half else 0, T, half, cs.data_ptr(),
          _stream())
    return cs


def qkv_tc_rope_fusable(x, w: torch.Tensor, rotary_dim: int, head_dim: int,
                        k_cache: Optional[torch.Tensor], pairing: str) -> bool:
    """Whether `gemm_tc_rope` takes this projection: more bfloat16 token rows than
    the few-rows product takes, in a product form that is not split along K, heads
    of whole 32-feature groups and a rotation of adjacent features."""
    values = x.values if isinstance(x, RowScaled) else x
    if not (FUSE_QKV_ROPE_MANY and values.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and pairing == "interleaved" and head_dim % 32 == 0 and rotary_dim % 2 == 0
            and (k_cache is None or k_cache.dtype == torch.bfloat16)
            and _tc_usable(values, w, values)):
        return False
    M, K = values.shape
    # not where `gemm_bf16` would split K over CTAs (float32 planes): unsplit, those
    # sizes run slower than the rotary kernel costs
    splits, fits = _one_tile_plan(M, w.shape[0], K)
    many = M > 128 and not (fits and M <= ONE_TILE_ROWS)
    return many or splits == 1


def gemm_tc_rope(x, w: torch.Tensor, cs: torch.Tensor, positions: torch.Tensor,
                 seq_of_token: torch.Tensor, page_table: torch.Tensor, rotary_dim: int,
                 k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                 num_heads: int, num_kv_heads: int, head_dim: int, ring_pages: int = 0,
                 write_cache: bool = True) -> torch.Tensor:
    """The fused q/k/v projection of many tokens on the token-major tcgen05
    products, rotated and stored by their epilogue: queries come back, keys and
    values go into the cache (see `gemm_skinny_rope`; the rotation pairs ADJACENT
    features, `cs` is `rope_table`'s). The product's form is chosen as
    `gemm_bf16` chooses it for these sizes."""
    scale = _NO_SCALE
    if isinstance(x, RowScaled):
        scale, x = x.scales_args(), x.values
    M, K = x.shape
    rows = (num_heads + 2 * num_kv_heads) * head_dim
    if w.shape != (rows, K):
        raise KernelError(f"gemm_tc_rope: w is {tuple(w.shape)} for {num_heads}+2x{num_kv_heads} "
                          f"heads of {head_dim} and K={K}")
    if positions.numel() != M or seq_of_token.numel() != M or \
            tuple(cs.shape) != (rotary_dim // 2, M, 2) or cs.dtype != torch.float32:
        raise KernelError("gemm_tc_rope: positions / seq_of_token / the angle table do not fit")
    q_out = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=w.device)
    kp = vp = page_stride = head_stride = 0
    if write_cache:
        _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        kp, vp = k_cache.data_ptr(), v_cache.data_ptr()
    else:
        w = w[:num_heads * head_dim]  # keys and values are another layer's: not computed
    N = w.shape[0]
    splits, fits = _one_tile_plan(M, N, K)
    many = M > 128 and not (fits and M <= ONE_TILE_ROWS and splits == 1)
    bn, form = prompt_plan(M, N) if many else (128, 0)  # never split along K
    scratch = (0, 0, 0, 0)
    if form == 2 and PAIR_TAIL_SHARES:
        work, counters = _pair_scratch(x.device)
        scratch = (work.data_ptr(), work.numel() * 4, counters.data_ptr(), counters.numel())
    _call("fb_gemm_tc_rope", _dev(x, "x", torch.bfloat16, contiguous=False), _rows(x, "x"), M,
          _dev(w, "w", torch.bfloat16, contiguous=False), _rows(w, "w"), K, bn, form, *scratch,
          PAIR_SHARE_MIN_KBLOCKS, *scale, cs.data_ptr(), rotary_dim // 2,
          _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1], ring_pages, kp, vp,
          page_stride, head_stride, num_heads, num_kv_heads, head_dim, 1 if write_cache else 0,
          q_out.data_ptr(), q_out.stride(0), _stream(),
          tag=("m{} n{} k{} tile{}", M, N, K, bn))
    return q_out


FUSE_QKV_ROPE = _os.environ.get("FOUNDRY_B200_FUSE_QKV_ROPE", "1") != "0"
# ... and in the token-major tcgen05 products' epilogue (prompt steps)
FUSE_QKV_ROPE_MANY = _os.environ.get("FOUNDRY_B200_FUSE_QKV_ROPE_MANY", "1") != "0"
ROPE_TRIGGER_PAGES = 64  # page-table width up to which the q/k/v product triggers its successor
# the projections around a norm take the norm over (see `ResidualSink`, `RowScaled`)
NORM_FUSION = _os.environ.get("FOUNDRY_B200_NORM_FUSION", "1") != "0"
# ... up to this many token rows. The products whose rows are tokens (more than 64)
# can do the same in their epilogue, and lose by it: a thread of their epilogue owns
# a token, so a warp's read-modify-write of the float32 residual touches 32 rows
# 12 KB apart with 16 bytes each, and a prompt step takes a quarter longer. The norm
# stays a kernel of its own there.
NORM_FUSION_ROWS = int(_os.environ.get("FOUNDRY_B200_NORM_FUSION_ROWS", "64"))


def skinny_plan(N: int, K: int, planes_ok: bool):
    """(K shares, warps per CTA; 0 = the launcher's rule) of the weight-streaming
    product for N weight rows. A CTA owns 16 rows. With fewer row groups than
    SMs, K is shared among CTAs (float32 planes for the consumer to sum) until
    the grid covers the SMs, each share keeping at least 8 chunks of 64.
    Measured on the 3B decode step, sharing K did not pay once the row groups
    alone covered the SMs."""
    override = _SKINNY_PLANS.get(N * 1000003 + K)
    if override:
        return override if planes_ok else (1, override[1])
    groups = (N + 15) // 16
    if planes_ok and groups < sm_count():
        return max(1, min(sm_count() // groups, (K + 63) // 64 // 8)), 0
    return 1, 0


def _parse_plans(text: str):
    plans = {}
    for item in filter(None, text.split(",")):
        n, k, ks, wp = (int(v) for v in item.split(":"))
        plans[n * 1000003 + k] = (ks, wp)
    return plans


_SKINNY_PLANS = _parse_plans(_os.environ.get("FOUNDRY_B200_SKINNY_PLANS", ""))


# token rows up to which the weight-streaming kernel is used
SKINNY_ROWS = int(_os.environ.get("FOUNDRY_B200_SKINNY_ROWS", "16"))


def set_dependent_launch(on: bool) -> None:
    """Switch programmatic dependent launch of the kernels on or off (on by default)."""
    lib = library.load()
    lib.fb_set_pdl.argtypes = [ctypes.c_int]
    lib.fb_set_pdl.restype = None
    lib.fb_set_pdl(1 if on else 0)


if _os.environ.get("FOUNDRY_B200_PDL", "1") == "0":
    set_dependent_launch(False)


_STATUS_READERS = ("fb_gemm_tc_status", "fb_gemm_tc_pair_status", "fb_attention_tc_status",
                   "fb_gemm_rows_status")
# kernel codes of the host-visible failure record (FB_STATUS_KERNEL in csrc)
_STATUS_KERNELS = {1: "tcgen05 product", 2: "paired tcgen05 product", 3: "tcgen05 prompt attention",
                   4: "tcgen05 product for few token rows"}
_STATUS_ROLES = {1: "tile loads", 2: "matrix instructions", 3: "epilogue",
                 20: "shared-memory alignment"}
_MIRROR = []


def gemm_tc_status():
    """0 when no bounded wait of the tcgen05 kernels (products and prompt
    attention) ever ran out, else (role, block, step). Reads and clears the
    status words on the device; synchronises the device."""
    for name in _STATUS_READERS:
        detail = (ctypes.c_int * 3)()
        code = _fn(name)(ctypes.cast(detail, ctypes.c_void_p))
        if code != 0:
            return (code, detail[1], detail[2])
    return 0


def _status_mirror():
    """The failure record in pinned host memory as four ints (kernel, role,
    block, K block), or None if the library could not make it."""
    if not _MIRROR:
        lib = library.load()
        lib.fb_status_mirror.restype = ctypes.c_void_p
        lib.fb_status_mirror.argtypes = []
        address = lib.fb_status_mirror()
        _MIRROR.append((ctypes.c_int * 4).from_address(address) if address else None)
    return _MIRROR[0]


def raise_on_device_failure() -> None:
    """Raise `KernelError` if a kernel gave up on a bounded wait since the last
    check: what it computed after that is garbage, so nothing computed since
    may leave the engine. The kernels record the failure in pinned host memory,
    so the check is a host load; call it where the stream was just
    synchronised (the reference turns device failures into errors of the
    call the same way, src/generate/error.rs `Forward`, `Synchronize`)."""
    record = _status_mirror()
    if record is None or record[0] == 0:
        return
    kernel, role, block, kblock = (int(v) for v in record)
    for i in range(4):
        record[i] = 0
    for name in _STATUS_READERS:  # clear the words on the device too
        _fn(name)(None)
    raise KernelError(
        f"{_STATUS_KERNELS.get(kernel, f'kernel {kernel}')}: a bounded wait ran out "
        f"({_STATUS_ROLES.get(role, f'role {role}')}, block {block}, K block {kblock}); "
        f"the results of this step are not valid")


def sum_planes(planes: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = planes.sum(0) for float32 planes [S, ...], in plane order."""
    S = planes.shape[0]
    n = out.numel()
    if planes.numel() != S * n:
        raise KernelError("sum_planes: plane size differs from the output")
    _call("fb_sum_planes", _dev(planes, "planes", torch.float32), S, n, n, _dev(out, "out"),
          code_of(out.dtype), _stream())
    return out


def _tc_usable(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.stride(1) == 1
            and w.stride(1) == 1 and out.stride(1) == 1)


def _one_tile_plan(M: int, N: int, K: int):
    """(K shares, fits) of the one-tile product: tiles of 128 token rows (the
    last one partly empty) by 128 weight rows; K is shared among CTAs until the
    grid covers the SMs once (a second round cost 0.2 ms a step at batch 64),
    each share writing a float32 plane. `fits`: all CTAs run at once and none
    walks more than 64 K blocks, which is where this form beat the paired one
    for 129 to 768 rows (e.g. 256 rows: O 13 against 22 us, down 22 against
    30, q/k/v 23 against 25; the gate/up product has too many tiles for it)."""
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    kblocks = (K + 63) // 64
    splits = max(1, min(kblocks // 4, sm_count() // tiles))
    per = (kblocks + splits - 1) // splits
    splits = (kblocks + per - 1) // per  # no empty share
    return splits, tiles * splits <= sm_count() and per <= 64


def prompt_tile_width(M: int, N: int) -> int:
    """Tile width (the weights' side) for many token rows: the width whose tile
    count wastes least of the last round over the SMs (rounds x width is the
    time in units of one 128 x 1 column strip); wider on ties."""
    if N < 128:
        return 64
    if not PERSISTENT:
        return 256 if N >= 256 else 128
    tiles_a = (M + 127) // 128
    best, best_cost = 256, None
    for bn in (256, 240, 224, 208, 192, 176, 160, 144, 128):
        rounds = (tiles_a * ((N + bn - 1) // bn) + sm_count() - 1) // sm_count()
        cost = rounds * (bn + 8)  # + a fixed cost per tile
        if best_cost is None or cost < best_cost:
            best, best_cost = bn, cost
    return best


def prompt_plan(M: int, N: int):
    """(tile width, form) of the product for more than 128 token rows: form 2
    pairs two SMs on tiles of 256 token rows (a CTA then takes half of each
    weight tile from L2), form 1 runs one CTA per SM on 128-row tiles, form 0
    one CTA per tile. Paired: the widest tile among those with the fewest
    rounds over the 74 CTA pairs (measured at 2,048 rows, the time of a round
    hardly depends on the width between 176 and 256)."""
    if PAIRED and PERSISTENT and N >= 128:
        blocks = (M + 255) // 256
        pairs = sm_count() // 2
        best, best_rounds = 256, None
        for bn in (256, 240, 224, 208, 192, 176, 160, 144, 128):
            rounds = (blocks * ((N + bn - 1) // bn) + pairs - 1) // pairs
            if best_rounds is None or rounds < best_rounds:
                best, best_rounds = bn, rounds
        return best, 2
    return prompt_tile_width(M, N), 1 if PERSISTENT else 0


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, allow_planes: bool = False,
              then_reads: Optional[torch.Tensor] = None,
              residual: Optional[ResidualSink] = None):
    """out[M,N] = x[M,K] @ w[N,K]^T in bfloat16 with 32-bit accumulation.

    Up to 16 rows: the weight-streaming kernel. More than 128 rows: token rows
    fill the 128-row operand (256 rows over a pair of SMs), weights the other
    (up to 256 wide), see `prompt_plan`. In between: one 128 x 128 tile per
    CTA, the weights stream through once; K is split over CTAs until the grid
    covers the SMs, each split writing a float32 plane.
    With `allow_planes` the planes are returned as `Planes` for a consumer that
    sums them as it reads; otherwise one more kernel sums them in a fixed order.
    Shapes TMA cannot address (K or a row stride not a multiple of 8 elements)
    take the CUDA-core kernel.
    `x` may be a `RowScaled` (the weight-streaming kernel applies the scale, the
    others get the plain tensor). `residual`: the caller would add the result to
    these residual rows and normalise them next; when the weight-streaming kernel
    runs unsplit it does both in its epilogue and a `NormPending` comes back,
    otherwise the result comes back as usual.
    """
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out_dtype = out_dtype or x.dtype
    if M == 0:
        return out if out is not None else torch.empty((0, N), dtype=out_dtype, device=x.device)
    values = x.values if isinstance(x, RowScaled) else x
    usable = _tc_usable(values, w, out if out is not None else values)
    if not usable:
        x = plain(x)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        return gemm_simt(x, w, out)
    if M <= SKINNY_ROWS:
        ksplit, warps = skinny_plan(N, K, allow_planes and out is None)
        if (residual is not None and NORM_FUSION and ksplit == 1 and out is None
                and tuple(residual.resid.shape) == (M, N) and not isinstance(x, RowScaled)
                and (N + 15) // 16 <= MAX_SCALE_SHARES):
            return gemm_skinny_residual(x, w, residual, then_reads=then_reads, warps=warps)
        if ksplit > 1:
            planes = torch.empty((ksplit, M, N), dtype=torch.float32, device=x.device)
            gemm_skinny(x, w, planes, then_reads=then_reads, ksplit=ksplit, warps=warps)
            return Planes(planes)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        return gemm_skinny(x, w, out, then_reads=then_reads, warps=warps)
    if rows_usable(x, w) and (out is None or out.stride(1) == 1):
        if (residual is not None and NORM_FUSION and out is None
                and tuple(residual.resid.shape) == (M, N) and not isinstance(x, RowScaled)):
            return gemm_rows_residual(x, w, residual)
        return gemm_rows(x, w, out, out_dtype)
    splits, fits = _one_tile_plan(M, N, K)
    many = M > 128 and not (fits and M <= ONE_TILE_ROWS)
    if many or splits == 1:
        # tokens are the rows of the tensor-core tile and nothing is split: the epilogue
        # applies a deferred row scale, and in front of a norm adds into the residual
        bn, form = prompt_plan(M, N) if many else (128, 0)
        if (residual is not None and NORM_FUSION and M <= NORM_FUSION_ROWS and out is None
                and tuple(residual.resid.shape) == (M, N) and not isinstance(x, RowScaled)):
            values = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
            shares = torch.empty(((N + bn - 1) // bn, (M + 31) // 32 * 32), dtype=torch.float32,
                                 device=w.device)
            gemm_tc(x, w, None, N, 1, bn, constant_operand=2, persistent=form, sink=residual,
                    sink_out=(values, shares))
            return NormPending(residual, values, shares)
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=w.device)
        gemm_tc(x, w, out, out.stride(0), 1, bn, constant_operand=2, persistent=form)
        return out
    # 17..128 rows (and more, while one round of tiles covers them) with K split over
    # CTAs: the tokens are the (partly empty) 128-row operand, so that a thread of the
    # epilogue owns a token's consecutive features and stores them as vectors; with
    # the weights as the row operand ("swapped") the same product was 2.5 us a call
    # slower, all of it in the scalar stores
    x = plain(x)
    planes = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
    gemm_tc(x, w, planes, N, 1, 128, splits, M * N, constant_operand=2)
    if allow_planes and out is None:
        return Planes(planes)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if out.is_contiguous():
        return sum_planes(planes, out)
    tmp = torch.empty((M, N), dtype=out.dtype, device=x.device)
    sum_planes(planes, tmp)
    out.copy_(tmp)
    return out


def gemm_bf16_silu_mul(x: torch.Tensor, w_pairs: torch.Tensor, out: torch.Tensor,
                       then_reads: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, I] = silu(x @ gate^T) * (x @ up^T) with `w_pairs` [2I, K] holding
    gate i in row 2i and up i in row 2i+1; the activation runs in the product's
    epilogue, so the [M, 2I] intermediate never reaches memory."""
    M, K = x.shape
    two_i = w_pairs.shape[0]
    if out.shape != (M, two_i // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise KernelError("gemm_bf16_silu_mul: out must be [M, I] bfloat16 with contiguous rows")
    if M == 0:
        return out
    usable = _tc_usable(x.values if isinstance(x, RowScaled) else x, w_pairs, out)
    if usable and rows_usable(x, w_pairs):
        return gemm_rows(x, w_pairs, out, silu_mul=True)
    if not usable:
        x = plain(x)
        tmp = torch.empty((M, two_i), dtype=torch.bfloat16, device=x.device)
        gemm_simt(x, w_pairs, tmp)
        return silu_mul(tmp, out, interleaved=True)
    if M <= SKINNY_ROWS:
        return gemm_skinny(x, w_pairs, out, epilogue=1, then_reads=then_reads,
                           warps=skinny_plan(two_i, K, False)[1])
    if M > 128:
        bn, form = prompt_plan(M, two_i)
        gemm_tc(x, w_pairs, out, out.stride(0), 1, bn, epilogue=1, constant_operand=2,
                persistent=form)
    else:
        gemm_tc(x, w_pairs, out, out.stride(0), 1, 128, epilogue=1, constant_operand=2)
    return out


FAST_HEAD_DIMS = (16, 32, 64, 128)  # head sizes of the tensor-core attention kernels


def attention(ctx, q: torch.Tensor, out: torch.Tensor, page_table: torch.Tensor,
              k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int, num_kv_heads: int,
              head_dim: int, scale: float, window: int = 0, ring_pages: int = 0,
              then_reads: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a step's tokens over the cache: the kernel that fits the
    element type and the step. bfloat16 with a built head size runs on the
    tensor cores (one kernel for single-token steps, one for prompts); float32,
    windows and other head sizes run on the CUDA cores."""
    fast = (q.dtype == torch.bfloat16 and head_dim in FAST_HEAD_DIMS and window == 0
            and ring_pages == 0 and num_heads // num_kv_heads <= 16)
    if not fast:
        return attention_simt(q, out, ctx.positions, ctx.seq_of_token, page_table, k_cache,
                              v_cache, num_heads, num_kv_heads, head_dim, scale, window, ring_pages)
    if ctx.is_decode:
        pairs, pages = ctx.n_seqs * num_kv_heads, (ctx.max_kv_len + PAGE - 1) // PAGE
        splits, stages = decode_plan(pairs, pages, head_dim,
                                     getattr(ctx, "unequal_lengths", False))
        return attention_decode(q, out, ctx.cu_tokens, ctx.kv_lens, page_table, k_cache, v_cache,
                                num_heads, num_kv_heads, head_dim, scale, splits, stages,
                                then_reads=then_reads)
    if ctx.cu_tokens_host is None:
        # a step replayed from a graph: the grid comes from the bucket's bound of
        # 64-row blocks (blocks beyond the real count return at once)
        blocks, blocks128, longest = (ctx.query_blocks_bound, (ctx.query_blocks_bound + 1) // 2
                                      + ctx.n_seqs, 64 if ctx.long_queries else 1)
    else:
        lens = [ctx.cu_tokens_host[i + 1] - ctx.cu_tokens_host[i] for i in range(ctx.n_seqs)]
        blocks, blocks128, longest = (sum((n + 63) // 64 for n in lens),
                                      sum((n + 127) // 128 for n in lens), max(lens))
    if head_dim in TC_HEAD_DIMS and PREFILL_TC and longest >= 64 and _tc_attention_ok(q, out):
        return attention_prefill_tc(q, out, ctx.cu_tokens, ctx.kv_lens, page_table, k_cache,
                                    v_cache, num_heads, num_kv_heads, head_dim, scale, blocks128)
    return attention_prefill(q, out, ctx.cu_tokens, ctx.kv_lens, page_table, k_cache, v_cache,
                             num_heads, num_kv_heads, head_dim, scale, blocks)


# Seconds a warp of the decode kernel takes for its 16 keys of a page (a chain of
# dependent instructions, whatever the head size or the load of the GPU), and the
# bytes a second that the cache streams at when enough CTAs ask: with these two a
# plan can tell whether a CTA that walks a whole sequence alone keeps up with memory.
DECODE_PAGE_SECONDS = 0.63e-6
DECODE_STREAM_BYTES_PER_SECOND = 6.5e12


def decode_plan(pairs: int, pages: int, head_dim: int = 128, unequal: bool = False):
    """(splits, page buffers) of decode attention for `pairs` (sequence, kv head)
    pairs of up to `pages` cache pages. Three page buffers per CTA (two pages on
    their way while one is multiplied); 2 CTAs of head size 128 fit an SM, 4 of
    64 or less. Ranges are split while all CTAs stay resident at once (a second
    round of CTAs costs more than it gains), at most eightfold (one cluster).
    Sequences of equal lengths are not split at all once their pairs are many
    enough for memory to be the limit: a CTA walks a page in DECODE_PAGE_SECONDS,
    so `pairs` CTAs ask for pairs * page bytes in that time, and where that
    exceeds what memory delivers, more CTAs only add merges. With unequal lengths
    the longest sequence's CTA is what the batch waits for, and ranges are split
    as far as residency allows. A long context with few pairs takes several
    clusters, whose results meet in the workspace."""
    resident = sm_count() * min(4, 256 // max(head_dim, 1))
    room = resident // max(pairs, 1)
    if room >= 16 and pages >= 160:
        # clusters of 8 while a CTA keeps 4 pages or more; the second merge pays
        # from about 10 K tokens on
        return min(room // 8 * 8, max(16, pages // 4 // 8 * 8)), 3
    page_bytes = 2 * PAGE * head_dim * 2  # keys and values of one kv head
    if not unequal and pairs * page_bytes >= DECODE_PAGE_SECONDS * DECODE_STREAM_BYTES_PER_SECOND:
        return 1, 3
    splits = max(1, min(DECODE_CLUSTER_MAX, pages, room))
    return 1 << (splits.bit_length() - 1), 3  # clusters of 3, 5, 6 or 7 were slower than the power of two below


TC_HEAD_DIMS = (64, 128)  # head sizes of the tcgen05 prompt-attention kernel
PREFILL_TC = _os.environ.get("FOUNDRY_B200_PREFILL_TC", "1") != "0"


def _tc_attention_ok(q: torch.Tensor, out: torch.Tensor) -> bool:
    return (q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0 and q.stride(1) == 1 and out.stride(1) == 1)


def attention_prefill_tc(q, out, cu_tokens, kv_lens, page_table, k_cache, v_cache, num_heads,
                         num_kv_heads, head_dim, scale, q_blocks) -> torch.Tensor:
    """Prompt attention on tcgen05 (csrc/attention_tcgen05.cu); `q_blocks` is the
    sum over sequences of ceil(tokens / 128)."""
    _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
    _call("fb_attention_prefill_tc", _dev(q, "q", torch.bfloat16, contiguous=False), _rows(q, "q"),
          q.shape[0], _dev(out, "out", torch.bfloat16, contiguous=False), _rows(out, "out"),
          _dev(cu_tokens, "cu_tokens", torch.int32), _dev(kv_lens, "kv_lens", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1], k_cache.data_ptr(),
          v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), k_cache.shape[0],
          kv_lens.numel(), q_blocks, num_heads, num_kv_heads, head_dim, float(scale), _stream())
    return out


def attention_prefill(q, out, cu_tokens, kv_lens, page_table, k_cache, v_cache, num_heads,
                      num_kv_heads, head_dim, scale, q_blocks) -> torch.Tensor:
    """Tensor-core attention for steps of any token counts; `q_blocks` is the
    sum over sequences of ceil(tokens / 64)."""
    _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
    _call("fb_attention_prefill", _dev(q, "q", torch.bfloat16, contiguous=False), _rows(q, "q"),
          _dev(out, "out", torch.bfloat16, contiguous=False), _rows(out, "out"),
          _dev(cu_tokens, "cu_tokens", torch.int32), _dev(kv_lens, "kv_lens", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1], k_cache.data_ptr(),
          v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), kv_lens.numel(), q_blocks,
          num_heads, num_kv_heads, head_dim, float(scale), _stream())
    return out


# Up to this many CTAs of a (sequence, kv head) merge their partial results
# through distributed shared memory; more go through a workspace in global memory.
DECODE_CLUSTER_MAX = 8
DECODE_CLUSTER = _os.environ.get("FOUNDRY_B200_DECODE_CLUSTER", "1") != "0"


def attention_decode(q, out, cu_tokens, kv_lens, page_table, k_cache, v_cache, num_heads,
                     num_kv_heads, head_dim, scale, splits, stages: int = 3,
                     then_reads: Optional[torch.Tensor] = None,
                     cluster: Optional[int] = None) -> torch.Tensor:
    """Tensor-core attention for one token per sequence, the cache range split
    over `splits` CTAs per (sequence, kv head). `cluster` of them (by default as
    many as divide `splits`, up to 8) form a thread-block cluster and merge their
    partial results through each other's shared memory; the clusters' results
    (or, without clusters, every CTA's) go to a workspace, and the CTA that
    finishes a pair last merges them. `then_reads`: weights to ask into L2 for
    the kernel that follows (see `gemm_skinny`)."""
    _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, torch.bfloat16)
    n = kv_lens.numel()
    if cluster is None:
        cluster = 1
        if DECODE_CLUSTER:
            cluster = max(c for c in range(1, DECODE_CLUSTER_MAX + 1) if splits % c == 0)
    parts = splits // max(cluster, 1)
    ws_o = ws_ml = counters = None
    if parts > 1:
        ws_o = torch.empty(n * num_kv_heads * parts * 16 * head_dim, dtype=torch.float32,
                           device=q.device)
        ws_ml = torch.empty(n * num_kv_heads * parts * 32, dtype=torch.float32, device=q.device)
        counters = _arrival_counters(q.device, n * num_kv_heads)
    _call("fb_attention_decode", _dev(q, "q", torch.bfloat16, contiguous=False), _rows(q, "q"),
          _dev(out, "out", torch.bfloat16, contiguous=False), _rows(out, "out"),
          _dev(cu_tokens, "cu_tokens", torch.int32), _dev(kv_lens, "kv_lens", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1], k_cache.data_ptr(),
          v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), n, num_heads, num_kv_heads,
          head_dim, float(scale), splits, stages, cluster,
          0 if ws_o is None else ws_o.data_ptr(), 0 if ws_ml is None else ws_ml.data_ptr(),
          0 if counters is None else counters.data_ptr(), *_prefetch_range(then_reads),
          1 if n > SKINNY_ROWS else 0,  # what follows is a tcgen05 product, not the streaming one
          _stream())
    return out


_COUNTERS = {}


def _arrival_counters(device, count: int) -> torch.Tensor:
    """Zeroed int32 counters shared by the decode-attention calls of a device and
    scratch owner: each call finds them zero and leaves them zero (an owner's
    calls follow one another on one stream)."""
    key = _scratch_key(device)
    held = _COUNTERS.get(key)
    if held is None or held.numel() < count:
        held = torch.zeros(max(65536, count), dtype=torch.int32, device=device)
        _COUNTERS[key] = held
    return held


def attention_simt(q: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                   scale: float, window: int = 0, ring_pages: int = 0) -> torch.Tensor:
    """Causal attention of every token over its sequence's cache rows [0, pos]
    (or the last `window` of them). `q` may be a strided view of the fused
    projection output; `out` is [T, heads * head_dim]."""
    T = q.shape[0]
    _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, q.dtype)
    if out.dtype != q.dtype or out.shape[0] != T:
        raise KernelError("attention: out does not match q")
    _call("fb_attention_simt", _dev(q, "q", contiguous=False), _rows(q, "q"),
          _dev(out, "out", contiguous=False), _rows(out, "out"), code_of(q.dtype),
          _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1], k_cache.data_ptr(),
          v_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), ring_pages, window, T,
          num_heads, num_kv_heads, head_dim, float(scale), _stream())
    return out


# ------------------------------------------------------------------- sampling
def select_tokens(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor],
                  streams: Optional[torch.Tensor] = None,
                  steps: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy where temperature is 0 (or None), Gumbel-max sampling elsewhere.
    `streams[r]` is the row's random stream (`sampling.stream_key(seed, key)`),
    `steps[r]` how many tokens its sequence has generated. Large vocabularies
    are scanned by several blocks per row and merged by a second small kernel."""
    n, V = logits.shape
    if out.numel() != n:
        raise KernelError("select_tokens: out does not hold one token per row")
    chunks = 1 if V < 16384 else min(64, (V + 2047) // 2048)
    part_val = part_idx = None
    if chunks > 1:
        part_val = torch.empty(n * chunks, dtype=torch.float32, device=logits.device)
        part_idx = torch.empty(n * chunks, dtype=torch.int32, device=logits.device)
        _COUNT[0] += 1  # the merge kernel
    _call("fb_select_tokens", _dev(logits, "logits", torch.float32, contiguous=False),
          _rows(logits, "logits"), n, V,
          0 if temperature is None else _dev(temperature, "temperature", torch.float32),
          0 if streams is None else _dev(streams, "streams", torch.int64),
          0 if steps is None else _dev(steps, "steps", torch.int64),
          _dev(out, "out", torch.int32), chunks,
          0 if part_val is None else part_val.data_ptr(),
          0 if part_idx is None else part_idx.data_ptr(), _stream())
    return out
