"""Python faces of the CUDA launchers: torch tensors in, checked, pointers out.

Each function checks device, dtype, contiguity and the sizes the kernel
assumes, then calls the `extern "C"` launcher on the current CUDA stream.
Nothing here computes: a tensor that is not on a CUDA device is an error, not
a reason to compute elsewhere.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page; equals FB_PAGE in csrc/common.cuh

_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_ll, c_float, c_ull = (ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                                         ctypes.c_float, ctypes.c_ulonglong)

_SIGNATURES = {
    "fb_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "fb_add_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int,
                       c_int, c_void_p],
    "fb_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "fb_gather_rows": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "fb_cast": [c_void_p, c_int, c_void_p, c_int, c_ll, c_void_p],
    "fb_rope_kv_write": [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                         c_int, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_void_p],
    "fb_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int,
                     c_int, c_void_p],
    "fb_attention_simt": [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p,
                          c_int, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_float, c_void_p],
    "fb_select_tokens": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p],
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


def launch_count() -> int:
    """Kernels of this library launched so far (graph replays included)."""
    return _COUNT[0]


def add_launches(n: int) -> None:
    _COUNT[0] += n


add_graph_launches = add_launches


def _call(name: str, *args) -> None:
    _COUNT[0] += 1
    code = _fn(name)(*args)
    if code != 0:
        message = library.load().fb_last_error().decode(errors="replace")
        raise KernelError(f"{name}: {message}")


def _stream() -> int:
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
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """resid += delta (when given), in place, float32; out = rmsnorm(resid) * weight.
    With `out=None` only the sum is made."""
    T, H = resid.shape
    if delta is not None and delta.shape != resid.shape:
        raise KernelError(f"add_rmsnorm: delta is {tuple(delta.shape)}, resid {tuple(resid.shape)}")
    if out is not None and out.shape != resid.shape:
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, resid {tuple(resid.shape)}")
    if weight.shape != (H,):
        raise KernelError(f"add_rmsnorm: weight is {tuple(weight.shape)}, expected {(H,)}")
    _call("fb_add_rmsnorm", _dev(resid, "resid", torch.float32),
          0 if delta is None else _dev(delta, "delta"),
          F32 if delta is None else code_of(delta.dtype),
          _dev(weight, "weight", torch.float32), float(eps),
          0 if out is None else _dev(out, "out"),
          F32 if out is None else code_of(out.dtype), T, H, _stream())
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t,i] = silu(gate_up[t,i]) * gate_up[t,I+i]."""
    T, two_i = gate_up.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} / out {tuple(out.shape)}")
    _call("fb_silu_mul", _dev(gate_up, "gate_up"), _dev(out, "out"), code_of(out.dtype), T,
          two_i // 2, _stream())
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
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int, ring_pages: int = 0,
                  write_cache: bool = True) -> None:
    """Rotate the query heads of `qkv` in place; rotate the key heads into the
    cache pages and copy the value heads there. `k_cache`/`v_cache` are one
    cache entry's views [pages, kv_heads, PAGE, head_dim]."""
    T = qkv.shape[0]
    stride = _rows(qkv, "qkv")
    if positions.numel() != T or seq_of_token.numel() != T:
        raise KernelError("rope_kv_write: positions / seq_of_token do not cover the tokens")
    if inv_freq.numel() * 2 != rotary_dim:
        raise KernelError("rope_kv_write: inv_freq does not hold rotary_dim / 2 entries")
    page_stride = head_stride = 0
    kp = vp = 0
    if write_cache:
        _check_cache_views(k_cache, v_cache, num_kv_heads, head_dim, qkv.dtype)
        page_stride, head_stride = k_cache.stride(0), k_cache.stride(1)
        kp, vp = k_cache.data_ptr(), v_cache.data_ptr()
    _call("fb_rope_kv_write", _dev(qkv, "qkv", contiguous=False), code_of(qkv.dtype), stride,
          _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
          _dev(page_table, "page_table", torch.int32), page_table.shape[1],
          _dev(inv_freq, "inv_freq", torch.float32), rotary_dim, kp, vp, page_stride, head_stride,
          ring_pages, T, num_heads, num_kv_heads, head_dim, 1 if write_cache else 0, _stream())


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
          _rows(out, "out"), code_of(x.dtype), code_of(out.dtype), _stream())
    return out


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """bfloat16 product with 32-bit accumulation: the kernel that fits the shape."""
    return gemm_simt(x, w, out)


# ------------------------------------------------------------------ attention
def attention(ctx, q: torch.Tensor, out: torch.Tensor, page_table: torch.Tensor,
              k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int, num_kv_heads: int,
              head_dim: int, scale: float, window: int = 0, ring_pages: int = 0) -> torch.Tensor:
    """Attention of a step's tokens over the cache: the kernel that fits the
    element type and the step (prompts or single tokens)."""
    return attention_simt(q, out, ctx.positions, ctx.seq_of_token, page_table, k_cache, v_cache,
                          num_heads, num_kv_heads, head_dim, scale, window, ring_pages)


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
    `steps[r]` how many tokens its sequence has generated."""
    n, V = logits.shape
    if out.numel() != n:
        raise KernelError("select_tokens: out does not hold one token per row")
    _call("fb_select_tokens", _dev(logits, "logits", torch.float32, contiguous=False),
          _rows(logits, "logits"), n, V,
          0 if temperature is None else _dev(temperature, "temperature", torch.float32),
          0 if streams is None else _dev(streams, "streams", torch.int64),
          0 if steps is None else _dev(steps, "steps", torch.int64),
          _dev(out, "out", torch.int32), _stream())
    return out
