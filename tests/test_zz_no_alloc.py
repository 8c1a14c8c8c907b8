"""The entry point that allocates nothing, called through its exported C
symbol, against the ordinary decode attention.

Some callers of the kernels cannot request device memory when they call: all
memory already belongs to their own arena, or they run where the CUDA
allocator must not be entered. For them the library keeps the scratch of
split-KV decode attention in a fixed device array of its own
(`csrc/attention_static.h`). This test calls `fb_attention_decode_static`
several times in a row with different shapes, so that each call meets the
leftovers of the one before in the shared array, and checks every result
against a float64 attention computed on the CPU and against
`fb_attention_decode` with a workspace from torch; the device's free memory
(which counts every allocation, the library's own too) must not move across a
call. It runs last, and passes alone in a fresh process as well as after
every other test.
"""
import ctypes
import gc
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 2 * 1024 * 1024  # FB_ATTENTION_STATIC_SCRATCH_FLOATS


def _case(n_seqs, lens, A, Kh, D, seed):
    """Random queries and a paged cache with scattered pages."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [(n + 63) // 64 for n in lens]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g)
    table = torch.zeros(n_seqs, max(pages_per), dtype=torch.int32)
    at = 0
    for i, n in enumerate(pages_per):
        table[i, :n] = perm[at:at + n].int()
        at += n
    store = torch.randn(total, 2, Kh, 64, D, generator=g).bfloat16().to(DEV)
    q = torch.randn(n_seqs, A * D, generator=g).bfloat16().to(DEV)
    cu = torch.arange(n_seqs + 1, dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return q, cu, kv, table.to(DEV), store[:, 0], store[:, 1]


def _call_static(lib, q, out, cu, kv, table, k, v, A, Kh, D, splits):
    fn = lib.fb_attention_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                   ctypes.c_int, ctypes.c_void_p]
    return fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), cu.data_ptr(),
              kv.data_ptr(), table.data_ptr(), table.shape[1], k.data_ptr(), v.data_ptr(),
              k.stride(0), k.stride(1), kv.numel(), A, Kh, D, 1.0 / math.sqrt(D), splits,
              torch.cuda.current_stream().cuda_stream)


def _plain_attention(q, kv, table, k, v, A, Kh, D):
    """Float64 attention of one query per sequence over its paged keys and
    values, computed on the CPU; a sequence of length 0 gives zeros."""
    q, k, v, table = q.double().cpu(), k.double().cpu(), v.double().cpu(), table.cpu()
    out = torch.zeros(q.shape[0], A, D, dtype=torch.float64)
    for i, n in enumerate(kv.tolist()):
        if n == 0:
            continue
        pages = table[i, :(n + 63) // 64].long()
        keys = k[pages].permute(1, 0, 2, 3).reshape(Kh, -1, D)[:, :n]
        values = v[pages].permute(1, 0, 2, 3).reshape(Kh, -1, D)[:, :n]
        for a in range(A):
            scores = keys[a // (A // Kh)] @ q[i].view(A, D)[a] / math.sqrt(D)
            out[i, a] = torch.softmax(scores, 0) @ values[a // (A // Kh)]
    return out.reshape(q.shape[0], A * D)


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from foundry_b200.kernels import library, ops
    lib = library.load()
    lib.fb_last_error.restype = ctypes.c_char_p
    # Calls in a row on the shared array, of other shapes and head sizes each time:
    # the second has a row without keys and more ranges than its short sequences
    # have pages (ranges that stay empty still have to arrive at the counters and
    # leave them zero for the third).
    cases = ((5, [700, 64, 1, 333, 129], 12, 4, 128, 6, 0),
             (4, [90, 0, 200, 65], 4, 2, 32, 5, 1),
             (3, [130, 64, 300], 8, 2, 64, 3, 2))
    for n_seqs, lens, A, Kh, D, splits, seed in cases:
        q, cu, kv, table, k, v = _case(n_seqs, lens, A, Kh, D, seed)
        want = torch.zeros_like(q)
        # the ordinary entry point with a workspace from torch, merging through the
        # workspace as the static one does (cluster 1): the same sums in the same order
        ops.attention_decode(q, want, cu, kv, table, k, v, A, Kh, D, 1.0 / math.sqrt(D), splits,
                             cluster=1)
        # A first call loads this head size's kernel and (the very first) looks the
        # array's address up; the device's free memory is compared around a second one.
        warm = torch.full_like(q, 7.0)
        rc = _call_static(lib, q, warm, cu, kv, table, k, v, A, Kh, D, splits)
        assert rc == 0, lib.fb_last_error().decode()
        got = torch.full_like(q, 7.0)
        gc.collect()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        rc = _call_static(lib, q, got, cu, kv, table, k, v, A, Kh, D, splits)
        assert rc == 0, lib.fb_last_error().decode()
        torch.cuda.synchronize()
        # cudaMemGetInfo sees every allocation on the device, the library's own included
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == torch_before
        plain = _plain_attention(q, kv, table, k, v, A, Kh, D)
        for result in (warm, got):
            err = (result.double().cpu() - plain).abs()
            bound = 3e-2 + 1e-2 * plain.abs()  # the tolerance of the attention kernel tests
            assert bool((err <= bound).all()), float(err.max())
        assert torch.equal(got, want) and torch.equal(warm, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from foundry_b200.kernels import library
    lib = library.load()
    lib.fb_last_error.restype = ctypes.c_char_p
    q, cu, kv, table, k, v = _case(2, [100, 100], 8, 8, 128, 2)
    out = torch.zeros_like(q)
    splits = SCRATCH_FLOATS // (2 * 8 * (16 * 128 + 32)) + 1
    rc = _call_static(lib, q, out, cu, kv, table, k, v, 8, 8, 128, splits)
    assert rc != 0
    message = lib.fb_last_error().decode()
    assert "scratch" in message and str(SCRATCH_FLOATS) in message
    assert float(out.abs().max()) == 0.0  # nothing ran
