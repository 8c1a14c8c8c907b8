"""Each kernel alone against a plain float32 PyTorch statement of the same
operation, at sizes other than the engine's: widths and vocabularies that are
no power of two, head sizes in steps of 16, odd token counts, strided views,
padding rows."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from foundry_b200.kernels import ops as o
    return o


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(a, b, atol, rtol):
    a, b = a.double().cpu(), b.double().cpu()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"max err {float(err.max()):.3e}, worst excess " \
                                        f"{float((err - bound).max()):.3e}"


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    V, H = 391, 200
    table = rnd(V, H, dtype=dtype)
    ids = torch.tensor([0, 390, 17, 17, 5, 391, -1], dtype=torch.int32, device=DEV)
    out = torch.full((7, H), 9.0, device=DEV)
    ops.embed_gather(table, ids, out)
    want = table.float()[ids[:5].long()]
    assert torch.equal(out[:5], want)
    assert torch.equal(out[5:], torch.zeros(2, H, device=DEV))  # ids outside the table: zero rows


# ------------------------------------------------------------------- rms norm
@pytest.mark.parametrize("T,H", [(1, 64), (5, 96), (3, 3072), (2, 5000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(ops, T, H, dtype):
    resid = rnd(T, H, scale=2.0)
    delta = rnd(T, H, dtype=dtype, seed=1)
    w = 1.0 + 0.1 * rnd(H, seed=2)
    eps = 1e-5
    r0 = resid.clone()
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(resid, delta, w, eps, out)
    h = r0.double() + delta.double()
    want = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * w.double()
    close(resid, h, 1e-6, 1e-6)
    if dtype == torch.float32:
        close(out, want, 1e-5, 1e-5)
    else:
        close(out, want, 1e-2, 8e-3)
    # without a delta the residual is untouched; without an output only the sum is made
    r1 = resid.clone()
    ops.add_rmsnorm(resid, None, w, eps, out)
    assert torch.equal(resid, r1)
    ops.add_rmsnorm(resid, delta, w, eps, None)
    close(resid, r1.double() + delta.double(), 1e-6, 1e-6)


# ------------------------------------------------------------------- silu mul
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(ops, dtype):
    T, I = 7, 176
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.silu_mul(gu, out)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    want = g / (1 + torch.exp(-g)) * u
    close(out, want, 1e-6 if dtype == torch.float32 else 2e-2, 1e-6 if dtype == torch.float32 else 8e-3)


def test_gather_rows_and_cast(ops):
    src = rnd(9, 40)
    rows = torch.tensor([8, 0, 3, -1], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 40, device=DEV)
    ops.gather_rows(src, rows, out)
    assert torch.equal(out[:3], src[[8, 0, 3]]) and torch.equal(out[3], torch.zeros(40, device=DEV))
    b = torch.empty(9, 40, dtype=torch.bfloat16, device=DEV)
    ops.cast(src, b)
    assert torch.equal(b, src.bfloat16())  # round to nearest even, as torch does


# ---------------------------------------------------------------------- gemm
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 100, 72), (70, 130, 200), (33, 17, 9),
                                   (200, 384, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(ops, M, N, K, dtype):
    x, w = rnd(M, K, dtype=dtype), rnd(N, K, dtype=dtype, seed=3)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_simt(x, w, out)
    want = x.double() @ w.double().T
    close(out, want, 1e-4 * math.sqrt(K), 1e-5)
    # strided input rows and a strided output
    big = rnd(M, 2 * K, dtype=dtype, seed=4)
    wide = torch.zeros(M, N + 8, dtype=dtype, device=DEV)
    ops.gemm_simt(big[:, :K], w, wide[:, :N])
    close(wide[:, :N], big[:, :K].double() @ w.double().T,
          1e-4 * math.sqrt(K) if dtype == torch.float32 else 0.05 * math.sqrt(K), 1e-2)
    assert float(wide[:, N:].abs().max()) == 0.0


TC_SHAPES = [(1, 128, 64), (1, 3072, 3072), (8, 5120, 3072), (3, 200, 72), (16, 384, 96),
             (17, 130, 200), (64, 1000, 512), (65, 256, 128), (128, 96, 64), (129, 384, 96),
             (300, 520, 328), (2048, 1024, 256), (500, 3072, 8192), (40, 3072, 8192)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tensor_core(ops, M, N, K):
    """The dispatcher's choice (plain or swapped operands, tile width, split-K)
    against float64 products of the same bfloat16 inputs."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=5)
    want = x.double() @ w.double().T
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((M, N), 7.0, dtype=out_dtype, device=DEV)
        ops.gemm_bf16(x, w, out)
        if out_dtype == torch.float32:
            close(out, want, 2e-4 * math.sqrt(K), 1e-5)
        else:
            close(out, want, 2e-4 * math.sqrt(K) + 1e-2, 8e-3)
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("splits", [1, 3])
def test_gemm_tensor_core_every_tile_width(ops, bn, splits):
    """Both operand roles, every tile width, split-K planes, ragged edges in
    all three dimensions."""
    rows_a, rows_b, K = 200, bn + 5, 264
    a, b = rnd(rows_a, K, dtype=torch.bfloat16), rnd(rows_b, K, dtype=torch.bfloat16, seed=6)
    want = a.double() @ b.double().T
    planes = torch.full((splits, rows_a, rows_b), 3.0, device=DEV)
    ops.gemm_tc(a, b, planes, rows_b, 1, bn, splits, rows_a * rows_b)
    close(planes.sum(0), want, 3e-3, 1e-5)
    planes_t = torch.full((splits, rows_b, rows_a), 3.0, device=DEV)  # swapped output
    ops.gemm_tc(a, b, planes_t, 1, rows_a, bn, splits, rows_a * rows_b)
    close(planes_t.sum(0).T, want, 3e-3, 1e-5)
    assert ops.gemm_tc_status() == 0


def test_gemm_tensor_core_rows_do_not_mix(ops):
    """A row of x only meets its own row of the result: with one-hot rows the
    product returns single columns of W exactly."""
    N, K = 300, 128
    w = rnd(N, K, dtype=torch.bfloat16, seed=7)
    for M in (3, 150):
        x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
        cols = [(5 * i + 1) % K for i in range(M)]
        x[torch.arange(M), cols] = 1.0
        out = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops.gemm_bf16(x, w, out)
        assert torch.equal(out, w.float()[:, cols].T.contiguous())


def test_gemm_falls_back_for_shapes_tma_cannot_address(ops):
    x, w = rnd(4, 36, dtype=torch.bfloat16), rnd(20, 36, dtype=torch.bfloat16, seed=8)
    out = torch.empty(4, 20, dtype=torch.float32, device=DEV)
    ops.gemm_bf16(x, w, out)  # K = 36 is no multiple of 8
    close(out, x.double() @ w.double().T, 1e-3, 1e-5)
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_tc(x, w, out, 20, 1, 16)
