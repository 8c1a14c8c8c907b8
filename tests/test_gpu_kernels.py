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


# ------------------------------------------------------------------ attention
def make_paged_case(lens_q, lens_kv, A, Kh, D, dtype, seed=0, sharp=False):
    """Random q and a paged cache whose pages are scattered and shared by no
    two sequences. Returns everything the kernels take plus dense K, V."""
    g = torch.Generator().manual_seed(seed)
    n = len(lens_q)
    T = sum(lens_q)
    pages_per = [(kv + 63) // 64 for kv in lens_kv]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    width = max(pages_per)
    table = torch.zeros(n, width, dtype=torch.int32)
    store = torch.randn(total_pages, 2, Kh, 64, D, generator=g)  # unused rows hold noise
    dense_k, dense_v = [], []
    at = 0
    for i in range(n):
        mine = perm[at:at + pages_per[i]]
        at += pages_per[i]
        table[i, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
        k = torch.randn(lens_kv[i], Kh, D, generator=g)
        v = torch.randn(lens_kv[i], Kh, D, generator=g)
        if sharp:  # one far key per sequence stands out for every head
            k[lens_kv[i] // 3] *= 6.0
        for j in range(lens_kv[i]):
            store[mine[j // 64], 0, :, j % 64] = k[j]
            store[mine[j // 64], 1, :, j % 64] = v[j]
        dense_k.append(k)
        dense_v.append(v)
    q = torch.randn(T, A * D, generator=g)
    cu = [0]
    for x in lens_q:
        cu.append(cu[-1] + x)
    positions = torch.cat([torch.arange(kv - ql, kv) for ql, kv in zip(lens_q, lens_kv)])
    seq_of = torch.cat([torch.full((ql,), i) for i, ql in enumerate(lens_q)])
    store = store.to(dtype).to(DEV)
    case = dict(q=q.to(dtype).to(DEV), table=table.to(DEV), k=store[:, 0], v=store[:, 1],
                cu=torch.tensor(cu, dtype=torch.int32, device=DEV),
                kv=torch.tensor(lens_kv, dtype=torch.int32, device=DEV),
                positions=positions.int().to(DEV), seq_of=seq_of.int().to(DEV), cu_host=cu)
    # plain attention on the rounded inputs
    want = torch.zeros(T, A * D, dtype=torch.float64)
    G = A // Kh
    qd = case["q"].double().cpu().view(T, A, D)
    for i in range(n):
        k = dense_k[i].to(dtype).double()
        v = dense_v[i].to(dtype).double()
        for r in range(lens_q[i]):
            tok, pos = cu[i] + r, lens_kv[i] - lens_q[i] + r
            for a in range(A):
                s = (k[:pos + 1, a // G] @ qd[tok, a]) / math.sqrt(D)
                p = torch.softmax(s, 0)
                want[tok, a * D:(a + 1) * D] = p @ v[:pos + 1, a // G]
    return case, want


ATT_CASES = [  # (q lengths, kv lengths, heads, kv heads, head_dim)
    ([1, 1, 1], [1, 64, 65], 4, 2, 16),
    ([1, 1, 1, 1], [200, 3, 128, 129], 6, 2, 32),
    ([1, 1], [500, 77], 8, 8, 64),
    ([1, 1, 1], [300, 64, 1000], 12, 4, 128),
    ([1, 1, 1], [90, 10, 260], 16, 2, 64),  # 8 query heads per kv head: the narrow form's most
    ([1, 1], [150, 70], 12, 1, 32),  # 12 per kv head: the 16-row form
    ([1, 1], [33, 190], 5, 1, 16),
    ([5, 70, 1], [5, 70, 130], 4, 2, 16),
    ([64, 65, 3], [64, 65, 200], 6, 3, 32),
    ([130, 20], [130, 220], 4, 1, 64),
    ([100, 7, 129], [100, 300, 129], 6, 2, 128),
]


@pytest.mark.parametrize("lens_q,lens_kv,A,Kh,D", ATT_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_cuda_cores(ops, lens_q, lens_kv, A, Kh, D, dtype):
    case, want = make_paged_case(lens_q, lens_kv, A, Kh, D, dtype, sharp=True)
    out = torch.full_like(case["q"], 5.0)
    ops.attention_simt(case["q"], out, case["positions"], case["seq_of"], case["table"], case["k"],
                       case["v"], A, Kh, D, 1.0 / math.sqrt(D))
    close(out, want, 2e-5 if dtype == torch.float32 else 3e-2, 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("lens_q,lens_kv,A,Kh,D", ATT_CASES)
def test_attention_tensor_cores_any_token_counts(ops, lens_q, lens_kv, A, Kh, D):
    case, want = make_paged_case(lens_q, lens_kv, A, Kh, D, torch.bfloat16, seed=1, sharp=True)
    out = torch.full_like(case["q"], 5.0)
    blocks = sum((x + 63) // 64 for x in lens_q)
    ops.attention_prefill(case["q"], out, case["cu"], case["kv"], case["table"], case["k"],
                          case["v"], A, Kh, D, 1.0 / math.sqrt(D), blocks + 2)
    close(out, want, 3e-2, 1e-2)


TC_ATT_CASES = [c for c in ATT_CASES if c[4] in (64, 128)] + [
    ([128, 129, 1], [128, 129, 400], 4, 2, 64),
    ([700, 64], [700, 1000], 6, 2, 128),
    ([256], [2000], 2, 1, 128),
]


@pytest.mark.parametrize("lens_q,lens_kv,A,Kh,D", TC_ATT_CASES)
def test_attention_tcgen05_any_token_counts(ops, lens_q, lens_kv, A, Kh, D):
    """The tcgen05 prompt kernel: whole prompts, continued prompts (keys before
    the first query), blocks of exactly and just over 128 rows, single tokens far
    into a sequence, a far key that stands out; q read as a strided view."""
    case, want = make_paged_case(lens_q, lens_kv, A, Kh, D, torch.bfloat16, seed=4, sharp=True)
    T = sum(lens_q)
    wide = torch.zeros(T, A * D + 2 * 8 * D, dtype=torch.bfloat16, device=DEV)
    wide[:, :A * D] = case["q"]
    out = torch.full_like(case["q"], 5.0)
    blocks = sum((x + 127) // 128 for x in lens_q)
    ops.attention_prefill_tc(wide[:, :A * D], out, case["cu"], case["kv"], case["table"], case["k"],
                             case["v"], A, Kh, D, 1.0 / math.sqrt(D), blocks + 1)
    assert ops.gemm_tc_status() == 0
    close(out, want, 3e-2, 1e-2)


@pytest.mark.parametrize("lens_q,lens_kv,A,Kh,D", [c for c in ATT_CASES if max(c[0]) == 1])
@pytest.mark.parametrize("splits,cluster", [(1, None), (2, None), (7, None), (7, 1), (12, None),
                                            (12, 4), (16, None), (24, 8)])
def test_attention_tensor_cores_single_tokens(ops, lens_q, lens_kv, A, Kh, D, splits, cluster):
    """Ranges merged in one cluster, through the workspace alone (cluster 1), and
    in several clusters whose results meet in the workspace."""
    # a padding row (length 0) sits between the real ones and must come out as zeros
    lens_q, lens_kv = list(lens_q), list(lens_kv)
    case, want = make_paged_case(lens_q, lens_kv, A, Kh, D, torch.bfloat16, seed=2, sharp=True)
    kv = torch.cat([case["kv"], torch.zeros(1, dtype=torch.int32, device=DEV)])
    cu = torch.cat([case["cu"], case["cu"][-1:] + 1])
    q = torch.cat([case["q"], rnd(1, A * D, dtype=torch.bfloat16)])
    table = torch.cat([case["table"], torch.zeros_like(case["table"][:1])])
    for stages in (2, 3):
        out = torch.full_like(q, 5.0)
        ops.attention_decode(q, out, cu, kv, table, case["k"], case["v"], A, Kh, D,
                             1.0 / math.sqrt(D), splits, stages, cluster=cluster)
        close(out[:-1], want, 3e-2, 1e-2)
        assert float(out[-1].abs().max()) == 0.0


@pytest.mark.parametrize("lens_kv,A,Kh,D", [([1000, 3, 64, 300, 129, 1], 12, 4, 128),
                                            ([70, 2000, 500, 65], 16, 2, 64), ([33, 190, 900], 6, 3, 32)])
@pytest.mark.parametrize("splits", [2, 4, 8])
def test_attention_single_tokens_of_unequal_lengths(ops, lens_kv, A, Kh, D, splits):
    """Every sequence's own pages cut into ranges: the short ones leave CTAs without
    a range (one page, eight ranges); merged through the workspace and in clusters."""
    lens_q = [1] * len(lens_kv)
    case, want = make_paged_case(lens_q, lens_kv, A, Kh, D, torch.bfloat16, seed=6, sharp=True)
    for cluster in (1, 1, None):  # the counters are back at zero for the second call
        out = torch.full_like(case["q"], 5.0)
        ops.attention_decode(case["q"], out, case["cu"], case["kv"], case["table"], case["k"],
                             case["v"], A, Kh, D, 1.0 / math.sqrt(D), splits, 3, cluster=cluster)
        close(out, want, 3e-2, 1e-2)


def test_attention_picks_out_a_far_key(ops):
    """One key among a thousand matches the query; the output must be that
    key's value, whichever kernel runs."""
    A, Kh, D, L = 4, 2, 64, 1000
    case, _ = make_paged_case([1], [L], A, Kh, D, torch.bfloat16, seed=3)
    k, v, table = case["k"], case["v"], case["table"]
    k.zero_()
    target = 137
    page, row = int(table[0, target // 64]), target % 64
    q = torch.zeros(1, A * D, dtype=torch.bfloat16, device=DEV)
    q[:, ::D] = 8.0  # first element of every head
    k[page, :, row, 0] = 8.0
    want = v[page, :, row].float().repeat_interleave(A // Kh, 0).reshape(1, A * D)
    for run in ("simt", "decode", "prefill"):
        out = torch.zeros_like(q)
        if run == "simt":
            ops.attention_simt(q, out, case["positions"], case["seq_of"], table, k, v, A, Kh, D, 1.0)
        elif run == "decode":
            ops.attention_decode(q, out, case["cu"], case["kv"], table, k, v, A, Kh, D, 1.0, 5)
        else:
            ops.attention_prefill(q, out, case["cu"], case["kv"], table, k, v, A, Kh, D, 1.0, 1)
        close(out, want, 2e-2, 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,L,queries", [(100, 500, 93), (64, 130, 1), (70, 70, 70), (33, 400, 5)])
def test_attention_cuda_cores_window_and_ring(ops, dtype, window, L, queries):
    """A windowed layer group: the sequence's pages are a ring of
    ceil(window / 64) + 1 in which position p lies in page (p / 64) % ring, and a
    query at p reads the keys (p - window, p]. The ring is filled as L
    single-token steps would leave it; the last `queries` tokens ask. For the
    last query the key just outside the window and the key just inside it both
    match the query far better than any other: the first must not count, the
    second must."""
    A, Kh, D = 4, 2, 32
    ring = (window + 63) // 64 + 1
    assert queries <= ring * 64 - window + 1  # what one step may bring
    g = torch.Generator().manual_seed(window)
    k = torch.randn(L, Kh, D, generator=g)
    v = torch.randn(L, Kh, D, generator=g)
    q = torch.randn(queries, A, D, generator=g)
    p_last = L - 1
    if p_last - window >= 0:
        q[-1] = 0.0
        q[-1, :, 0] = 6.0
        k[p_last - window, :, 0] = 9.0      # just outside
        k[p_last - window + 1, :, 0] = 8.0  # just inside
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    pages = [5, 2, 7, 1, 4][:ring]
    store = torch.randn(8, 2, Kh, 64, D, generator=g).to(dtype)
    for pos in range(L):  # later positions overwrite the ring's rows
        store[pages[(pos // 64) % ring], 0, :, pos % 64] = k[pos]
        store[pages[(pos // 64) % ring], 1, :, pos % 64] = v[pos]
    store = store.to(DEV)
    table = torch.tensor([pages], dtype=torch.int32, device=DEV)
    positions = torch.arange(L - queries, L, dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(queries, dtype=torch.int32, device=DEV)
    out = torch.full((queries, A * D), 5.0, dtype=dtype, device=DEV)
    ops.attention_simt(q.reshape(queries, A * D).to(DEV), out, positions, seq_of, table,
                       store[:, 0], store[:, 1], A, Kh, D, 1.0 / math.sqrt(D), window=window,
                       ring_pages=ring)
    want = torch.zeros(queries, A, D, dtype=torch.float64)
    kd, vd, qd = k.double(), v.double(), q.double()
    for r in range(queries):
        pos = L - queries + r
        lo = max(0, pos - window + 1)
        for a in range(A):
            s_ = (kd[lo:pos + 1, a // (A // Kh)] @ qd[r, a]) / math.sqrt(D)
            want[r, a] = torch.softmax(s_, 0) @ vd[lo:pos + 1, a // (A // Kh)]
    close(out, want.reshape(queries, A * D), 2e-5 if dtype == torch.float32 else 3e-2,
          1e-5 if dtype == torch.float32 else 1e-2)


def test_attention_refuses_sizes_it_does_not_build(ops):
    case, _ = make_paged_case([1], [10], 4, 2, 48, torch.bfloat16)
    out = torch.zeros_like(case["q"])
    with pytest.raises(ops.KernelError, match="head size 48"):
        ops.attention_decode(case["q"], out, case["cu"], case["kv"], case["table"], case["k"],
                             case["v"], 4, 2, 48, 1.0, 1)
    # the dispatcher serves the same size on the CUDA cores
    ops.attention_simt(case["q"], out, case["positions"], case["seq_of"], case["table"], case["k"],
                       case["v"], 4, 2, 48, 1.0 / math.sqrt(48))
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        bad, _ = make_paged_case([1], [10], 2, 2, 24, torch.bfloat16)
        ops.attention_simt(bad["q"], torch.zeros_like(bad["q"]), bad["positions"], bad["seq_of"],
                           bad["table"], bad["k"], bad["v"], 2, 2, 24, 1.0)


# ---------------------------------------------------- fused consumers of planes
def test_add_rmsnorm_sums_split_planes(ops):
    T, H, S = 5, 96, 3
    planes = rnd(S, T, H)
    resid, w = rnd(T, H, seed=1), 1.0 + 0.1 * rnd(H, seed=2)
    r0 = resid.clone()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(resid, ops.Planes(planes), w, 1e-5, out)
    h = r0.double() + planes.double().sum(0)
    close(resid, h, 1e-5, 1e-6)
    close(out, h / torch.sqrt((h * h).mean(-1, keepdim=True) + 1e-5) * w.double(), 2e-2, 8e-3)


def test_silu_mul_interleaved(ops):
    T, I = 5, 88
    gu = rnd(T, 2 * I, dtype=torch.bfloat16, scale=2.0)
    out = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(gu, out, interleaved=True)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    close(out, g / (1 + torch.exp(-g)) * u, 2e-2, 8e-3)


@pytest.mark.parametrize("M", [1, 8, 33, 64, 100, 129, 300])
def test_gemm_with_silu_mul_epilogue(ops, M):
    K, I = 200, 152  # neither a multiple of the tile sizes
    x = rnd(M, K, dtype=torch.bfloat16, scale=0.5)
    gate, up = rnd(I, K, dtype=torch.bfloat16, scale=0.3, seed=1), rnd(I, K, dtype=torch.bfloat16, scale=0.3, seed=2)
    pairs = torch.stack([gate, up], 1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), 9.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16_silu_mul(x, pairs, out)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    close(out, g / (1 + torch.exp(-g)) * u, 3e-2, 1e-2)
    assert ops.gemm_tc_status() == 0


# ------------------------------------------------------------- rope + cache
def plain_rope(x, pos, inv_freq, rotary_dim, pairing="half"):
    """x [heads, D] float64; frequency i turns the pair (i, i + rotary_dim/2), or
    (2i, 2i + 1) when interleaved; angle as a 32-bit product."""
    half = rotary_dim // 2
    angle = (np.float32(pos) * inv_freq.astype(np.float32)).astype(np.float64)
    c, s = torch.from_numpy(np.cos(angle)), torch.from_numpy(np.sin(angle))
    y = x.clone()
    if pairing == "interleaved":
        a, b = x[:, 0:rotary_dim:2], x[:, 1:rotary_dim:2]
        y[:, 0:rotary_dim:2] = a * c - b * s
        y[:, 1:rotary_dim:2] = b * c + a * s
        return y
    y[:, :half] = x[:, :half] * c - x[:, half:rotary_dim] * s
    y[:, half:rotary_dim] = x[:, half:rotary_dim] * c + x[:, :half] * s
    return y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("A,Kh,D,rot", [(4, 2, 16, 16), (6, 3, 32, 32), (3, 1, 48, 32), (8, 2, 128, 128)])
@pytest.mark.parametrize("source", ["tensor", "planes"])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_rope_kv_write(ops, dtype, A, Kh, D, rot, source, pairing):
    """Positions far apart (a 32-bit angle matters at 100k), a padding token,
    pages scattered; queries in place or from split planes; partial rotary
    width; both ways of pairing the rotated elements."""
    positions = [0, 1, 63, 64, 100000, 7]
    seqs = [0, 0, 1, 1, 2, -1]
    T = len(positions)
    width = (A + 2 * Kh) * D
    n_pages = 1600
    table = torch.zeros(3, 1563, dtype=torch.int32)
    table[0, 0], table[1, 0], table[1, 1], table[2, 100000 // 64] = 5, 9, 2, 11
    inv_freq = (10000.0 ** (-np.arange(0, rot, 2, dtype=np.float32) / rot)).astype(np.float32)
    qkv = rnd(T, width, dtype=dtype)
    k_cache = torch.zeros(n_pages, Kh, 64, D, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    ref = qkv.double().cpu()
    args = (torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seqs, dtype=torch.int32, device=DEV), table.to(DEV),
            torch.from_numpy(inv_freq).to(DEV), rot, k_cache, v_cache, A, Kh, D)
    if source == "tensor":
        q = ops.rope_kv_write(qkv, *args, pairing=pairing)
        assert q.data_ptr() == qkv.data_ptr()  # rotated in place
    else:
        parts = torch.stack([qkv.float() * 0.25, qkv.float() * 0.5, qkv.float() * 0.25])
        q = ops.rope_kv_write(ops.Planes(parts.contiguous()), *args, dtype=dtype, pairing=pairing)
    a, r = (1e-6, 1e-6) if dtype == torch.float32 else (2e-2, 8e-3)
    for t in range(T - 1):
        row = ref[t].view(A + 2 * Kh, D)
        close(q[t].view(A, D), plain_rope(row[:A], positions[t], inv_freq, rot, pairing), a, r)
        page = int(table[seqs[t], positions[t] // 64])
        close(k_cache[page, :, positions[t] % 64],
              plain_rope(row[A:A + Kh], positions[t], inv_freq, rot, pairing), a, r)
        close(v_cache[page, :, positions[t] % 64], row[A + Kh:], a, r)
    # nothing else was written, and the padding token wrote nothing
    written = {(int(table[seqs[t], positions[t] // 64]), positions[t] % 64) for t in range(T - 1)}
    mask = torch.ones(n_pages, 64, dtype=torch.bool)
    for p, rr in written:
        mask[p, rr] = False
    assert float(k_cache.float().abs().sum(dim=(1, 3)).cpu()[mask].max()) == 0.0


@pytest.mark.parametrize("A,Kh,D,rot", [(4, 2, 16, 16), (6, 3, 32, 32), (3, 1, 48, 32), (8, 2, 128, 128),
                                        (2, 2, 64, 0), (5, 1, 80, 48)])
@pytest.mark.parametrize("T", [6, 13])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_gemm_skinny_rope(ops, A, Kh, D, rot, T, pairing):
    """Projection, rotation and cache write in one kernel against the plain
    formulas: far positions, a padding token, scattered pages, partial and
    absent rotation, both pairings; without cache writes only the queries appear."""
    K = 264
    positions = ([0, 1, 63, 64, 100000, 7] + list(range(200, 200 + T)))[:T]
    seqs = ([0, 0, 1, 1, 2, -1] + [0] * T)[:T]
    width = (A + 2 * Kh) * D
    n_pages = 1600
    table = torch.zeros(3, 1563, dtype=torch.int32)
    table[0, 0], table[1, 0], table[1, 1], table[2, 100000 // 64] = 5, 9, 2, 11
    table[0, 3] = 17  # positions 200.. of sequence 0
    inv_freq = (10000.0 ** (-np.arange(0, rot, 2, dtype=np.float32) / max(rot, 1))).astype(np.float32)
    x, w = rnd(T, K, dtype=torch.bfloat16), rnd(width, K, dtype=torch.bfloat16, scale=0.1, seed=4)
    ref = (x.double() @ w.double().T).cpu()
    k_cache = torch.zeros(n_pages, Kh, 64, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    args = (torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seqs, dtype=torch.int32, device=DEV), table.to(DEV),
            torch.from_numpy(inv_freq).to(DEV), rot)
    q = ops.gemm_skinny_rope(x, w, *args, k_cache, v_cache, A, Kh, D,
                             then_reads=rnd(8, 64, dtype=torch.bfloat16), pairing=pairing)
    a, r = 2e-2, 8e-3
    written = set()
    for t in range(T):
        if seqs[t] < 0:
            continue
        row = ref[t].view(A + 2 * Kh, D)
        close(q[t].view(A, D), plain_rope(row[:A], positions[t], inv_freq, rot, pairing), a, r)
        page = int(table[seqs[t], positions[t] // 64])
        written.add((page, positions[t] % 64))
        close(k_cache[page, :, positions[t] % 64],
              plain_rope(row[A:A + Kh], positions[t], inv_freq, rot, pairing), a, r)
        close(v_cache[page, :, positions[t] % 64], row[A + Kh:], a, r)
    mask = torch.ones(n_pages, 64, dtype=torch.bool)
    for p, rr in written:
        mask[p, rr] = False
    for cache in (k_cache, v_cache):
        assert float(cache.float().abs().sum(dim=(1, 3)).cpu()[mask].max()) == 0.0
    # agrees with the two separate kernels to the rounding of their intermediate
    qkv = torch.empty(T, width, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(x, w, qkv)
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    q2 = ops.rope_kv_write(qkv, *args, k2, v2, A, Kh, D, pairing=pairing)
    live = [t for t in range(T) if seqs[t] >= 0]
    close(q[live], q2[live].double(), a, r)
    close(k_cache, k2.double(), a, r)
    close(v_cache, v2.double(), a, r)
    # reading another layer's cache: no key or value is computed or stored
    k_cache.zero_(), v_cache.zero_()
    q3 = ops.gemm_skinny_rope(x, w, *args, k_cache, v_cache, A, Kh, D, write_cache=False,
                              pairing=pairing)
    assert torch.equal(q3[live], q[live])
    assert float(k_cache.float().abs().max()) == 0.0 and float(v_cache.float().abs().max()) == 0.0


@pytest.mark.parametrize("T,H,K", [(1, 96, 72), (8, 200, 264), (13, 3072, 520), (16, 104, 64)])
def test_gemm_skinny_takes_the_norm_over(ops, T, H, K):
    """The projection in front of a norm adds into the residual rows and leaves
    resid * gamma and the shares of the sums of squares; the projections behind
    the norm (plain, SiLU-mul, rotary) apply 1/sqrt(mean + eps) to their sums.
    Against the plain formulas, and against the norm as a kernel of its own."""
    eps = 3e-5
    x, w = rnd(T, K, dtype=torch.bfloat16), rnd(H, K, dtype=torch.bfloat16, scale=0.2, seed=1)
    resid0 = rnd(T, H, seed=2) * 3.0
    resid0[0] *= 40.0  # rows of very different scale
    gamma = (1.0 + 0.3 * rnd(H, seed=3)).contiguous()
    resid = resid0.clone()
    pending = ops.gemm_skinny_residual(x, w, ops.ResidualSink(resid, gamma, eps),
                                       then_reads=rnd(8, 64, dtype=torch.bfloat16))
    want_resid = resid0.double() + x.double() @ w.double().T
    close(resid, want_resid, 1e-4, 1e-5)
    close(pending.values, want_resid * gamma.double(), 1e-6, 2.0 ** -8)
    assert pending.shares.shape == ((H + 15) // 16, 16)
    close(pending.shares[:, :T].sum(0), (want_resid ** 2).sum(1), 1e-3, 1e-5)
    scaled = ops.add_rmsnorm(resid, pending, gamma, eps, None)
    assert isinstance(scaled, ops.RowScaled)
    rstd = 1.0 / torch.sqrt((resid.double() ** 2).mean(1, keepdim=True) + eps)
    # the plain tensor
    close(scaled.materialize(), pending.values.double() * rstd, 1e-6, 2.0 ** -8)
    # behind the norm: plain product (whole and in K shares), SiLU-mul, rotary
    N = 80
    w2 = rnd(N, H, dtype=torch.bfloat16, scale=0.1, seed=5)
    want = (pending.values.double() @ w2.double().T) * rstd
    out = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(scaled, w2, out)
    close(out, want, 1e-3, 8e-3)
    planes = torch.empty(2, T, N, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(scaled, w2, planes, ksplit=2)
    close(planes.sum(0), want, 1e-4, 1e-4)
    act = torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(scaled, w2, act, epilogue=1)
    close(act, torch.nn.functional.silu(want[:, 0::2]) * want[:, 1::2], 1e-3, 1e-2)
    A, Kh, D = 3, 1, 16
    inv_freq = torch.from_numpy((10000.0 ** (-np.arange(0, D, 2, dtype=np.float32) / D))).to(DEV)
    positions = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    seqs = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.tensor([[1]], dtype=torch.int32, device=DEV)
    k_cache = torch.zeros(2, Kh, 64, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    q = ops.gemm_skinny_rope(scaled, w2, positions, seqs, table, inv_freq, D, k_cache, v_cache,
                             A, Kh, D)
    for t in range(T):
        row = want[t].cpu().view(A + 2 * Kh, D)
        close(q[t].view(A, D), plain_rope(row[:A], 5 + t, inv_freq.cpu().numpy(), D), 2e-3, 8e-3)
        close(v_cache[1, :, 5 + t], row[A + Kh:], 2e-3, 8e-3)
    # the same through the general entry: it hands the sink to the skinny kernel
    resid2 = resid0.clone()
    pending2 = ops.gemm_bf16(x, w, residual=ops.ResidualSink(resid2, gamma, eps))
    assert isinstance(pending2, ops.NormPending) and torch.equal(resid2, resid)
    # ... and agrees with the norm as its own kernel to the rounding of its output
    resid3, delta = resid0.clone(), torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(x, w, delta)
    normed = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(resid3, delta, gamma, eps, normed)
    apart = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(normed, w2, apart)
    close(out, apart.double(), 2e-2 * float(want.abs().max()), 2e-2)
    # a sink for other rows or another norm is refused
    with pytest.raises(ops.KernelError, match="another"):
        ops.add_rmsnorm(resid3, pending, gamma, eps, None)


def test_gemm_skinny_rope_ring_pages(ops):
    """A windowed group's pages are a ring: position p lands in page slot (p / 64) % ring."""
    A, Kh, D, K, ring = 2, 1, 32, 64, 3
    positions, seqs = [64 * 7 + 5], [0]
    table = torch.tensor([[4, 8, 6]], dtype=torch.int32, device=DEV)
    inv_freq = torch.from_numpy((10000.0 ** (-np.arange(0, D, 2, dtype=np.float32) / D)).astype(np.float32)).to(DEV)
    x, w = rnd(1, K, dtype=torch.bfloat16), rnd((A + 2 * Kh) * D, K, dtype=torch.bfloat16, scale=0.2, seed=4)
    k_cache = torch.zeros(10, Kh, 64, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    ops.gemm_skinny_rope(x, w, torch.tensor(positions, dtype=torch.int32, device=DEV),
                         torch.tensor(seqs, dtype=torch.int32, device=DEV), table, inv_freq, D,
                         k_cache, v_cache, A, Kh, D, ring_pages=ring)
    ref = (x.double() @ w.double().T).cpu().view(A + 2 * Kh, D)
    page = int(table[0, 7 % ring])
    close(v_cache[page, :, 5], ref[A + Kh:], 2e-2, 8e-3)
    assert float(v_cache.float().abs().sum()) == pytest.approx(float(v_cache[page, :, 5].float().abs().sum()))


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("V", [384, 5001, 128256])
def test_select_tokens_greedy_first_index_wins(ops, V):
    logits = rnd(6, V)
    logits[0, 17] = logits[0, V - 1] = 50.0      # equal maxima: the lower index
    logits[1, :] = 1.0                            # all equal: index 0
    logits[2, V - 1] = 60.0                       # the last element
    logits[3, 5] = float("nan")                   # a NaN never wins
    logits[4, :] = float("-inf")
    logits[4, 123] = -1e30
    out = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.select_tokens(logits, out, None)
    want = [17, 0, V - 1, int(torch.argmax(torch.nan_to_num(logits[3], nan=-1e38))), 123,
            int(torch.argmax(logits[5]))]
    assert out.tolist() == want


@pytest.mark.parametrize("V", [384, 128256])
def test_select_tokens_sampling_matches_the_host_restatement(ops, V):
    from foundry_b200.sampling import gumbel_scores, stream_key
    n, seed = 4, 77
    logits = rnd(n, V, scale=2.0)
    keys, steps, temps = [3, 0, 9, 3], [0, 5, 2, 1], [0.8, 1.0, 0.0, 0.8]
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    ops.select_tokens(logits, out, torch.tensor(temps, device=DEV),
                      torch.tensor([stream_key(seed, k) for k in keys], device=DEV),
                      torch.tensor(steps, device=DEV))
    host = logits.cpu().numpy()
    for r in range(n):
        if temps[r] == 0.0:
            assert out[r] == int(np.argmax(host[r]))
            continue
        scores = gumbel_scores(host[r], temps[r], seed, keys[r], steps[r])
        best = int(np.argmax(scores))
        assert int(out[r]) == best or scores[best] - scores[int(out[r])] < 1e-4
    assert out[0] != out[3] or V < 1000  # same key, another step: another draw


def test_sampling_follows_the_distribution(ops):
    """Over many steps the sampled frequencies approach softmax(logits / T)."""
    from foundry_b200.sampling import stream_key
    V, draws, T = 8, 4000, 0.7
    base = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -2.0, 0.0])
    logits = base.repeat(draws, 1).to(DEV)
    out = torch.zeros(draws, dtype=torch.int32, device=DEV)
    ops.select_tokens(logits, out, torch.full((draws,), T, device=DEV),
                      torch.full((draws,), stream_key(5, 0), dtype=torch.int64, device=DEV),
                      torch.arange(draws, device=DEV))
    freq = torch.bincount(out.long().cpu(), minlength=V).double() / draws
    want = torch.softmax(base.double() / T, 0)
    assert float((freq - want).abs().max()) < 0.03


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 64), (100, 72), (130, 200), (3072, 3072), (384, 8192), (50, 4104)])
def test_gemm_skinny(ops, M, N, K):
    """The weight-streaming kernel: ragged rows, K tails inside a chunk, both
    warp counts, both token-tile counts, strided input and output."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=9)
    want = x.double() @ w.double().T
    out = torch.full((M, N), 7.0, device=DEV)
    ops.gemm_skinny(x, w, out)
    close(out, want, 2e-4 * math.sqrt(K), 1e-5)
    wide_x = rnd(M, K + 64, dtype=torch.bfloat16, seed=10)
    wide_out = torch.zeros(M, N + 3, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(wide_x[:, 8:8 + K], w, wide_out[:, :N])
    close(wide_out[:, :N], wide_x[:, 8:8 + K].double() @ w.double().T, 2e-4 * math.sqrt(K) + 1e-2, 8e-3)
    assert float(wide_out[:, N:].abs().max()) == 0.0


@pytest.mark.parametrize("warps", [4, 8, 16])
@pytest.mark.parametrize("M,N,K,ksplit", [(3, 100, 72, 2), (8, 384, 8192, 5), (16, 50, 4104, 3),
                                          (9, 16, 64, 4), (1, 130, 200, 1)])
def test_gemm_skinny_shared_k(ops, M, N, K, ksplit, warps):
    """K shared among CTAs: float32 planes whose sum is the product (shares that
    hold no chunk write zeros); every warp count; a weight range handed over
    for prefetching changes nothing."""
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=9)
    want = x.double() @ w.double().T
    later = rnd(64, 256, dtype=torch.bfloat16, seed=3)
    if ksplit == 1:
        out = torch.full((M, N), 7.0, device=DEV)
        ops.gemm_skinny(x, w, out, warps=warps, then_reads=later)
        close(out, want, 2e-4 * math.sqrt(K), 1e-5)
        return
    planes = torch.full((ksplit, M, N), 7.0, device=DEV)
    ops.gemm_skinny(x, w, planes, ksplit=ksplit, warps=warps, then_reads=later)
    close(planes.sum(0), want, 2e-4 * math.sqrt(K), 1e-5)
    with pytest.raises(ops.KernelError):
        ops.gemm_skinny(x, w, torch.zeros(ksplit, M, N, dtype=torch.bfloat16, device=DEV), ksplit=ksplit)


def test_gemm_bf16_few_rows_few_features_shares_k(ops):
    """Fewer row groups than SMs: the dispatcher shares K and hands planes to a
    consumer that allows them, a tensor to one that does not."""
    x, w = rnd(4, 2048, dtype=torch.bfloat16), rnd(256, 2048, dtype=torch.bfloat16, seed=2)
    want = x.double() @ w.double().T
    got = ops.gemm_bf16(x, w, allow_planes=True)
    assert isinstance(got, ops.Planes) and got.count > 1
    close(got.tensor.sum(0), want, 2e-4 * math.sqrt(2048), 1e-5)
    plain = ops.gemm_bf16(x, w)
    assert isinstance(plain, torch.Tensor)
    close(plain, want, 2e-4 * math.sqrt(2048) + 1e-2, 8e-3)


@pytest.mark.parametrize("bn", [128, 144, 160, 176, 192, 208, 224, 240, 256])
@pytest.mark.parametrize("rows_a,rows_b,K", [(300, 700, 264), (2048, 1024, 512), (130, 70, 64),
                                              (1000, 5000, 72), (257, 130, 4104)])
def test_gemm_tensor_core_paired(ops, bn, rows_a, rows_b, K):
    """Two SMs on one 256-row tile (cta_group::2): more tiles than CTA pairs and
    fewer, a second CTA whose rows or weight half lie wholly outside, ragged
    edges, short and long K loops; with and without the SiLU-mul epilogue."""
    a, b = rnd(rows_a, K, dtype=torch.bfloat16, scale=0.5), rnd(rows_b, K, dtype=torch.bfloat16, scale=0.5, seed=6)
    want = a.double() @ b.double().T
    out = torch.full((rows_a, rows_b), 3.0, device=DEV)
    ops.gemm_tc(a, b, out, rows_b, 1, bn, persistent=2, constant_operand=2)
    close(out, want, 2e-4 * math.sqrt(K), 1e-5)
    act = torch.full((rows_a, rows_b // 2), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(a, b, act, rows_b // 2, 1, bn, epilogue=1, persistent=2, constant_operand=2)
    g, u = want[:, 0::2], want[:, 1::2]
    close(act, g / (1 + torch.exp(-g)) * u, 3e-2, 1e-2)
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("rows_a,rows_b,K,bn", [(2048, 3072, 1024, 256), (2560, 2304, 2048, 256),
                                                 (2048, 3000, 520, 176), (4000, 2500, 264, 208)])
def test_gemm_paired_shares_the_last_round(ops, monkeypatch, rows_a, rows_b, K, bn):
    """More tiles than CTA pairs with a thin last round: its tiles are shared
    along K, the shares meet in the workspace, the warp that delivers last sums
    them. Twice in a row (the counters must be back at zero), with and without
    the SiLU-mul epilogue, and the same result as with whole tiles only."""
    a, b = rnd(rows_a, K, dtype=torch.bfloat16, scale=0.5), rnd(rows_b, K, dtype=torch.bfloat16, scale=0.5, seed=6)
    want = a.double() @ b.double().T
    assert ops.PAIR_TAIL_SHARES
    monkeypatch.setattr(ops, "PAIR_SHARE_MIN_KBLOCKS", 4)  # share even these short K loops
    for _ in range(2):
        out = torch.full((rows_a, rows_b), 3.0, device=DEV)
        ops.gemm_tc(a, b, out, rows_b, 1, bn, persistent=2, constant_operand=2)
        close(out, want, 2e-4 * math.sqrt(K), 1e-5)
        act = torch.full((rows_a, rows_b // 2), 3.0, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(a, b, act, rows_b // 2, 1, bn, epilogue=1, persistent=2, constant_operand=2)
        g, u = want[:, 0::2], want[:, 1::2]
        close(act, g / (1 + torch.exp(-g)) * u, 3e-2, 1e-2)
    ops.PAIR_TAIL_SHARES = False
    try:
        whole = torch.full((rows_a, rows_b), 3.0, device=DEV)
        ops.gemm_tc(a, b, whole, rows_b, 1, bn, persistent=2, constant_operand=2)
    finally:
        ops.PAIR_TAIL_SHARES = True
    close(out, whole.double(), 1e-4 * math.sqrt(K), 1e-5)
    assert int(ops._pair_scratch(a.device)[1].abs().sum()) == 0
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("bn", [64, 128, 144, 176, 192, 208, 240, 256])
@pytest.mark.parametrize("rows_a,rows_b,K", [(300, 700, 264), (2048, 1024, 512), (130, 70, 64),
                                              (1000, 5000, 72)])
def test_gemm_tensor_core_persistent(ops, bn, rows_a, rows_b, K):
    """One CTA per SM over many tiles, alternating accumulators: more tiles than
    SMs, fewer tiles than SMs, ragged edges, short and long K loops; with and
    without the SiLU-mul epilogue."""
    a, b = rnd(rows_a, K, dtype=torch.bfloat16, scale=0.5), rnd(rows_b, K, dtype=torch.bfloat16, scale=0.5, seed=6)
    want = a.double() @ b.double().T
    out = torch.full((rows_a, rows_b), 3.0, device=DEV)
    ops.gemm_tc(a, b, out, rows_b, 1, bn, persistent=True, constant_operand=2)
    close(out, want, 2e-4 * math.sqrt(K), 1e-5)
    act = torch.full((rows_a, rows_b // 2), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(a, b, act, rows_b // 2, 1, bn, epilogue=1, persistent=True, constant_operand=2)
    g, u = want[:, 0::2], want[:, 1::2]
    close(act, g / (1 + torch.exp(-g)) * u, 3e-2, 1e-2)
    assert ops.gemm_tc_status() == 0


# ------------------------------------------- 17 .. 256 token rows on tcgen05
ROWS_SHAPES = [(3072, 3072), (5120, 3072), (384, 8192), (200, 264), (130, 64), (2048, 2048),
               (16384, 2048), (1000, 4104)]


@pytest.mark.parametrize("M", [17, 32, 33, 64, 100, 128, 129, 256])
@pytest.mark.parametrize("N,K", ROWS_SHAPES)
def test_gemm_rows(ops, M, N, K):
    """The few-rows product: weight tiles whose K several CTAs of a cluster share
    (summed in the kernel), tiles one CTA computes alone, ragged N and K; twice
    in a row, bit for bit the same both times; float32 and bfloat16 outputs."""
    x = rnd(M, K, dtype=torch.bfloat16, scale=0.5)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=1)
    want = x.double() @ w.double().T
    first = ops.gemm_rows(x, w, out_dtype=torch.float32)
    close(first, want, 2e-3, 1e-4)
    again = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    ops.gemm_rows(x, w, again)
    assert torch.equal(first, again)
    half = torch.full((M, N + 8), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_rows(x, w, half[:, :N])  # rows of a wider tensor
    close(half[:, :N], want, 3e-2, 1e-2)
    assert float(half[:, N:].float().min()) == 7.0
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
def test_gemm_rows_every_cluster_size(ops, monkeypatch, splits):
    """K shared by 1 to 8 CTAs of a cluster, more tokens than CTAs and fewer."""
    monkeypatch.setattr(ops, "ROWS_SPLITS", splits)
    for M, N, K in ((70, 300, 1024), (19, 128, 520), (256, 200, 4096)):
        x = rnd(M, K, dtype=torch.bfloat16, scale=0.5)
        w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=1)
        close(ops.gemm_rows(x, w, out_dtype=torch.float32), x.double() @ w.double().T, 2e-3, 1e-4)
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M", [20, 64, 200])
def test_gemm_rows_with_silu_mul_epilogue(ops, monkeypatch, M):
    monkeypatch.setattr(ops, "ROWS_MAX", 256)  # the dispatcher below takes this kernel for all M here
    K, I = 264, 1000
    x = rnd(M, K, dtype=torch.bfloat16, scale=0.5)
    gate, up = rnd(I, K, dtype=torch.bfloat16, scale=0.3, seed=1), rnd(I, K, dtype=torch.bfloat16, scale=0.3, seed=2)
    pairs = torch.stack([gate, up], 1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), 9.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_rows(x, pairs, out, silu_mul=True)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    close(out, g / (1 + torch.exp(-g)) * u, 3e-2, 1e-2)
    # the dispatcher takes the same kernel for these row counts
    out2 = torch.empty_like(out)
    ops.gemm_bf16_silu_mul(x, pairs, out2)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M,H,K", [(17, 96, 72), (40, 200, 264), (64, 3072, 520), (130, 2048, 8192)])
def test_gemm_rows_takes_the_norm_over(ops, monkeypatch, M, H, K):
    """As test_gemm_skinny_takes_the_norm_over, for 17 to 256 rows: the product in
    front of a norm adds into the residual rows, leaves resid * gamma and each
    weight tile's share of the sums of squares; the products behind the norm
    (plain, SiLU-mul, rotary) apply 1 / sqrt(mean + eps) to their sums."""
    monkeypatch.setattr(ops, "ROWS_MAX", 256)  # through the dispatcher at every M here
    eps = 3e-5
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(H, K, dtype=torch.bfloat16, scale=0.2, seed=1)
    resid0 = rnd(M, H, seed=2) * 3.0
    resid0[0] *= 40.0  # rows of very different scale
    gamma = (1.0 + 0.3 * rnd(H, seed=3)).contiguous()
    resid = resid0.clone()
    sink = ops.ResidualSink(resid, gamma, eps)
    pending = ops.gemm_bf16(x, w, residual=sink)
    assert isinstance(pending, ops.NormPending)
    want_resid = resid0.double() + x.double() @ w.double().T
    close(resid, want_resid, 2e-3, 1e-5)
    # bfloat16 of a float32 sum: half a unit in the last place of the rounded value,
    # plus what the float32 sum itself is off the float64 one
    close(pending.values, resid.double() * gamma.double(), 1e-6, 2.0 ** -8)
    assert pending.shares.shape[0] == (H + 127) // 128
    close(pending.shares[:, :M].sum(0), (want_resid ** 2).sum(1), 1e-3, 1e-4)
    scaled = ops.add_rmsnorm(resid, pending, gamma, eps, None)
    assert isinstance(scaled, ops.RowScaled)
    normed = want_resid / torch.sqrt((want_resid ** 2).mean(1, keepdim=True) + eps) * gamma.double()
    close(scaled.materialize(), normed, 2e-2, 8e-3)
    # a plain product and a SiLU-mul product behind the norm, against the products of
    # the rounded values the kernels read
    rstd = 1.0 / torch.sqrt((resid.double() ** 2).mean(1, keepdim=True) + eps)
    w2 = rnd(264, H, dtype=torch.bfloat16, scale=0.1, seed=5)
    close(ops.gemm_bf16(scaled, w2, out_dtype=torch.float32),
          (pending.values.double() @ w2.double().T) * rstd, 2e-3, 1e-4)
    pairs = rnd(400, H, dtype=torch.bfloat16, scale=0.1, seed=6)
    hidden = torch.empty(M, 200, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16_silu_mul(scaled, pairs, hidden)
    gu = (pending.values.double() @ pairs.double().T) * rstd
    close(hidden, gu[:, 0::2] / (1 + torch.exp(-gu[:, 0::2])) * gu[:, 1::2], 1e-3, 1e-2)
    # the sink must belong to the norm that takes the result
    with pytest.raises(ops.KernelError, match="another"):
        ops.add_rmsnorm(resid0.clone(), pending, gamma, eps, None)


@pytest.mark.parametrize("A,Kh,D,rot", [(4, 2, 16, 16), (6, 3, 32, 32), (3, 1, 48, 32), (8, 2, 128, 128),
                                        (2, 2, 64, 0), (32, 8, 64, 64)])
@pytest.mark.parametrize("T", [17, 70])
def test_gemm_rows_rope(ops, A, Kh, D, rot, T):
    """Projection, rotation of adjacent feature pairs and cache write in the
    few-rows product's epilogue: far positions, padding tokens, scattered pages,
    partial and absent rotation, a row-scaled input; without cache writes only
    the queries are computed. Against the plain formulas and the separate kernels."""
    K = 264
    positions = ([0, 1, 63, 64, 100000, 7] + list(range(200, 200 + T)))[:T]
    seqs = ([0, 0, 1, 1, 2, -1] + [0] * T)[:T]
    seqs[-1] = -1
    width = (A + 2 * Kh) * D
    n_pages = 1600
    table = torch.zeros(3, 1563, dtype=torch.int32)
    table[0, 0], table[1, 0], table[1, 1], table[2, 100000 // 64] = 5, 9, 2, 11
    table[0, 3], table[0, 4] = 17, 23  # positions 200.. of sequence 0
    inv_freq = (10000.0 ** (-np.arange(0, rot, 2, dtype=np.float32) / max(rot, 1))).astype(np.float32)
    x, w = rnd(T, K, dtype=torch.bfloat16), rnd(width, K, dtype=torch.bfloat16, scale=0.1, seed=4)
    ref = (x.double() @ w.double().T).cpu()
    k_cache = torch.zeros(n_pages, Kh, 64, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    args = (torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(seqs, dtype=torch.int32, device=DEV), table.to(DEV),
            torch.from_numpy(inv_freq).to(DEV), rot)
    q = ops.gemm_rows_rope(x, w, *args, k_cache, v_cache, A, Kh, D)
    a, r = 2e-2, 8e-3
    written = set()
    for t in range(T):
        if seqs[t] < 0:
            continue
        row = ref[t].view(A + 2 * Kh, D)
        close(q[t].view(A, D), plain_rope(row[:A], positions[t], inv_freq, rot, "interleaved"), a, r)
        page = int(table[seqs[t], positions[t] // 64])
        written.add((page, positions[t] % 64))
        close(k_cache[page, :, positions[t] % 64],
              plain_rope(row[A:A + Kh], positions[t], inv_freq, rot, "interleaved"), a, r)
        close(v_cache[page, :, positions[t] % 64], row[A + Kh:], a, r)
    mask = torch.ones(n_pages, 64, dtype=torch.bool)
    for p, rr in written:
        mask[p, rr] = False
    for cache in (k_cache, v_cache):
        assert float(cache.float().abs().sum(dim=(1, 3)).cpu()[mask].max()) == 0.0
    live = [t for t in range(T) if seqs[t] >= 0]
    # reading another layer's cache: no key or value is computed or stored
    k_cache.zero_(), v_cache.zero_()
    q3 = ops.gemm_rows_rope(x, w, *args, k_cache, v_cache, A, Kh, D, write_cache=False)
    assert torch.equal(q3[live], q[live])
    assert float(k_cache.float().abs().max()) == 0.0 and float(v_cache.float().abs().max()) == 0.0
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("A,Kh,D,rot,T", [(4, 2, 64, 64, 130), (6, 2, 128, 128, 300), (3, 1, 32, 16, 200),
                                          (8, 4, 64, 32, 700), (2, 2, 96, 0, 260), (24, 8, 128, 128, 520)])
def test_gemm_tc_rope(ops, A, Kh, D, rot, T):
    """Projection, rotation of adjacent feature pairs and cache write in the
    epilogue of the products whose rows are tokens (one tile per CTA, and two SMs
    per tile): far positions, padding tokens, scattered pages, partial and absent
    rotation, a row-scaled input; without cache writes only the queries are
    computed. Against the plain formulas in float64."""
    K = 264 if A < 24 else 3072
    positions = ([0, 1, 63, 64, 100000, 7] + list(range(200, 200 + T)))[:T]
    seqs = ([0, 0, 1, 1, 2, -1] + [0] * T)[:T]
    seqs[-1] = -1
    width = (A + 2 * Kh) * D
    n_pages = 1600
    table = torch.zeros(3, 1563, dtype=torch.int32)
    table[0, 0], table[1, 0], table[1, 1], table[2, 100000 // 64] = 5, 9, 2, 11
    for i, lp in enumerate(range(3, (200 + T) // 64 + 1)):
        table[0, lp] = 17 + 3 * i  # positions 200.. of sequence 0
    inv_freq = (10000.0 ** (-np.arange(0, rot, 2, dtype=np.float32) / max(rot, 1))).astype(np.float32)
    x, w = rnd(T, K, dtype=torch.bfloat16), rnd(width, K, dtype=torch.bfloat16, scale=0.1, seed=4)
    ref = (x.double() @ w.double().T).cpu()
    k_cache = torch.zeros(n_pages, Kh, 64, D, dtype=torch.bfloat16, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    pos_d = torch.tensor(positions, dtype=torch.int32, device=DEV)
    freq_d = torch.from_numpy(inv_freq).to(DEV)
    cs = ops.rope_table(pos_d, freq_d)
    angle = (np.array(positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    want_cs = np.stack([np.cos(angle.astype(np.float64)), np.sin(angle.astype(np.float64))], -1)
    assert cs.shape == (rot // 2, T, 2)  # a frequency's angles of all tokens lie together
    if rot:
        assert float(np.abs(cs.cpu().numpy().transpose(1, 0, 2) - want_cs).max()) < 2e-6
    args = (cs, pos_d, torch.tensor(seqs, dtype=torch.int32, device=DEV), table.to(DEV), rot)
    assert ops.qkv_tc_rope_fusable(x, w, rot, D, k_cache, "interleaved")
    q = ops.gemm_tc_rope(x, w, *args, k_cache, v_cache, A, Kh, D)
    a, r = 2e-2, 8e-3
    if K > 1000:
        a = 6e-2
    written = set()
    for t in range(T):
        if seqs[t] < 0:
            continue
        row = ref[t].view(A + 2 * Kh, D)
        close(q[t].view(A, D), plain_rope(row[:A], positions[t], inv_freq, rot, "interleaved"), a, r)
        page = int(table[seqs[t], positions[t] // 64])
        written.add((page, positions[t] % 64))
        close(k_cache[page, :, positions[t] % 64],
              plain_rope(row[A:A + Kh], positions[t], inv_freq, rot, "interleaved"), a, r)
        close(v_cache[page, :, positions[t] % 64], row[A + Kh:], a, r)
    mask = torch.ones(n_pages, 64, dtype=torch.bool)
    for p, rr in written:
        mask[p, rr] = False
    for cache in (k_cache, v_cache):
        assert float(cache.float().abs().sum(dim=(1, 3)).cpu()[mask].max()) == 0.0
    live = [t for t in range(T) if seqs[t] >= 0]
    # the product followed by the rotary kernel rounds to 16 bits twice, this once: the
    # two agree to three units of bfloat16's last place
    qkv = ops.gemm_bf16(x, w)
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    q2 = ops.rope_kv_write(qkv, args[1], args[2], args[3], freq_d, rot, k2, v2, A, Kh, D,
                           pairing="interleaved")
    # (of the values that meet in a rotation, so of the largest of a token's row)
    gap = (q2[live].float() - q[live].float()).abs().amax(dim=1)
    assert bool((gap <= 3 * 2.0 ** -8 * q[live].float().abs().amax(dim=1)).all())
    # a row-scaled input: the epilogue multiplies by the tokens' scales first
    shares = torch.rand(3, T, device=DEV) + 0.5
    scaled = ops.RowScaled(x, shares, 1e-5)
    k3, v3 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    q3 = ops.gemm_tc_rope(scaled, w, *args, k3, v3, A, Kh, D)
    rstd = (1.0 / torch.sqrt(shares.double().sum(0) / K + 1e-5)).cpu()
    for t in live[:40]:
        row = (ref[t] * rstd[t]).view(A + 2 * Kh, D)
        close(q3[t].view(A, D), plain_rope(row[:A], positions[t], inv_freq, rot, "interleaved"),
              a * float(rstd[t]) + a, r)
    # reading another layer's cache: no key or value is computed or stored
    k_cache.zero_(), v_cache.zero_()
    q4 = ops.gemm_tc_rope(x, w, *args, k_cache, v_cache, A, Kh, D, write_cache=False)
    assert torch.equal(q4[live], q[live])
    assert float(k_cache.float().abs().max()) == 0.0 and float(v_cache.float().abs().max()) == 0.0
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("M,H,K", [(100, 200, 264), (128, 3072, 520), (300, 2048, 1024), (700, 3072, 8192),
                                   (2048, 3072, 3072), (2500, 1000, 264)])
def test_gemm_many_rows_takes_the_norm_over(ops, monkeypatch, M, H, K):
    monkeypatch.setattr(ops, "NORM_FUSION_ROWS", 1 << 20)  # off by default for these row counts
    _many_rows_norm(ops, M, H, K)


def _many_rows_norm(ops, M, H, K):
    """The products whose rows are tokens (one tile per CTA without K shares, one
    CTA per SM, two SMs per tile, the shared last round): in front of a norm they
    add into the residual rows and leave resid * gamma and each feature tile's share
    of the sums of squares; behind the norm they apply 1 / sqrt(mean + eps) in their
    epilogue, the plain product and the SiLU-mul product alike."""
    eps = 3e-5
    x, w = rnd(M, K, dtype=torch.bfloat16), rnd(H, K, dtype=torch.bfloat16, scale=0.2, seed=1)
    resid0 = rnd(M, H, seed=2) * 3.0
    resid0[0] *= 40.0
    gamma = (1.0 + 0.3 * rnd(H, seed=3)).contiguous()
    resid = resid0.clone()
    pending = ops.gemm_bf16(x, w, residual=ops.ResidualSink(resid, gamma, eps))
    if not isinstance(pending, ops.NormPending):
        # K shared among CTAs as float32 planes: the norm stays a kernel of its own
        assert ops._one_tile_plan(M, H, K)[0] > 1
        return
    want_resid = resid0.double() + x.double() @ w.double().T
    close(resid, want_resid, 4e-3, 1e-5)
    close(pending.values, resid.double() * gamma.double(), 1e-6, 2.0 ** -8)
    close(pending.shares[:, :M].sum(0), (want_resid ** 2).sum(1), 1e-3, 1e-4)
    scaled = ops.add_rmsnorm(resid, pending, gamma, eps, None)
    assert isinstance(scaled, ops.RowScaled)
    rstd = 1.0 / torch.sqrt((resid.double() ** 2).mean(1, keepdim=True) + eps)
    w2 = rnd(264, H, dtype=torch.bfloat16, scale=0.1, seed=5)
    many = M > 128 and not (ops._one_tile_plan(M, 264, H)[1] and M <= ops.ONE_TILE_ROWS)
    if many or ops._one_tile_plan(M, 264, H)[0] == 1:
        inputs = pending.values.double() * rstd  # the scale is applied in the epilogue
    else:
        inputs = scaled.materialize().double()   # K is shared as planes: the scaled tensor is made first
    close(ops.gemm_bf16(scaled, w2, out_dtype=torch.float32), inputs @ w2.double().T, 4e-3, 1e-4)
    pairs = rnd(400, H, dtype=torch.bfloat16, scale=0.1, seed=6)
    hidden = torch.empty(M, 200, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16_silu_mul(scaled, pairs, hidden)
    gu = (pending.values.double() @ pairs.double().T) * rstd
    close(hidden, gu[:, 0::2] / (1 + torch.exp(-gu[:, 0::2])) * gu[:, 1::2], 2e-3, 1e-2)
    assert ops.gemm_tc_status() == 0
