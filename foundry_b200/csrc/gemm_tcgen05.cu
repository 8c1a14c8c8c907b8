// bfloat16 matrix product on the 5th-generation tensor cores:
//   D[i, j] = sum_k A[i, k] * B[j, k],  A: [rows_a, K], B: [rows_b, K], both K-major,
// accumulated in 32-bit in tensor memory. A projection y = x W^T
// (src/nn/linear.rs:19-36; the reference's own 16x16-tile kernel is
// src/metal/kernels/matmul.metal:29-73) maps onto it in two ways:
//   many tokens:  A = x (tokens), B = W (features): out[i * ldo + j]
//   few tokens:   A = W (features), B = x (tokens): out[j * ldo + i]   ("swapped")
// so that the 128-row operand is always full. In swapped form the weights
// stream through once and the token count is only the instruction's N (16..256).
//
// One CTA computes one 128 x BN tile over one K range (split-K gives each CTA
// of a tile a range of its own and a float32 partial plane of its own).
// Roles: warp 0 issues TMA loads (one lane); warp 1 allocates tensor memory and
// issues tcgen05.mma (one lane); warps 2-5 read the accumulator back with
// tcgen05.ld and store. Operand tiles are 64 elements (128 bytes) wide in K,
// laid out by TMA with the 128-byte swizzle that the MMA descriptors name.
// No load is multicast; every CTA fetches its own tiles.
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records
// where in `fb_gemm_tc_status`, stops issuing work, lets the other roles run
// out as well, frees its tensor memory and returns.
#define FB_STATUS_KERNEL 1
#include "gemm_tcgen05.cuh"

namespace {

// Dynamic shared memory: [stages][A tile 128x64][B tile BNx64] bf16, 1024-aligned,
// then the barriers.
template <int BN>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES =
      (200 * 1024) / STAGE_BYTES > 10 ? 10 : (200 * 1024) / STAGE_BYTES;
  static constexpr int BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256;
};

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  constexpr int STAGES = Smem<BN>::STAGES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;  // power of two >= 32
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * Smem<BN>::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
  const int total_kb = (p.K + BK - 1) / BK;
  const int kb0 = split * p.kblocks_per_split;
  int nkb = total_kb - kb0;
  if (nkb > p.kblocks_per_split) nkb = p.kblocks_per_split;
  if (nkb < 0) nkb = 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The operand that holds weights does not depend on the kernel before this
      // one: its first stages are requested at once, the other operand's after
      // the wait. (The stages are empty at the start: no wait on `empty` yet.)
      const int early = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * Smem<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
        mbar_expect_tx(&full[i], Smem<BN>::STAGE_BYTES);
        const int k = (kb0 + i) * BK;
        if (p.constant_operand == 1) tma_load_2d(a_dst, &map_a, &full[i], k, tile_a * BM);
        if (p.constant_operand == 2) tma_load_2d(b_dst, &map_b, &full[i], k, tile_b * BN);
      }
      fb_pdl_wait();
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * Smem<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
        const int k = (kb0 + i) * BK;
        if (p.constant_operand != 1) tma_load_2d(a_dst, &map_a, &full[i], k, tile_a * BM);
        if (p.constant_operand != 2) tma_load_2d(b_dst, &map_b, &full[i], k, tile_b * BN);
      }
      for (int i = early; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, 1, i)) break;
        uint8_t* a_dst = tiles + s * Smem<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
        mbar_expect_tx(&full[s], Smem<BN>::STAGE_BYTES);
        const int k = (kb0 + i) * BK;
        tma_load_2d(a_dst, &map_a, &full[s], k, tile_a * BM);
        tma_load_2d(b_dst, &map_b, &full[s], k, tile_b * BN);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(&full[s], phase, abort_flag, 2, i);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * Smem<BN>::STAGE_BYTES);
        const uint32_t b_addr = a_addr + Smem<BN>::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing K by 16 elements inside the swizzle row = +32 bytes
          umma(tmem_base, make_desc(a_addr + k * UMMA_K * 2), make_desc(b_addr + k * UMMA_K * 2),
               idesc, (i | k) != 0 ? 1u : 0u);
        }
        tc_commit(&empty[s]);  // frees the stage when these MMAs have read it
      }
      if (ok) tc_commit(acc_full);  // accumulator complete
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;             // the TMEM lanes this warp may read
    const int i_local = quarter * 32 + lane;  // row of A within the tile
    const long long i_global = (long long)tile_a * BM + i_local;
    bool ok = true;
    if (nkb > 0) ok = mbar_wait(acc_full, 0, abort_flag, 3, 0);
    tc_fence_after();
    fb_pdl_wait();  // returns at once when operands arrived; orders the stores for nkb == 0
    if (ok) {
      float* out_f = (float*)p.out + (long long)split * p.split_stride;
      __nv_bfloat16* out_h = (__nv_bfloat16*)p.out;
      constexpr int CHUNK = (BN % 32 == 0) ? 32 : 16;
      const float scale = token_scale(p, i_global);
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += CHUNK) {
        float v[CHUNK];
        if (nkb > 0) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c;
          if constexpr (CHUNK == 32) {
            uint32_t r[32];
            tmem_ld32(taddr, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
          } else {
            uint32_t r[16];
            tmem_ld16(taddr, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < CHUNK; ++e) v[e] = 0.f;
        }
        ss += finish_chunk<CHUNK>(p, v, scale, i_global, (long long)tile_b * BN + c, lane, out_f, out_h);
      }
      finish_tile(p, ss, i_global, tile_b);
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------ persistent
// The same product for many token rows, as one CTA per SM that walks over
// tiles (tile index = blockIdx.x, += gridDim.x; the A tile index runs fastest,
// so the CTAs of a wave share weight tiles in L2). Two accumulators live in
// tensor memory: while the epilogue warps read tile j out of one, the MMA warp
// already fills the other with tile j + 1, and the TMA warp runs ahead of both
// through the ring of shared-memory stages, across tile boundaries.

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_b, const GemmParams p,
                          int tiles_a, int tiles_b) {
  constexpr int STAGES = Smem<BN>::STAGES;
  constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * Smem<BN>::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = tiles_a * tiles_b;
  const int nkb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;  // stage uses so far, across tiles
      bool ok = true;
      // the first tile's first stages: constants at once, the rest after the wait
      const int first = (int)blockIdx.x;
      const int early = (first < total_tiles) ? (nkb < STAGES ? nkb : STAGES) : 0;
      const int fa = first % tiles_a, fb = first / tiles_a;
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * Smem<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
        mbar_expect_tx(&full[i], Smem<BN>::STAGE_BYTES);
        if (p.constant_operand == 1) tma_load_2d(a_dst, &map_a, &full[i], i * BK, fa * BM);
        if (p.constant_operand == 2) tma_load_2d(b_dst, &map_b, &full[i], i * BK, fb * BN);
      }
      fb_pdl_wait();
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * Smem<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
        if (p.constant_operand != 1) tma_load_2d(a_dst, &map_a, &full[i], i * BK, fa * BM);
        if (p.constant_operand != 2) tma_load_2d(b_dst, &map_b, &full[i], i * BK, fb * BN);
      }
      for (int tile = first; tile < total_tiles && ok; tile += gridDim.x) {
        const int ta = tile % tiles_a, tb = tile / tiles_a;
        for (int kb = (tile == first ? early : 0); kb < nkb; ++kb) {
          const int use = it + kb;
          const int s = use % STAGES;
          const uint32_t phase = (uint32_t)(use / STAGES) & 1u;
          if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, 1, kb)) { ok = false; break; }
          uint8_t* a_dst = tiles + s * Smem<BN>::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Smem<BN>::A_BYTES;
          mbar_expect_tx(&full[s], Smem<BN>::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full[s], kb * BK, ta * BM);
          tma_load_2d(b_dst, &map_b, &full[s], kb * BK, tb * BN);
        }
        it += nkb;
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int it = 0, j = 0;
      bool ok = true;
      for (int tile = (int)blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++j) {
        const int buf = j & 1;
        // the epilogue must have emptied this accumulator (free at its first two uses)
        ok = mbar_wait(&acc_empty[buf], (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag, 4, j);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < nkb; ++kb) {
          const int use = it + kb;
          const int s = use % STAGES;
          const uint32_t phase = (uint32_t)(use / STAGES) & 1u;
          ok = mbar_wait(&full[s], phase, abort_flag, 2, kb);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * Smem<BN>::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Smem<BN>::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(d_tmem, make_desc(a_addr + k * UMMA_K * 2), make_desc(b_addr + k * UMMA_K * 2),
                 idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);
        it += nkb;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    float* out_f = (float*)p.out;
    __nv_bfloat16* out_h = (__nv_bfloat16*)p.out;
    constexpr int CHUNK = (BN % 32 == 0) ? 32 : 16;
    fb_pdl_wait();
    int j = 0;
    bool ok = true;
    for (int tile = (int)blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++j) {
      const int ta = tile % tiles_a, tb = tile / tiles_a;
      const int buf = j & 1;
      ok = mbar_wait(&acc_full[buf], (uint32_t)((j >> 1) & 1), abort_flag, 3, j);
      if (!ok) break;
      tc_fence_after();
      const long long i_global = (long long)ta * BM + quarter * 32 + lane;
      const float scale = token_scale(p, i_global);
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += CHUNK) {
        float v[CHUNK];
        const uint32_t taddr =
            tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c);
        if constexpr (CHUNK == 32) {
          uint32_t r[32];
          tmem_ld32(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
        } else {
          uint32_t r[16];
          tmem_ld16(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
        }
        ss += finish_chunk<CHUNK>(p, v, scale, i_global, (long long)tb * BN + c, lane, out_f, out_h);
      }
      finish_tile(p, ss, i_global, tb);
      // this warp has read its lanes of the accumulator: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
           cudaStream_t stream) {
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<BN>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
  }
  fb_launch(gemm_tc_kernel<BN>, dim3(grid), dim3(THREADS), Smem<BN>::BYTES, stream, ma, mb, p);
  return fb_check_launch("gemm_tc");
}

template <int BN>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p,
                      int tiles_a, int tiles_b, cudaStream_t stream) {
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<BN>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
  }
  const int total = tiles_a * tiles_b;
  const int ctas = total < sm_count() ? total : sm_count();
  fb_launch(gemm_tc_persistent_kernel<BN>, dim3(ctas), dim3(THREADS), Smem<BN>::BYTES, stream, ma,
            mb, p, tiles_a, tiles_b);
  return fb_check_launch("gemm_tc_persistent");
}

}  // namespace

// out = A * B^T in the layout the strides give; see the file header.
//   a: [rows_a, K] bf16, row stride lda;  b: [rows_b, K] bf16, row stride ldb
//   out[i * stride_a + j * stride_b (+ split * split_stride)], float32 when out_f32
//   bn: the B-tile height (16, 32, 64, 128 or 256); splits: K ranges per tile
// With splits > 1 the output must be float32 and holds `splits` partial planes
// that the caller sums.
// constant_operand names the operand (1: a, 2: b, 0: none) that no earlier kernel
// in the stream writes (weights); its first loads do not wait for that kernel.
// persistent 1 runs one CTA per SM over all tiles with two accumulators in
// tensor memory (for many token rows; one split); persistent 2 does the same
// with two SMs on each 256 x bn tile (cta_group::2). The paired form may share
// the K of a thin last round's tiles among pairs: for that it takes a float32
// `workspace` of `workspace_bytes` and `counters` (zero between calls, 8 per
// tile of a round); without them every tile is computed whole. A share keeps at
// least `share_min_kblocks` K blocks of 64 (0: the default, 32).
// scale_*: the row scale of an input that is a norm's output without it
// (scale_ss null: none); epilogue 2: resid / gamma / xg / ss_out as in
// fb_gemm_skinny_residual, ss_out being [ceil(rows_b / bn), ss_stride]. Both need
// tokens as the A rows and one split.
// epilogue 1 fuses SiLU(gate) * up: the feature operand's rows are (gate, up)
// pairs and `out` is [tokens, features / 2] bf16; the stride of the feature
// dimension must be 1 and then indexes pairs.
static int run_gemm_tc(const void* a, long long lda, const void* b, long long ldb, int bn,
                       int splits, int persistent, const GemmParams& p, void* workspace,
                       long long workspace_bytes, int* counters, int counters_len,
                       int share_min_kblocks, cudaStream_t stream);

FB_API int fb_gemm_tc(const void* a, long long lda, int rows_a, const void* b, long long ldb,
                      int rows_b, int K, void* out, long long stride_a, long long stride_b,
                      int out_f32, int bn, int splits, long long split_stride, int epilogue,
                      int constant_operand, int persistent, void* workspace,
                      long long workspace_bytes, int* counters, int counters_len,
                      int share_min_kblocks, const float* scale_ss, int scale_count,
                      int scale_stride, int scale_dim, float scale_eps, float* resid,
                      long long ldr, const float* gamma, void* xg, long long ldxg, float* ss_out,
                      int ss_stride, cudaStream_t stream) {
  FB_REQUIRE(rows_a > 0 && rows_b > 0 && K > 0, "gemm_tc: bad sizes %d x %d x %d", rows_a, rows_b, K);
  FB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0,
             "gemm_tc: K and the row strides must be multiples of 8 elements (16 bytes), got K=%d "
             "lda=%lld ldb=%lld", K, lda, ldb);
  FB_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0,
             "gemm_tc: operands must start on 16-byte boundaries");
  FB_REQUIRE(splits >= 1 && (splits == 1 || out_f32), "gemm_tc: split-K needs a float32 output");
  FB_REQUIRE(epilogue == 0 || epilogue == 2 ||
                 (epilogue == 1 && splits == 1 && !out_f32 && (stride_a == 1 || stride_b == 1)),
             "gemm_tc: the SiLU-mul epilogue needs one split, a bf16 output and features on a "
             "unit stride");
  FB_REQUIRE((epilogue != 2 && scale_ss == nullptr) || (splits == 1 && stride_b == 1),
             "gemm_tc: the row scale and the residual epilogue need tokens as the A rows "
             "(stride_b == 1) and one split");
  FB_REQUIRE(epilogue != 2 || (resid && gamma && xg && ss_out && ss_stride >= rows_a &&
                               ldr >= rows_b && ldxg >= rows_b),
             "gemm_tc: the residual epilogue lacks an argument or a stride is too small");
  const int total_kb = (K + BK - 1) / BK;
  FB_REQUIRE(splits <= total_kb, "gemm_tc: %d splits for %d K blocks", splits, total_kb);
  bind_status_mirror(stream);
  GemmParams p;
  p.rows_a = rows_a; p.rows_b = rows_b; p.K = K;
  p.kblocks_per_split = (total_kb + splits - 1) / splits;
  p.stride_a = stride_a; p.stride_b = stride_b; p.split_stride = split_stride;
  p.out = out; p.out_f32 = out_f32; p.epilogue = epilogue;
  p.constant_operand = constant_operand;
  p.full_tiles = 0; p.tail_splits = 1; p.tail_kblocks = total_kb; p.partial = nullptr;
  p.tail_counters = nullptr;
  p.rows = FbRowExtras{scale_ss, scale_count, scale_stride,
                       scale_dim > 0 ? 1.0f / (float)scale_dim : 0.f, scale_eps, resid, ldr, gamma,
                       (__nv_bfloat16*)xg, ldxg, ss_out, ss_stride};
  p.rope = FbRopeExtras{};
  return run_gemm_tc(a, lda, b, ldb, bn, splits, persistent, p, workspace, workspace_bytes,
                     counters, counters_len, share_min_kblocks, stream);
}

// The launch of a product whose parameters are complete: the form and the tile width
// pick the kernel.
static int run_gemm_tc(const void* a, long long lda, const void* b, long long ldb, int bn,
                       int splits, int persistent, const GemmParams& p, void* workspace,
                       long long workspace_bytes, int* counters, int counters_len,
                       int share_min_kblocks, cudaStream_t stream) {
  const int rows_a = p.rows_a, rows_b = p.rows_b, K = p.K;
  if (persistent == 2) {
    // two SMs per tile (gemm_tcgen05_pair.cu)
    FB_REQUIRE(splits == 1, "gemm_tc: the paired form takes one split");
    return fb_gemm_tc_pair(a, lda, rows_a, b, ldb, rows_b, bn, p, workspace, workspace_bytes,
                           counters, counters_len, share_min_kblocks, stream);
  }
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, rows_a, K, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, rows_b, K, ldb, bn);
  if (rc) return rc;
  dim3 grid((rows_a + BM - 1) / BM, (rows_b + bn - 1) / bn, splits);
  FB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
  if (persistent) {
    FB_REQUIRE(splits == 1, "gemm_tc: the persistent form takes one split");
    switch (bn) {
      case 64: return launch_persistent<64>(ma, mb, p, grid.x, grid.y, stream);
      case 128: return launch_persistent<128>(ma, mb, p, grid.x, grid.y, stream);
      case 144: return launch_persistent<144>(ma, mb, p, grid.x, grid.y, stream);
      case 160: return launch_persistent<160>(ma, mb, p, grid.x, grid.y, stream);
      case 176: return launch_persistent<176>(ma, mb, p, grid.x, grid.y, stream);
      case 192: return launch_persistent<192>(ma, mb, p, grid.x, grid.y, stream);
      case 208: return launch_persistent<208>(ma, mb, p, grid.x, grid.y, stream);
      case 224: return launch_persistent<224>(ma, mb, p, grid.x, grid.y, stream);
      case 240: return launch_persistent<240>(ma, mb, p, grid.x, grid.y, stream);
      case 256: return launch_persistent<256>(ma, mb, p, grid.x, grid.y, stream);
      default:
        return fb_fail(1, "gemm_tc: the persistent form takes tiles 64 or 128..256 (steps of 16) "
                          "wide, not %d", bn);
    }
  }
  switch (bn) {
    case 16: return launch<16>(ma, mb, p, grid, stream);
    case 32: return launch<32>(ma, mb, p, grid, stream);
    case 64: return launch<64>(ma, mb, p, grid, stream);
    case 128: return launch<128>(ma, mb, p, grid, stream);
    case 256: return launch<256>(ma, mb, p, grid, stream);
    default: return fb_fail(1, "gemm_tc: tile height %d is not one of 16, 32, 64, 128, 256", bn);
  }
}

// The fused q/k/v projection of many tokens: x [T, K] (row stride ldx) times
// w [(A + 2 Kh) * D, K]^T with rotation and cache write in the epilogue (see
// FbRopeExtras), an optional row scale of x as in fb_gemm_tc. `cs` comes from
// fb_rope_table. D must be a multiple of 32 (a thread's 32 consecutive features
// lie in one head) and the rotation pairs neighbouring features.
FB_API int fb_gemm_tc_rope(const void* x, long long ldx, int T, const void* w, long long ldw, int K,
                           int bn, int persistent, void* workspace, long long workspace_bytes,
                           int* counters, int counters_len, int share_min_kblocks,
                           const float* scale_ss, int scale_count, int scale_stride, int scale_dim,
                           float scale_eps, const void* cs, int half, const int* positions,
                           const int* seq_of_token, const int* page_table, int max_pages,
                           int ring_pages, void* k_cache, void* v_cache, long long page_stride,
                           long long head_stride, int A, int Kh, int D, int write_cache,
                           void* q_out, long long ldq, cudaStream_t stream) {
  FB_REQUIRE(T > 0 && K > 0 && A > 0 && Kh > 0 && D > 0, "gemm_tc_rope: bad sizes");
  FB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)x % 16) == 0 &&
                 ((uintptr_t)w % 16) == 0,
             "gemm_tc_rope: K, the row strides and the operands must keep 16-byte alignment");
  FB_REQUIRE(D % 32 == 0 && half >= 0 && 2 * half <= D,
             "gemm_tc_rope: head size %d must be a multiple of 32 and hold the rotary width %d", D,
             2 * half);
  FB_REQUIRE(half == 0 || (cs != nullptr && ((uintptr_t)cs % 8) == 0),
             "gemm_tc_rope: the table of cos and sin is missing or misaligned");
  FB_REQUIRE(q_out != nullptr && ldq % 8 == 0 && ldq >= (long long)A * D &&
                 ((uintptr_t)q_out % 16) == 0,
             "gemm_tc_rope: the query rows must be 16-byte aligned with a stride of %d or more",
             A * D);
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && page_stride % 8 == 0 &&
                              head_stride % 8 == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                              ((uintptr_t)v_cache % 16) == 0),
             "gemm_tc_rope: the cache is missing or its strides break 16-byte alignment");
  FB_REQUIRE(positions && seq_of_token, "gemm_tc_rope: positions and sequence indices are missing");
  bind_status_mirror(stream);
  const int total_kb = (K + BK - 1) / BK;
  GemmParams p;
  p.rows_a = T; p.rows_b = (write_cache ? A + 2 * Kh : A) * D; p.K = K;  // w holds only the rows that are wanted
  p.kblocks_per_split = total_kb;
  p.stride_a = ldq; p.stride_b = 1; p.split_stride = 0;
  p.out = q_out; p.out_f32 = 0; p.epilogue = 3;
  p.constant_operand = 2;
  p.full_tiles = 0; p.tail_splits = 1; p.tail_kblocks = total_kb; p.partial = nullptr;
  p.tail_counters = nullptr;
  p.rows = FbRowExtras{scale_ss, scale_count, scale_stride,
                       scale_dim > 0 ? 1.0f / (float)scale_dim : 0.f, scale_eps, nullptr, 0,
                       nullptr, nullptr, 0, nullptr, 0};
  p.rope = FbRopeExtras{(const float2*)cs, half, positions, seq_of_token, page_table, max_pages,
                        ring_pages, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_stride,
                        head_stride, A, Kh, D, write_cache, (__nv_bfloat16*)q_out, ldq};
  return run_gemm_tc(x, ldx, w, ldw, bn, 1, persistent, p, workspace, workspace_bytes, counters,
                     counters_len, share_min_kblocks, stream);
}

// Reads and clears the device-side status: 0 when no wait ever ran out, else
// the code of the role that gave up (1 producer, 2 MMA, 3 epilogue); `detail`
// receives {where, block, k-block}. Synchronises the device.
FB_API int fb_gemm_tc_status(int* detail) {
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, g_status, sizeof(host));
  if (e != cudaSuccess) return fb_fail(2, "gemm_tc_status: %s", cudaGetErrorString(e));
  if (detail) { detail[0] = host[1]; detail[1] = host[2]; detail[2] = host[3]; }
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  return host[0] ? host[1] : 0;
}

