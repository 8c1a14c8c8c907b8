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
#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;            // rows of A per tile = instruction M
constexpr int BK = 64;             // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;         // K of one tcgen05.mma for 16-bit inputs
constexpr int THREADS = 192;       // 6 warps
struct GemmParams {
  int rows_a, rows_b, K;
  int kblocks_per_split;      // K blocks of BK each CTA of a tile walks
  long long stride_a, stride_b;  // out[i * stride_a + j * stride_b]
  long long split_stride;        // elements between split-K planes
  void* out;
  int out_f32;                // 1: float32 output, 0: bfloat16
  int constant_operand;       // 1: A holds constants (weights), 2: B does, 0: neither
  int epilogue;               // 0: store D; 1: SiLU(gate) * up over interleaved feature pairs
  // paired form only: the tiles of the last, partly filled round are shared along K
  int full_tiles;             // tiles [0, full_tiles) are computed whole
  int tail_splits;            // K shares of every later tile (1: whole too)
  int tail_kblocks;           // K blocks per share
  float* partial;             // float32 partial sums of the shares (layout: see the kernel)
  int* tail_counters;         // [tail tile][8]: shares delivered per (CTA of the pair, epilogue warp)
};

// Stores CHUNK consecutive accumulator columns (j0 .. j0 + CHUNK) of row
// i_global, in the layout and with the epilogue the parameters name.
template <int CHUNK>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const float (&v)[CHUNK],
                                            long long i_global, long long j0, int lane,
                                            float* out_f, __nv_bfloat16* out_h) {
  if (p.epilogue == 1) {
    // Feature rows come in (gate, up) pairs: 2f holds gate f, 2f+1 up f.
    // out[token, f] = gate / (1 + exp(-gate)) * up, in 32-bit, stored bf16.
    if (p.stride_b == 1) {
      // features run along j: pairs sit in this thread's registers
      if (i_global < p.rows_a) {
        const long long base = i_global * p.stride_a + (j0 >> 1);
        if (j0 + CHUNK <= p.rows_b && (base % 8) == 0) {
#pragma unroll
          for (int e = 0; e < CHUNK; e += 16) {  // 8 results = 16 bytes per store
            float r8[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float gate = v[e + 2 * q];
              r8[q] = gate / (1.0f + __expf(-gate)) * v[e + 2 * q + 1];
            }
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(r8[0], r8[1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(r8[2], r8[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(r8[4], r8[5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(r8[6], r8[7]);
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2);
            pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(out_h + base + (e >> 1)) = pk;
          }
        } else {
#pragma unroll
          for (int e = 0; e < CHUNK; e += 2) {
            if (j0 + e + 1 < p.rows_b) {
              const float gate = v[e];
              out_h[base + (e >> 1)] =
                  __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * v[e + 1]);
            }
          }
        }
      }
    } else {
      // features run along i (the lanes): the partner row is the next lane
#pragma unroll
      for (int e = 0; e < CHUNK; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, v[e], 1);
        if ((lane & 1) == 0 && i_global + 1 < p.rows_a && j0 + e < p.rows_b) {
          const float gate = v[e];
          out_h[(i_global >> 1) + (j0 + e) * p.stride_b] =
              __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * other);
        }
      }
    }
  } else if (i_global < p.rows_a) {
    const long long base = i_global * p.stride_a + j0 * p.stride_b;
    if (p.stride_b == 1 && j0 + CHUNK <= p.rows_b && (base % 8) == 0) {
      // this thread's elements are contiguous: vector stores
      if (p.out_f32) {
#pragma unroll
        for (int e = 0; e < CHUNK; e += 4)
          *reinterpret_cast<float4*>(out_f + base + e) =
              make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < CHUNK; e += 8) {
          uint4 pk;
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v[e], v[e + 1]);
          __nv_bfloat162 h1 = __floats2bfloat162_rn(v[e + 2], v[e + 3]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v[e + 4], v[e + 5]);
          __nv_bfloat162 h3 = __floats2bfloat162_rn(v[e + 6], v[e + 7]);
          pk.x = *reinterpret_cast<uint32_t*>(&h0);
          pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2);
          pk.w = *reinterpret_cast<uint32_t*>(&h3);
          *reinterpret_cast<uint4*>(out_h + base + e) = pk;
        }
      }
    } else {
      // swapped form (stride_a == 1): for each j the warp's lanes are contiguous
#pragma unroll
      for (int e = 0; e < CHUNK; ++e) {
        if (j0 + e < p.rows_b) {
          const long long idx = base + (long long)e * p.stride_b;
          if (p.out_f32) out_f[idx] = v[e];
          else out_h[idx] = __float2bfloat16_rn(v[e]);
        }
      }
    }
  }
}

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
        store_chunk<CHUNK>(p, v, i_global, (long long)tile_b * BN + c, lane, out_f, out_h);
      }
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
        store_chunk<CHUNK>(p, v, i_global, (long long)tb * BN + c, lane, out_f, out_h);
      }
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

// ------------------------------------------------------------------------ pairs
// The persistent product with two SMs on one tile (tcgen05 cta_group::2): a
// cluster of two CTAs owns a 256 x BN tile. Each CTA loads its own 128 token
// rows of A and its own half (BN / 2 weight rows) of B; one thread of the
// first CTA (the leader) issues the MMAs for both, the hardware reads A and B
// from both CTAs' shared memory and writes each CTA's 128 rows of D into that
// CTA's tensor memory. What it buys: per 64-wide K step a CTA takes
// (128 + BN / 2) x 128 bytes from L2 instead of (128 + BN) x 128 for BN x 2
// tensor-core cycles, and the L2 -> SM rate (about 60 bytes per cycle and SM)
// is what caps the one-CTA form.
//
// Protocol. Both CTAs' TMA loads of a stage complete on the LEADER's full
// barrier (cp.async.bulk.tensor.cta_group::2 may name the peer's barrier;
// no multicast), which the leader arms with the bytes of both. The leader's
// commits arrive on both CTAs' barriers (tcgen05.commit ... multicast::cluster):
// `empty` frees a stage in both, `acc_full` hands each CTA's epilogue its
// accumulator. The epilogue warps of both CTAs arrive on the leader's
// `acc_empty` (8 arrivals; the peer's through its cluster address). Tensor
// memory is allocated per CTA, all 512 columns, so both bases are 0. Every wait
// is bounded as elsewhere; both CTAs pass the same two cluster barriers on every
// path, the second one before either frees its tensor memory or exits.

template <int BN>
struct SmemPair {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // All the shared memory a CTA can have (227 KB): the bytes a CTA has on their
  // way from L2, over the latency of that way, is its intake, and the intake is
  // what bounds these kernels.
  static constexpr int BUDGET = 227 * 1024 - 1024 - 256;
  static constexpr int STAGES = BUDGET / STAGE_BYTES > 12 ? 12 : BUDGET / STAGE_BYTES;
  static constexpr int BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256;
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared-memory window, of `local` in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_address(const void* local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(local)), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile load whose completion is counted on a barrier of the CTA pair (its
// address in the cluster window), not necessarily this CTA's own.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, when the MMAs issued so far are complete, on the barrier at this
// shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster)
               : "memory");
}
// mbar_wait for a barrier that the peer CTA arrives on: acquire at cluster scope.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag, int where, int kb) {
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (atomicCAS(&g_status[0], 0, 1) == 0) {
    g_status[1] = where;
    g_status[2] = (int)blockIdx.x;
    g_status[3] = kb;
  }
  return false;
}

constexpr int MAX_TAIL_SHARES = 4;

// One piece of work of a CTA pair: a tile, whole (share < 0) or one share of its K.
struct PairUnit {
  int ta, tb, kb0, kb1, share, tail_tile;
};
__device__ __forceinline__ PairUnit pair_unit(const GemmParams& p, int u, int tiles_a, int nkb) {
  PairUnit w;
  int tile = u;
  w.share = -1; w.tail_tile = 0; w.kb0 = 0; w.kb1 = nkb;
  if (u >= p.full_tiles && p.tail_splits > 1) {
    const int v = u - p.full_tiles;
    w.tail_tile = v / p.tail_splits;
    w.share = v - w.tail_tile * p.tail_splits;
    tile = p.full_tiles + w.tail_tile;
    w.kb0 = w.share * p.tail_kblocks;
    w.kb1 = min(nkb, w.kb0 + p.tail_kblocks);
  }
  w.ta = tile % tiles_a;
  w.tb = tile / tiles_a;
  return w;
}

// tiles_a counts 256-row blocks of A. gridDim.x is even: CTAs 2c and 2c + 1 are
// cluster c, which walks the units c, c + clusters, ... A unit is a whole tile,
// or, for the tiles of the last round when they would leave most pairs idle, one
// of `tail_splits` shares of a tile's K. A share's accumulator goes to the
// float32 workspace; the epilogue warp that delivers a tile's last share (an
// atomic counter per tile, CTA and warp, no waiting) sums the shares in share
// order and runs the usual epilogue on the sum.
template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const GemmParams p, int tiles_a,
                    int tiles_b) {
  constexpr int STAGES = SmemPair<BN>::STAGES;
  constexpr int TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * SmemPair<BN>::STAGE_BYTES);  // used in the leader
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2], used in the leader
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int cluster = (int)(blockIdx.x >> 1), clusters = (int)(gridDim.x >> 1);
  const int nkb = (p.K + BK - 1) / BK;
  const int n_tiles = tiles_a * tiles_b;
  const int total_units =
      p.tail_splits > 1 ? p.full_tiles + (n_tiles - p.full_tiles) * p.tail_splits : n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // the four epilogue warps of both CTAs
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
  cluster_barrier();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t full_leader = cluster_address(&full[0], 0);
      // The first tile's first stages (all empty at the start): the operand that
      // holds constants (weights) is requested before this kernel waits for the
      // one before it, the other operand after.
      const PairUnit first = pair_unit(p, cluster < total_units ? cluster : 0, tiles_a, nkb);
      const int first_kb = first.kb1 - first.kb0;
      const int early = (cluster < total_units) ? (first_kb < STAGES ? first_kb : STAGES) : 0;
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * SmemPair<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + SmemPair<BN>::A_BYTES;
        if (leader) mbar_expect_tx(&full[i], 2 * SmemPair<BN>::STAGE_BYTES);
        const uint32_t bar = full_leader + (uint32_t)(i * 8);
        const int k = (first.kb0 + i) * BK;
        if (p.constant_operand == 1)
          tma_load_2d_pair(a_dst, &map_a, bar, k, first.ta * 2 * BM + (int)rank * BM);
        if (p.constant_operand == 2)
          tma_load_2d_pair(b_dst, &map_b, bar, k, first.tb * BN + (int)rank * (BN / 2));
      }
      fb_pdl_wait();
      for (int i = 0; i < early; ++i) {
        uint8_t* a_dst = tiles + i * SmemPair<BN>::STAGE_BYTES;
        uint8_t* b_dst = a_dst + SmemPair<BN>::A_BYTES;
        const uint32_t bar = full_leader + (uint32_t)(i * 8);
        const int k = (first.kb0 + i) * BK;
        if (p.constant_operand != 1)
          tma_load_2d_pair(a_dst, &map_a, bar, k, first.ta * 2 * BM + (int)rank * BM);
        if (p.constant_operand != 2)
          tma_load_2d_pair(b_dst, &map_b, bar, k, first.tb * BN + (int)rank * (BN / 2));
      }
      int it = 0;
      bool ok = true;
      for (int u = cluster; u < total_units && ok; u += clusters) {
        const PairUnit w = pair_unit(p, u, tiles_a, nkb);
        for (int kb = w.kb0 + (u == cluster ? early : 0); kb < w.kb1; ++kb) {
          const int use = it + (kb - w.kb0);
          const int s = use % STAGES;
          const uint32_t phase = (uint32_t)(use / STAGES) & 1u;
          if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, 1, kb)) { ok = false; break; }
          uint8_t* a_dst = tiles + s * SmemPair<BN>::STAGE_BYTES;
          uint8_t* b_dst = a_dst + SmemPair<BN>::A_BYTES;
          if (leader) mbar_expect_tx(&full[s], 2 * SmemPair<BN>::STAGE_BYTES);
          const uint32_t bar = full_leader + (uint32_t)(s * 8);
          tma_load_2d_pair(a_dst, &map_a, bar, kb * BK, w.ta * 2 * BM + (int)rank * BM);
          tma_load_2d_pair(b_dst, &map_b, bar, kb * BK, w.tb * BN + (int)rank * (BN / 2));
        }
        it += w.kb1 - w.kb0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN);
      int it = 0, j = 0;
      bool ok = true;
      for (int u = cluster; u < total_units && ok; u += clusters, ++j) {
        const PairUnit w = pair_unit(p, u, tiles_a, nkb);
        const int buf = j & 1;
        ok = mbar_wait_cluster(&acc_empty[buf], (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag, 4, j);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          const int use = it + (kb - w.kb0);
          const int s = use % STAGES;
          const uint32_t phase = (uint32_t)(use / STAGES) & 1u;
          ok = mbar_wait_cluster(&full[s], phase, abort_flag, 2, kb);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * SmemPair<BN>::STAGE_BYTES);
          const uint32_t b_addr = a_addr + SmemPair<BN>::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_pair(d_tmem, make_desc(a_addr + k * UMMA_K * 2),
                      make_desc(b_addr + k * UMMA_K * 2), idesc,
                      (kb != w.kb0 || k != 0) ? 1u : 0u);
          tc_commit_pair(&empty[s]);
        }
        if (!ok) break;
        tc_commit_pair(&acc_full[buf]);
        it += w.kb1 - w.kb0;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    float* out_f = (float*)p.out;
    __nv_bfloat16* out_h = (__nv_bfloat16*)p.out;
    constexpr int CHUNK = (BN % 32 == 0) ? 32 : 16;
    const uint32_t acc_empty_leader = cluster_address(&acc_empty[0], 0);
    fb_pdl_wait();
    int j = 0;
    bool ok = true;
    for (int u = cluster; u < total_units && ok; u += clusters, ++j) {
      const PairUnit w = pair_unit(p, u, tiles_a, nkb);
      const int ta = w.ta, tb = w.tb;
      const int buf = j & 1;
      ok = mbar_wait(&acc_full[buf], (uint32_t)((j >> 1) & 1), abort_flag, 3, j);
      if (!ok) break;
      tc_fence_after();
      const int row_in_tile = (int)rank * BM + quarter * 32 + lane;
      const long long i_global = (long long)ta * 2 * BM + row_in_tile;
      // a share's sums go to the workspace instead of the output
      // A share's sums go to the workspace instead of the output. Its layout is this
      // kernel's own: per (tile, share, CTA, warp) a block of BN / 4 groups of 32
      // float4, group g holding columns 4g..4g+3 of the warp's 32 rows, so that a warp
      // writes and later reads 512 contiguous bytes per instruction.
      float4* mine = w.share < 0 ? nullptr
                                 : reinterpret_cast<float4*>(p.partial) +
                                       (((size_t)(w.tail_tile * p.tail_splits + w.share) * 8 +
                                         rank * 4 + quarter) * (BN / 4)) * 32 + lane;
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
        if (mine == nullptr) {
          store_chunk<CHUNK>(p, v, i_global, (long long)tb * BN + c, lane, out_f, out_h);
        } else {
#pragma unroll
          for (int e = 0; e < CHUNK; e += 4)
            mine[(size_t)((c + e) / 4) * 32] = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
      }
      // this warp has read its lanes of the accumulator: tell the leader's MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + (uint32_t)(buf * 8));
      if (mine != nullptr) {
        // publish this warp's 32 rows of the share; the warp that completes the set
        // (the same rows of every share) sums them and stores the result
        __threadfence();
        __syncwarp();
        int before = 0;
        int* counter = p.tail_counters + w.tail_tile * 8 + (int)rank * 4 + quarter;
        if (lane == 0) before = atomicAdd(counter, 1);
        before = __shfl_sync(0xffffffffu, before, 0);
        if (before == p.tail_splits - 1) {
          __threadfence();
          const float4* base = reinterpret_cast<const float4*>(p.partial) +
                               (((size_t)(w.tail_tile * p.tail_splits) * 8 + rank * 4 + quarter) *
                                (BN / 4)) * 32 + lane;
          const size_t share_stride = (size_t)8 * (BN / 4) * 32;  // float4s between shares
#pragma unroll 1
          for (int c = 0; c < BN; c += CHUNK) {
            // all shares' loads of this chunk are issued before the first is used:
            // one warp reads the whole 32 x BN x shares block, and what it has in
            // flight decides how long that takes
            float4 q[MAX_TAIL_SHARES][CHUNK / 4];
#pragma unroll
            for (int sh = 0; sh < MAX_TAIL_SHARES; ++sh) {
              if (sh < p.tail_splits) {
                const float4* src = base + sh * share_stride + (size_t)(c / 4) * 32;
#pragma unroll
                for (int e = 0; e < CHUNK / 4; ++e) q[sh][e] = __ldcg(src + (size_t)e * 32);
              }
            }
            float v[CHUNK];
#pragma unroll
            for (int e = 0; e < CHUNK; ++e) v[e] = 0.f;
#pragma unroll
            for (int sh = 0; sh < MAX_TAIL_SHARES; ++sh) {
              if (sh < p.tail_splits) {
#pragma unroll
                for (int e = 0; e < CHUNK / 4; ++e) {
                  v[4 * e] += q[sh][e].x; v[4 * e + 1] += q[sh][e].y;
                  v[4 * e + 2] += q[sh][e].z; v[4 * e + 3] += q[sh][e].w;
                }
              }
            }
            store_chunk<CHUNK>(p, v, i_global, (long long)tb * BN + c, lane, out_f, out_h);
          }
          if (lane == 0) *counter = 0;  // as the next call expects it
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_barrier();  // nothing of the peer's may still be on its way to this CTA
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------- host: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) ==
            cudaSuccess && res == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    return h * 1000003u ^ (size_t)k.box_rows;
  }
};

// A [rows, cols] bf16 matrix with row stride `ld` elements, fetched in boxes of
// box_rows x 64 elements with the 128-byte swizzle; out-of-range elements read 0.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
             int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return 0;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fb_fail(3, "gemm_tc: cuTensorMapEncodeTiled is not available in this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fb_fail(3, "gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return 0;
}

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
           cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<BN>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
    configured = true;
  }
  fb_launch(gemm_tc_kernel<BN>, dim3(grid), dim3(THREADS), Smem<BN>::BYTES, stream, ma, mb, p);
  return fb_check_launch("gemm_tc");
}

int sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (count <= 0) count = 148;
  }
  return count;
}

template <int BN>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p,
                      int tiles_a, int tiles_b, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<BN>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int total = tiles_a * tiles_b;
  const int ctas = total < sm_count() ? total : sm_count();
  fb_launch(gemm_tc_persistent_kernel<BN>, dim3(ctas), dim3(THREADS), Smem<BN>::BYTES, stream, ma,
            mb, p, tiles_a, tiles_b);
  return fb_check_launch("gemm_tc_persistent");
}

template <int BN>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int tiles_a,
                int tiles_b, void* workspace, long long workspace_bytes, int* counters,
                int counters_len, int share_min_kblocks, cudaStream_t stream) {
  static int clusters_max = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SmemPair<BN>::BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (clusters_max == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SmemPair<BN>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_tc: shared memory opt-in: %s", cudaGetErrorString(e));
    cfg.gridDim = dim3(sm_count() / 2 * 2);
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<BN>, &cfg);
    if (e != cudaSuccess || n <= 0)
      return fb_fail(2, "gemm_tc: no CTA pair of this kernel fits the device (%s)",
                     cudaGetErrorString(e));
    clusters_max = n;
  }
  // Units of work: whole tiles, except that the tiles of a last round that would
  // leave more than half of the pairs idle are shared along K (see the kernel),
  // when a share still has `share_min_kblocks` K blocks: measured at 2,048 rows, a
  // unit costs a few microseconds beside its K loop and the last share's warp
  // adds the sum and the stores, so sharing paid at K = 8,192 in three shares
  // (92.5 -> 78.6 us) and did not at K = 3,072 (16 or 12 blocks a share).
  const int total = tiles_a * tiles_b;
  const int nkb = (p.K + BK - 1) / BK;
  GemmParams q = p;
  q.full_tiles = total;
  q.tail_splits = 1;
  q.tail_kblocks = nkb;
  const int tail = total % clusters_max;
  if (workspace != nullptr && counters != nullptr && total > clusters_max && tail > 0 &&
      2 * tail <= clusters_max) {
    int shares = clusters_max / tail;
    if (shares > MAX_TAIL_SHARES) shares = MAX_TAIL_SHARES;
    if (shares > nkb / share_min_kblocks) shares = nkb / share_min_kblocks;
    if (shares >= 2) {
      const int per = (nkb + shares - 1) / shares;
      shares = (nkb + per - 1) / per;                 // no empty share
      const long long need = (long long)tail * shares * (2 * BM) * BN * 4;
      if (shares >= 2 && need <= workspace_bytes && tail * 8 <= counters_len) {
        q.full_tiles = total - tail;
        q.tail_splits = shares;
        q.tail_kblocks = per;
        q.partial = (float*)workspace;
        q.tail_counters = counters;
      }
    }
  }
  const int units = q.full_tiles + (total - q.full_tiles) * q.tail_splits;
  const int clusters = units < clusters_max ? units : clusters_max;
  cfg.gridDim = dim3(2 * clusters);
  cfg.numAttrs = g_fb_pdl ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN>, ma, mb, q, tiles_a, tiles_b);
  return fb_check_launch("gemm_tc_pair");
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
// epilogue 1 fuses SiLU(gate) * up: the feature operand's rows are (gate, up)
// pairs and `out` is [tokens, features / 2] bf16; the stride of the feature
// dimension must be 1 and then indexes pairs.
FB_API int fb_gemm_tc(const void* a, long long lda, int rows_a, const void* b, long long ldb,
                      int rows_b, int K, void* out, long long stride_a, long long stride_b,
                      int out_f32, int bn, int splits, long long split_stride, int epilogue,
                      int constant_operand, int persistent, void* workspace,
                      long long workspace_bytes, int* counters, int counters_len,
                      int share_min_kblocks, cudaStream_t stream) {
  FB_REQUIRE(rows_a > 0 && rows_b > 0 && K > 0, "gemm_tc: bad sizes %d x %d x %d", rows_a, rows_b, K);
  FB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0,
             "gemm_tc: K and the row strides must be multiples of 8 elements (16 bytes), got K=%d "
             "lda=%lld ldb=%lld", K, lda, ldb);
  FB_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0,
             "gemm_tc: operands must start on 16-byte boundaries");
  FB_REQUIRE(splits >= 1 && (splits == 1 || out_f32), "gemm_tc: split-K needs a float32 output");
  FB_REQUIRE(epilogue == 0 || (epilogue == 1 && splits == 1 && !out_f32 &&
                               (stride_a == 1 || stride_b == 1)),
             "gemm_tc: the SiLU-mul epilogue needs one split, a bf16 output and features on a "
             "unit stride");
  const int total_kb = (K + BK - 1) / BK;
  FB_REQUIRE(splits <= total_kb, "gemm_tc: %d splits for %d K blocks", splits, total_kb);
  GemmParams p;
  p.rows_a = rows_a; p.rows_b = rows_b; p.K = K;
  p.kblocks_per_split = (total_kb + splits - 1) / splits;
  p.stride_a = stride_a; p.stride_b = stride_b; p.split_stride = split_stride;
  p.out = out; p.out_f32 = out_f32; p.epilogue = epilogue;
  p.constant_operand = constant_operand;
  p.full_tiles = 0; p.tail_splits = 1; p.tail_kblocks = total_kb; p.partial = nullptr;
  p.tail_counters = nullptr;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, rows_a, K, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, rows_b, K, ldb, bn);
  if (rc) return rc;
  dim3 grid((rows_a + BM - 1) / BM, (rows_b + bn - 1) / bn, splits);
  FB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
  if (persistent == 2) {
    // two SMs per tile: A in blocks of 256 rows, each CTA loads half of a B tile
    FB_REQUIRE(splits == 1, "gemm_tc: the paired form takes one split");
    const int share_min = share_min_kblocks > 0 ? share_min_kblocks : 32;
    rc = make_map(&mb, b, rows_b, K, ldb, bn / 2);
    if (rc) return rc;
    const int pairs_a = (rows_a + 2 * BM - 1) / (2 * BM);
    switch (bn) {
      case 128: return launch_pair<128>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 144: return launch_pair<144>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 160: return launch_pair<160>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 176: return launch_pair<176>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 192: return launch_pair<192>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 208: return launch_pair<208>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 224: return launch_pair<224>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 240: return launch_pair<240>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      case 256: return launch_pair<256>(ma, mb, p, pairs_a, grid.y, workspace, workspace_bytes, counters, counters_len, share_min, stream);
      default:
        return fb_fail(1, "gemm_tc: the paired form takes tiles 128..256 (steps of 16) wide, "
                          "not %d", bn);
    }
  }
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

// How many CTA pairs of the paired product (256-wide tiles) the device runs at
// once: the number of tiles of one round. <= 0 on failure (see fb_last_error).
FB_API int fb_gemm_tc_pair_slots() {
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SmemPair<256>::BYTES;
  cfg.gridDim = dim3(sm_count() / 2 * 2);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<256>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SmemPair<256>::BYTES);
  int n = 0;
  if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<256>, &cfg);
  if (e != cudaSuccess) return -fb_fail(2, "gemm_tc_pair_slots: %s", cudaGetErrorString(e));
  return n;
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
