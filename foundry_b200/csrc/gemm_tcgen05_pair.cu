// The tcgen05 product with two SMs on one tile (cta_group::2); the one-CTA forms
// and the entry point `fb_gemm_tc` are in gemm_tcgen05.cu.
#define FB_STATUS_KERNEL 2
#include "gemm_tcgen05.cuh"

namespace {

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
  record_failure(where, (int)blockIdx.x, kb);
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
      const float scale = token_scale(p, i_global);
      float ss = 0.f;
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
          ss += finish_chunk<CHUNK>(p, v, scale, i_global, (long long)tb * BN + c, lane, out_f, out_h);
        } else {
#pragma unroll
          for (int e = 0; e < CHUNK; e += 4)
            mine[(size_t)((c + e) / 4) * 32] = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
      }
      if (mine == nullptr) finish_tile(p, ss, i_global, tb);
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
            ss += finish_chunk<CHUNK>(p, v, scale, i_global, (long long)tb * BN + c, lane, out_f, out_h);
          }
          finish_tile(p, ss, i_global, tb);
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

template <int BN>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int tiles_a,
                int tiles_b, void* workspace, long long workspace_bytes, int* counters,
                int counters_len, int share_min_kblocks, cudaStream_t stream) {
  static int clusters_of_device[64] = {};  // CTA pairs that run at once, per device
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) device = 63;
  int& clusters_max = clusters_of_device[device];
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
  // and did not at K = 3,072 (16 or 12 blocks a share).
  const int total = tiles_a * tiles_b;
  const int nkb = (p.K + BK - 1) / BK;
  GemmParams q = p;
  q.full_tiles = total;
  q.tail_splits = 1;
  q.tail_kblocks = nkb;
  // tiles of the last round (all tiles, when there are fewer than pairs) and the K
  // blocks a share must keep: half as many when the pairs would otherwise idle for
  // the whole call, not only for its last round
  const int tail = total % clusters_max;
  const bool few = total < clusters_max;
  const int min_kblocks = few ? (share_min_kblocks + 1) / 2 : share_min_kblocks;
  if (workspace != nullptr && counters != nullptr && tail > 0 && 2 * tail <= clusters_max) {
    int shares = clusters_max / tail;
    if (shares > MAX_TAIL_SHARES) shares = MAX_TAIL_SHARES;
    if (shares > nkb / min_kblocks) shares = nkb / min_kblocks;
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

// a, b as in fb_gemm_tc; `p` filled by it. A in blocks of 256 rows, each CTA of a
// pair loads half of a B tile (bn / 2 rows).
int fb_gemm_tc_pair(const void* a, long long lda, int rows_a, const void* b, long long ldb,
                    int rows_b, int bn, const FbGemmParams& p, void* workspace,
                    long long workspace_bytes, int* counters, int counters_len,
                    int share_min_kblocks, cudaStream_t stream) {
  bind_status_mirror(stream);
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, rows_a, p.K, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, rows_b, p.K, ldb, bn / 2);
  if (rc) return rc;
  const int share_min = share_min_kblocks > 0 ? share_min_kblocks : 32;
  const int pairs_a = (rows_a + 2 * BM - 1) / (2 * BM);
  const int tiles_b = (rows_b + bn - 1) / bn;
  switch (bn) {
#define FB_PAIR_CASE(N)                                                                        \
    case N:                                                                                    \
      return launch_pair<N>(ma, mb, p, pairs_a, tiles_b, workspace, workspace_bytes, counters, \
                            counters_len, share_min, stream);
    FB_PAIR_CASE(128) FB_PAIR_CASE(144) FB_PAIR_CASE(160) FB_PAIR_CASE(176) FB_PAIR_CASE(192)
    FB_PAIR_CASE(208) FB_PAIR_CASE(224) FB_PAIR_CASE(240) FB_PAIR_CASE(256)
#undef FB_PAIR_CASE
    default:
      return fb_fail(1, "gemm_tc: the paired form takes tiles 128..256 (steps of 16) wide, "
                        "not %d", bn);
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

// As fb_gemm_tc_status, for the kernels of this file.
FB_API int fb_gemm_tc_pair_status(int* detail) {
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, g_status, sizeof(host));
  if (e != cudaSuccess) return fb_fail(2, "gemm_tc_pair_status: %s", cudaGetErrorString(e));
  if (detail) { detail[0] = host[1]; detail[1] = host[2]; detail[2] = host[3]; }
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  return host[0] ? host[1] : 0;
}
