// The product y = x W^T for 17 to 256 token rows on the 5th-generation tensor
// cores: the weights stream through once, in the orientation that keeps the
// 128-row operand full (A = 128 weight rows, B = the tokens, N = 32 .. 256),
// and the step's other work rides on the product's epilogue as it does in the
// weight-streaming kernel for up to 16 rows (gemm_skinny.cu).
//
// A product of few weight tiles cannot keep 148 SMs busy with one CTA per
// tile, so K is shared: the S CTAs of a tile each stream 1/S of its K blocks,
// and they are one thread-block cluster. When their accumulators are complete
// every CTA puts its float32 partial tile into its own shared memory (where
// the operand stages were), the cluster meets at a hardware barrier, and every
// CTA then sums, for its own share of the TOKENS, the S partial tiles out of
// its peers' shared memory (distributed shared memory), in the order of the
// CTAs' ranks, and runs the epilogue for those tokens. No workspace in global
// memory, no counters, no CTA spins on another; a second cluster barrier keeps
// every CTA's shared memory alive until its peers have read it.
// (A first form of this kernel cut the (tile, K block) units evenly over the SMs
// and let the CTA that arrived last at a tile sum the others' partial tiles
// from a workspace: perfectly balanced, and 8 to 12 us a call slower, because
// that one CTA walked 6 to 12 partial tiles through L2 one round trip after
// another.)
//
// Roles: warp 0 issues TMA loads (one lane); warp 1 owns tensor memory and
// issues tcgen05.mma (one lane); warps 2-5 read the accumulator with
// tcgen05.ld. A thread of the epilogue owns one weight row (feature) and holds
// that feature's value for its tokens; for a given token the lanes of a warp
// are 32 consecutive features, which is what every store below relies on.
//
// Epilogues (formulas with the reference's lines in gemm_skinny.cu, rope_cache.cu):
//   0  out[token, feature] (bfloat16 or float32)
//   1  weight rows are (gate, up) pairs: out[token, f] = SiLU(gate) * up
//   2  in front of a norm: resid[token, feature] += y (float32), xg = bf16(resid *
//      gamma[feature]), and this tile's share of every token's sum of squares
//   3  the fused q/k/v projection: rotate query and key heads by the token's
//      position (pairs of ADJACENT features, frequency i for features 2i, 2i+1),
//      queries to q_out, keys and values into the token's cache page
// and, for a product whose input is a norm's output that still lacks its row
// scale, every token's results are multiplied by 1 / sqrt(mean square + eps).
//
// Shared memory stays near 100 KB for up to 128 tokens, so that the CTAs of the
// next kernel in the stream find room on the SMs while this kernel's epilogues
// run: every CTA lets them be placed (griddepcontrol.launch_dependents) once its
// last load is issued, and they request their weights before they wait for
// this kernel's results.
//
// Every mbarrier wait is bounded as in the other tcgen05 kernels; a CTA whose
// wait ran out still passes both cluster barriers, so its peers never hang.
#define FB_STATUS_KERNEL 4
#include "gemm_tcgen05.cuh"

namespace {

constexpr int A_BYTES = BM * BK * 2;  // a stage's weight tile

struct RowsScale {      // the input's row scale: see `RowScale` in gemm_skinny.cu
  const float* ss;      // [count, stride] shares of the tokens' sums of squares; null: none
  int count, stride;
  float inv_dim, eps;
};
struct RowsSink {       // epilogue 2
  float* resid;         // [M, N] float32, row stride ldr
  long long ldr;
  const float* gamma;   // [N]
  __nv_bfloat16* xg;    // [M, N], row stride ldxg
  long long ldxg;
  float* ss_out;        // [tiles, ss_stride]
  int ss_stride;
};
struct RowsRope {       // epilogue 3
  const int* positions;     // [M]
  const int* seq_of_token;  // [M], -1 = padding
  const int* page_table;    // [n_seqs, max_pages]
  int max_pages;
  const float* inv_freq;    // [rotary_dim / 2]
  int rotary_dim;
  __nv_bfloat16* q_out;     // [M, A * D], row stride q_stride
  long long q_stride;
  __nv_bfloat16* k_cache;   // pages [*, Kh, FB_PAGE, D]
  __nv_bfloat16* v_cache;
  long long page_stride, head_stride;
  int ring_pages;
  int A, Kh, D;
};
struct RowsParams {
  int M, N, K;
  int kblocks;          // K blocks of 64
  int splits;           // CTAs per weight tile = cluster size (1: no cluster)
  int per;              // K blocks per CTA
  int cols_per;         // tokens each CTA of a cluster finishes
  void* out;
  long long ldo;
  int out_f32;
  int epilogue;
  int vector_ok;        // the epilogue's rows are aligned for 16- and 8-byte accesses
  RowsScale scale;
  RowsSink sink;
  RowsRope rope;
};

template <int NB> struct RowsCfg {
  static constexpr int B_BYTES = NB * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // near 100 KB up to 128 tokens (two kernels' CTAs share an SM); one CTA per SM beyond
  static constexpr int STAGES = NB <= 32 ? 5 : NB <= 64 ? 4 : NB <= 128 ? 3 : 4;
  static constexpr int TMEM_COLS = NB < 32 ? 32 : NB;
  // barriers and flags, the tokens' scales, positions and cache rows
  static constexpr int TAIL_BYTES = 256 + NB * (4 + 4 + 8);
  static constexpr int BYTES = STAGES * STAGE_BYTES + 1024 + TAIL_BYTES;
  static_assert(STAGES * STAGE_BYTES >= NB * BM * 4 + 32 * BM * 4,
                "the partial tile and the epilogue's turn table take the stages' place");
};

__device__ __forceinline__ void epi_barrier() {  // the four epilogue warps
  asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A float of the CTA of rank `rank` in this cluster, at the address `mine` has here.
__device__ __forceinline__ float ld_cluster(const float* mine, unsigned rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(mine)), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
  return v;
}

template <int NB, bool CLUSTER, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const RowsParams p) {
  using Cfg = RowsCfg<NB>;
  constexpr int STAGES = Cfg::STAGES;
  // The epilogue is a template parameter: with all four in one kernel the
  // epilogue's straight-line code did not fit the instruction cache and every
  // token's stores waited for instructions (1.1 instead of 0.6 us per 32 tokens).
  constexpr int epi = EPI;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* s_scale = (float*)(tiles + STAGES * Cfg::STAGE_BYTES + 256);  // [NB]
  int* s_pos = (int*)(s_scale + NB);                                    // [NB]
  long long* s_row = (long long*)(s_pos + NB);                          // [NB] cache row offset, -1: none
  float* partial = (float*)tiles;  // [NB][128] once the products are through
  float* turn = partial + NB * BM;  // [32 tokens][128 weight rows]: the epilogue's turn table

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int split = CLUSTER ? (int)blockIdx.z : 0;  // = the CTA's rank in its cluster
  const int kb0 = split * p.per;
  const int n = max(min(p.kblocks - kb0, p.per), 0);

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
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int quarter = warp & 3;             // the TMEM lanes an epilogue warp may read
  const int row = quarter * 32 + lane;      // an epilogue thread's weight row within the tile
  const int et = (int)threadIdx.x - 64;     // 0..127 among the epilogue threads
  bool acc_ok = false;                      // epilogue warps: the accumulator arrived

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the weights are constants: the first stages' weight tiles are requested
      // before the wait for the kernel that produces x
      const int early = n < STAGES ? n : STAGES;
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&full[i], Cfg::STAGE_BYTES);
        tma_load_2d(tiles + i * Cfg::STAGE_BYTES, &map_w, &full[i], (kb0 + i) * BK, tile * BM);
      }
      fb_pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(tiles + i * Cfg::STAGE_BYTES + A_BYTES, &map_x, &full[i], (kb0 + i) * BK, 0);
      for (int i = early; i < n; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, 1, i)) break;
        uint8_t* dst = tiles + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
        tma_load_2d(dst, &map_w, &full[s], (kb0 + i) * BK, tile * BM);
        tma_load_2d(dst + A_BYTES, &map_x, &full[s], (kb0 + i) * BK, 0);
      }
      // every load of this CTA is on its way: the next kernel's blocks may be placed
      fb_pdl_launch();
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, NB);
      bool ok = true;
      for (int i = 0; i < n && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(&full[s], phase, abort_flag, 2, i);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * Cfg::STAGE_BYTES);
        const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma(tmem_base, make_desc(a_addr + k * UMMA_K * 2), make_desc(b_addr + k * UMMA_K * 2),
               idesc, (i | k) != 0 ? 1u : 0u);
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    // ------------------------------------------------- epilogue, first part
    fb_pdl_wait();
    // per-token values that the epilogue uses
    for (int j = et; j < NB; j += 128) {
      float sc = 1.f;
      if (p.scale.ss != nullptr && j < p.M) {
        float sum = 0.f;
        for (int c = 0; c < p.scale.count; ++c) sum += __ldcg(p.scale.ss + (size_t)c * p.scale.stride + j);
        sc = 1.0f / sqrtf(sum * p.scale.inv_dim + p.scale.eps);
      }
      s_scale[j] = sc;
      if (epi == 3) {
        int pos = 0;
        long long off = -1;
        if (j < p.M) {
          const int seq = p.rope.seq_of_token[j];
          pos = p.rope.positions[j];
          if (seq >= 0 && p.rope.k_cache != nullptr) {
            int lp = pos / FB_PAGE;
            if (p.rope.ring_pages > 0) lp %= p.rope.ring_pages;
            off = (long long)p.rope.page_table[(size_t)seq * p.rope.max_pages + lp] * p.rope.page_stride +
                  (long long)(pos % FB_PAGE) * p.rope.D;
          } else if (seq >= 0) {
            off = 0;  // queries only
          }
        }
        s_pos[j] = pos;
        s_row[j] = off;
      }
    }
    acc_ok = n > 0 ? mbar_wait(acc_full, 0, abort_flag, 3, 0) : true;
    tc_fence_after();
    if (CLUSTER) {
      // this CTA's partial tile, [token][weight row], where the stages were: every
      // product has read them by now
#pragma unroll 1
      for (int c0 = 0; c0 < NB; c0 += 32) {
        uint32_t r[32];
        if (acc_ok && n > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) partial[(c0 + e) * BM + row] = __uint_as_float(r[e]);
      }
    }
  }
  __syncwarp();
  if (CLUSTER) cluster_barrier();  // every CTA's partial tile is in place (all threads)

  if (warp >= 2) {
    // ------------------------------------------------ epilogue, second part
    // A thread holds its weight row's values for 32 tokens. Stored from there, a
    // warp's store instruction covers 32 neighbouring features of ONE token, 64
    // bytes, and a tile of 128 tokens took 10 us longer than it streamed. So
    // the values take a turn through shared memory: written [token][weight row],
    // read back by a warp per token with four neighbouring features per lane,
    // and every global access below is a 16- or 8-byte piece of a 256- or
    // 512-byte run.
    epi_barrier();  // s_scale and its companions are written
    const int ewarp = et >> 5;  // 0..3
    // the tokens this CTA finishes
    const int j_begin = CLUSTER ? min(p.M, split * p.cols_per) : 0;
    const int j_end = CLUSTER ? min(p.M, j_begin + p.cols_per) : p.M;
    const long long f0 = (long long)tile * BM + 4 * lane;  // this lane's four features
    const int live = (int)max(0LL, min(4LL, (long long)p.N - f0));  // how many of them exist
    // rotary epilogue: this lane's two pairs
    const RowsRope& rw = p.rope;
    int head = 0, el = 0, kind = 0;
    float freq[2] = {0.f, 0.f};
    bool rotated = false;
    if (epi == 3 && live > 0) {
      head = (int)(f0 / rw.D);
      el = (int)(f0 - (long long)head * rw.D);
      kind = head < rw.A ? 0 : head < rw.A + rw.Kh ? 1 : 2;
      rotated = kind < 2 && el < rw.rotary_dim;  // rotary_dim and D are multiples of 4 here
      if (rotated) { freq[0] = rw.inv_freq[el >> 1]; freq[1] = rw.inv_freq[(el >> 1) + 1]; }
    }
    float gamma[4] = {0.f, 0.f, 0.f, 0.f};
    if (epi == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) if (q < live) gamma[q] = p.sink.gamma[f0 + q];
    }
    const bool vec = live == 4 && p.vector_ok;  // else element by element
#pragma unroll 1
    for (int c0 = j_begin; c0 < j_end; c0 += 32) {
      float v[32];
      if (CLUSTER) {
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = 0.f;
        // Summed in the order of the ranks. The loads of four ranks for sixteen
        // tokens go out together before the first is added: a warp issues in
        // order, so a load followed by its own add waits out the whole trip to
        // the other SM (0.6 us), once per load.
#pragma unroll
        for (int h = 0; h < 32; h += 16) {
          if (c0 + h >= j_end) break;
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float t[4][16];
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int e = 0; e < 16; ++e)
                t[q][e] = (s0 + q < p.splits && c0 + h + e < j_end)
                              ? ld_cluster(partial + (c0 + h + e) * BM + row, (unsigned)(s0 + q)) : 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int e = 0; e < 16; ++e) v[h + e] += t[q][e];
          }
        }
      } else {
        uint32_t r[32];
        if (acc_ok && n > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
      }
#pragma unroll
#pragma unroll
      for (int e = 0; e < 32; ++e) turn[e * BM + row] = v[e];
      epi_barrier();
      // a warp per token: tokens c0 + ewarp, c0 + ewarp + 4, ...
      // (a scheduler has one epilogue warp and nothing to hide a token's chain of
      // dependent instructions behind: the eight tokens of a warp are unrolled)
      float4 ys[8];
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int e = ewarp + 4 * it;
        const float sc = s_scale[min(c0 + e, NB - 1)];
        ys[it] = *reinterpret_cast<const float4*>(turn + e * BM + 4 * lane);
        ys[it].x *= sc; ys[it].y *= sc; ys[it].z *= sc; ys[it].w *= sc;
      }
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int e = ewarp + 4 * it;
        const int j = c0 + e;
        if (j >= j_end) continue;
        const float4 y = ys[it];
        float val[4] = {y.x, y.y, y.z, y.w};
        if (epi == 0) {
          if (p.out_f32) {
            float* dst = (float*)p.out + (long long)j * p.ldo + f0;
            if (vec) *reinterpret_cast<float4*>(dst) = y;
            else {
#pragma unroll
              for (int q = 0; q < 4; ++q) if (q < live) dst[q] = val[q];
            }
          } else {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (long long)j * p.ldo + f0;
            if (vec) {
              const __nv_bfloat162 lo = __floats2bfloat162_rn(val[0], val[1]);
              const __nv_bfloat162 hi = __floats2bfloat162_rn(val[2], val[3]);
              uint2 pk;
              pk.x = *reinterpret_cast<const uint32_t*>(&lo);
              pk.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(dst) = pk;
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) if (q < live) dst[q] = __float2bfloat16_rn(val[q]);
            }
          }
        } else if (epi == 1) {
          // (gate, up) pairs: two results per lane
          __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (long long)j * p.ldo + (f0 >> 1);
          const float h0 = val[0] / (1.0f + __expf(-val[0])) * val[1];
          const float h1 = val[2] / (1.0f + __expf(-val[2])) * val[3];
          if (vec) {
            const __nv_bfloat162 pk = __floats2bfloat162_rn(h0, h1);
            *reinterpret_cast<__nv_bfloat162*>(dst) = pk;
          } else {
            if (live >= 2) dst[0] = __float2bfloat16_rn(h0);
            if (live >= 4) dst[1] = __float2bfloat16_rn(h1);
          }
        } else if (epi == 2) {
          float* rp = p.sink.resid + (long long)j * p.sink.ldr + f0;
          __nv_bfloat16* xp = p.sink.xg + (long long)j * p.sink.ldxg + f0;
          float r[4] = {0.f, 0.f, 0.f, 0.f};
          if (vec) {
            const float4 old = __ldcg(reinterpret_cast<const float4*>(rp));
            r[0] = old.x + val[0]; r[1] = old.y + val[1]; r[2] = old.z + val[2]; r[3] = old.w + val[3];
            *reinterpret_cast<float4*>(rp) = make_float4(r[0], r[1], r[2], r[3]);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0] * gamma[0], r[1] * gamma[1]);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(r[2] * gamma[2], r[3] * gamma[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(xp) = pk;
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (q < live) {
                r[q] = __ldcg(rp + q) + val[q];
                rp[q] = r[q];
                xp[q] = __float2bfloat16_rn(r[q] * gamma[q]);
              }
            }
          }
          // this tile's share of the token's sum of squares, in a fixed order
          float sq = (r[0] * r[0] + r[1] * r[1]) + (r[2] * r[2] + r[3] * r[3]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
          if (lane == 0) p.sink.ss_out[(size_t)tile * p.sink.ss_stride + j] = sq;
        } else {
          const long long off = s_row[j];
          if (live > 0 && off >= 0) {
            if (rotated) {
              const float fpos = (float)s_pos[j];
#pragma unroll
              for (int q = 0; q < 2; ++q) {  // features 2q, 2q + 1 of the four turn by freq[q]
                float sn, cs;
                sincosf(fpos * freq[q], &sn, &cs);
                const float a = val[2 * q], b = val[2 * q + 1];
                val[2 * q] = a * cs - b * sn;
                val[2 * q + 1] = b * cs + a * sn;
              }
            }
            __nv_bfloat16* dst;
            if (kind == 0) dst = rw.q_out + (long long)j * rw.q_stride + (long long)head * rw.D + el;
            else dst = (kind == 1 ? rw.k_cache + (long long)(head - rw.A) * rw.head_stride
                                  : rw.v_cache + (long long)(head - rw.A - rw.Kh) * rw.head_stride) + off + el;
            const __nv_bfloat162 lo = __floats2bfloat162_rn(val[0], val[1]);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(val[2], val[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = pk;
          }
        }
      }
      epi_barrier();  // the turn table is rewritten by the next 32 tokens
    }
  }
  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (CLUSTER) cluster_barrier();  // the peers have read this CTA's partial tile
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
  }
}

template <int NB, int EPI>
int launch_rows_as(const CUtensorMap& mw, const CUtensorMap& mx, const RowsParams& p, int tiles,
                   cudaStream_t stream) {
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rows_kernel<NB, true, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         RowsCfg<NB>::BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_rows_kernel<NB, false, EPI>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, RowsCfg<NB>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "gemm_rows: shared memory opt-in: %s", cudaGetErrorString(e));
  }
  if (p.splits > 1)
    fb_launch_cluster(gemm_rows_kernel<NB, true, EPI>, dim3(tiles, 1, p.splits), dim3(THREADS),
                      RowsCfg<NB>::BYTES, stream, (unsigned)p.splits, mw, mx, p);
  else
    fb_launch(gemm_rows_kernel<NB, false, EPI>, dim3(tiles), dim3(THREADS), RowsCfg<NB>::BYTES,
              stream, mw, mx, p);
  return fb_check_launch("gemm_rows");
}

template <int NB>
int launch_rows(const CUtensorMap& mw, const CUtensorMap& mx, const RowsParams& p, int tiles,
                cudaStream_t stream) {
  switch (p.epilogue) {
    case 0: return launch_rows_as<NB, 0>(mw, mx, p, tiles, stream);
    case 1: return launch_rows_as<NB, 1>(mw, mx, p, tiles, stream);
    case 2: return launch_rows_as<NB, 2>(mw, mx, p, tiles, stream);
    default: return launch_rows_as<NB, 3>(mw, mx, p, tiles, stream);
  }
}

}  // namespace

// CTAs per weight tile (the cluster size) for a product of N weight rows and K:
// as many as keep all CTAs on the SMs at once, at most 8 (the portable cluster
// size), every CTA keeping at least two K blocks.
FB_API int fb_gemm_rows_splits(int N, int K) {
  const int tiles = (N + BM - 1) / BM, kblocks = (K + BK - 1) / BK;
  int splits = sm_count() / (tiles > 0 ? tiles : 1);
  if (splits > 8) splits = 8;
  if (splits > kblocks / 2) splits = kblocks / 2;
  if (splits < 1) splits = 1;
  const int per = (kblocks + splits - 1) / splits;
  return (kblocks + per - 1) / per;  // no CTA without a K block
}

// out = x W^T with the epilogue named; see the head of the file.
//   x: [M, K] bf16, row stride ldx, 17 <= M <= 256 (fewer work, at the cost of a
//      mostly empty tile); w: [N, K] bf16, row stride ldw
//   epilogue 0: out [M, N] (float32 when out_f32), row stride ldo
//   epilogue 1: out [M, N / 2] bf16
//   epilogue 2: resid / gamma / xg / ss_out as in fb_gemm_skinny_residual; ss_out is
//      [ceil(N / 128), ss_stride] with ss_stride >= M
//   epilogue 3: the arguments of fb_gemm_skinny_rope; the rotation pairs adjacent
//      features, so the caller's weight rows must be laid out that way
//   scale_*: the input's row scale (scale_ss null: none)
//   splits: CTAs per weight tile, 1 to 8 (0: fb_gemm_rows_splits' choice)
FB_API int fb_gemm_rows(const void* x, long long ldx, int M, const void* w, long long ldw, int N,
                        int K, void* out, long long ldo, int out_f32, int epilogue,
                        const float* scale_ss, int scale_count, int scale_stride, int scale_dim,
                        float scale_eps, float* resid, long long ldr, const float* gamma,
                        void* xg, long long ldxg, float* ss_out, int ss_stride,
                        const int* positions, const int* seq_of_token, const int* page_table,
                        int max_pages, const float* inv_freq, int rotary_dim, void* q_out,
                        long long q_stride, void* k_cache, void* v_cache, long long page_stride,
                        long long head_stride, int ring_pages, int A, int Kh, int D, int splits,
                        cudaStream_t stream) {
  FB_REQUIRE(M > 0 && M <= 256 && N > 0 && K > 0, "gemm_rows: bad sizes %d x %d x %d", M, N, K);
  FB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)x % 16) == 0 &&
                 ((uintptr_t)w % 16) == 0,
             "gemm_rows: K and the row strides must be multiples of 8 elements and the operands "
             "16-byte aligned (K=%d ldx=%lld ldw=%lld)", K, ldx, ldw);
  FB_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_rows: unknown epilogue %d", epilogue);
  RowsParams p{};
  p.M = M; p.N = N; p.K = K;
  const int tiles = (N + BM - 1) / BM;
  p.kblocks = (K + BK - 1) / BK;
  if (splits <= 0) splits = fb_gemm_rows_splits(N, K);
  FB_REQUIRE(splits <= 8 && splits <= p.kblocks, "gemm_rows: %d CTAs per tile for %d K blocks "
             "(at most 8)", splits, p.kblocks);
  p.per = (p.kblocks + splits - 1) / splits;
  p.splits = (p.kblocks + p.per - 1) / p.per;
  p.cols_per = (M + p.splits - 1) / p.splits;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32; p.epilogue = epilogue;
  p.scale = RowsScale{scale_ss, scale_count, scale_stride,
                      scale_dim > 0 ? 1.0f / (float)scale_dim : 0.f, scale_eps};
  const int NB = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  if (epilogue <= 1) {
    FB_REQUIRE(out != nullptr && (epilogue == 0 || (!out_f32 && N % 2 == 0)),
               "gemm_rows: the SiLU-mul epilogue writes bfloat16 pairs");
    p.vector_ok = ldo % 4 == 0 && ((uintptr_t)out % 16) == 0;
  } else if (epilogue == 2) {
    FB_REQUIRE(resid && gamma && xg && ss_out && ss_stride >= M && ldr >= N && ldxg >= N,
               "gemm_rows: the residual epilogue lacks an argument or a stride is too small");
    p.vector_ok = ldr % 4 == 0 && ldxg % 4 == 0 && ((uintptr_t)resid % 16) == 0 &&
                  ((uintptr_t)xg % 8) == 0;
    p.sink = RowsSink{resid, ldr, gamma, (__nv_bfloat16*)xg, ldxg, ss_out, ss_stride};
  } else {
    FB_REQUIRE(A > 0 && Kh > 0 && D > 0 && D % 4 == 0 && rotary_dim >= 0 && rotary_dim <= D &&
                   rotary_dim % 4 == 0,
               "gemm_rows: head size %d and rotary width %d must be multiples of 4 (A=%d Kh=%d)",
               D, rotary_dim, A, Kh);
    FB_REQUIRE(q_stride % 4 == 0 && ((uintptr_t)q_out % 8) == 0 &&
                   (k_cache == nullptr || (page_stride % 4 == 0 && head_stride % 4 == 0 &&
                                           ((uintptr_t)k_cache % 8) == 0 && ((uintptr_t)v_cache % 8) == 0)),
               "gemm_rows: queries and cache rows must keep 8-byte alignment");
    const bool cache = k_cache != nullptr;
    FB_REQUIRE(N == (cache ? A + 2 * Kh : A) * D, "gemm_rows: %d weight rows for %d heads of %d", N,
               cache ? A + 2 * Kh : A, D);
    FB_REQUIRE(positions && seq_of_token && q_out && q_stride >= (long long)A * D &&
                   (!cache || (v_cache && page_table && max_pages > 0)) &&
                   (rotary_dim == 0 || inv_freq),
               "gemm_rows: the rotary epilogue lacks an argument");
    p.rope = RowsRope{positions, seq_of_token, page_table, max_pages, inv_freq, rotary_dim,
                      (__nv_bfloat16*)q_out, q_stride, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, page_stride, head_stride, ring_pages, A, Kh, D};
    p.vector_ok = 1;
  }
  bind_status_mirror(stream);
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, N, K, ldw, BM);
  if (rc) return rc;
  rc = make_map(&mx, x, M, K, ldx, NB);
  if (rc) return rc;
  switch (NB) {
    case 32: return launch_rows<32>(mw, mx, p, tiles, stream);
    case 64: return launch_rows<64>(mw, mx, p, tiles, stream);
    case 128: return launch_rows<128>(mw, mx, p, tiles, stream);
    default: return launch_rows<256>(mw, mx, p, tiles, stream);
  }
}

// As fb_gemm_tc_status, for the kernel of this file.
FB_API int fb_gemm_rows_status(int* detail) {
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, g_status, sizeof(host));
  if (e != cudaSuccess) return fb_fail(2, "gemm_rows_status: %s", cudaGetErrorString(e));
  if (detail) { detail[0] = host[1]; detail[1] = host[2]; detail[2] = host[3]; }
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  return host[0] ? host[1] : 0;
}
