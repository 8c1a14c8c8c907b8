// bfloat16 attention over the paged cache on the tensor cores, two kernels:
//
//   prefill   a 64-row block of one sequence's queries for one head walks the
//             sequence's pages (64 keys each) with an online softmax; the four
//             warps own 16 query rows each.
//   decode    one new token per sequence: the G query heads that share a
//             key-value head are one tile. With G <= 8 the keys are the 16 rows
//             of the instruction and the heads its 8 columns (S^T = K Q^T,
//             O^T = V^T P^T); with more, the heads are a 16-row tile (rows >= G
//             padding). Each of the four warps streams its own 16 keys of every
//             page into its own buffers and waits for no other warp; the cache
//             range is split over CTAs, up to eight of which merge inside a
//             thread-block cluster; what is left meets in a workspace, where the
//             CTA that delivers a pair's last result merges (it learns that it
//             is the last from an atomic counter; nobody waits for anybody).
//
// Formulas are the reference's (src/nn/attention.rs:23-60: head a reads kv head
// a / G; src/models/llama/attention.rs:56-58: scale 1/sqrt(D);
// src/nn/masking.rs:76-92: key j visible iff j <= query position;
// src/nn/activation.rs:30-40: softmax with the maximum subtracted). Scores,
// softmax statistics and the output accumulate in 32-bit; probabilities are
// rounded to bfloat16 only as the operand of the P.V product. The reference
// materialises [S, L] scores; nothing of that size exists here.
//
// Pages arrive in shared memory by cp.async (16-byte pieces, XOR-swizzled so
// that ldmatrix is conflict-free), two or three buffers deep. Head sizes 16, 32, 64 and
// 128 are built; other sizes, windows and more than 16 query heads per kv head
// are served by the CUDA-core kernel (attention_simt.cu).
#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

// ------------------------------------------------------------- small PTX faces
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}
// Transposes an 8 x 8 matrix of 16-bit elements held one row per four lanes.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Shared-memory layout of a [rows, D] bfloat16 tile: 16-byte chunks of a row
// are XORed with low bits of the row number.
template <int D>
struct Swz {
  static constexpr int CHUNKS = D / 8;
  static constexpr int MASK = CHUNKS >= 8 ? 7 : CHUNKS - 1;
  static constexpr int SHIFT = CHUNKS >= 8 ? 0 : (CHUNKS == 4 ? 1 : 2);
  __device__ static __forceinline__ int off(int row, int col) {
    const int chunk = col >> 3;
    return row * D + (((chunk ^ ((row >> SHIFT) & MASK))) << 3) + (col & 7);
  }
};

// Copies `rows` x D elements (row stride `ld`) into a swizzled tile; rows at or
// beyond `valid_rows` are zero-filled.
template <int D>
__device__ __forceinline__ void load_tile(__nv_bfloat16* dst, const __nv_bfloat16* src,
                                          long long ld, int rows, int valid_rows) {
  constexpr int CH = D / 8;
  for (int id = threadIdx.x; id < rows * CH; id += THREADS) {
    const int r = id / CH, c = id - r * CH;
    const bool ok = r < valid_rows;
    const __nv_bfloat16* s = src + (ok ? (long long)r * ld + c * 8 : 0);
    cp_async16(smem_u32(dst + Swz<D>::off(r, c * 8)), s, ok);
  }
}

struct AttnParams {
  const __nv_bfloat16* q;
  long long q_stride;
  __nv_bfloat16* out;
  long long out_stride;
  const int* cu_tokens;  // [n_seqs + 1]
  const int* kv_lens;    // [n_seqs]: length after this step
  const int* page_table; // [n_seqs, max_pages]
  int max_pages;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  long long page_stride, head_stride;
  int n_seqs, A, Kh;
  float scale_log2;  // scale * log2(e)
  // decode only
  int splits;    // CTAs per (sequence, kv head)
  int cluster;   // of which this many merge inside a thread-block cluster (1: none)
  int parts;     // partial results per pair that meet in the workspace: splits / cluster
  float* ws_o;   // [n_seqs, Kh, parts, 16, D]
  float* ws_ml;  // [n_seqs, Kh, parts, 16, 2]
  int* counters; // [n_seqs, Kh]: CTAs that have delivered; zero between calls
  const void* next;      // constant data to bring into L2 for the kernel after this one
  long long next_bytes;  // 0 = none
  int trigger_next;      // 1: let the next kernel's blocks be placed once a CTA's pages are in
};

// --------------------------------------------------------------------- prefill
template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const AttnParams p) {
  fb_pdl_wait();
  constexpr int KT = D / 16;  // k-steps of Q.K^T
  constexpr int NT = D / 8;   // n-tiles of P.V
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sK = sQ + 64 * D;          // [2][64][D]
  __nv_bfloat16* sV = sK + 2 * 64 * D;      // [2][64][D]
  __shared__ int s_info[2];

  if (threadIdx.x == 0) {
    // Later blocks of a sequence walk more pages: hand them out first, so that the
    // long ones do not end up alone at the tail of the grid.
    int b = (int)(gridDim.x - 1 - blockIdx.x), s = 0;
    for (; s < p.n_seqs; ++s) {
      const int nb = (p.cu_tokens[s + 1] - p.cu_tokens[s] + 63) / 64;
      if (b < nb) break;
      b -= nb;
    }
    s_info[0] = s < p.n_seqs ? s : -1;
    s_info[1] = b;
  }
  __syncthreads();
  const int seq = s_info[0];
  if (seq < 0) return;
  const int row0 = s_info[1] * 64;
  const int head = blockIdx.y, kvh = head / (p.A / p.Kh);
  const int tok0 = p.cu_tokens[seq], q_len = p.cu_tokens[seq + 1] - tok0;
  const int kv_len = p.kv_lens[seq];
  const int pos0 = kv_len - q_len + row0;  // position of this block's first query
  const int rows_valid = min(64, q_len - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int last_key = pos0 + rows_valid - 1;
  const int n_pages = last_key / FB_PAGE + 1;
  const int* pages = p.page_table + (size_t)seq * p.max_pages;
  const __nv_bfloat16* kbase = p.k_cache + (long long)kvh * p.head_stride;
  const __nv_bfloat16* vbase = p.v_cache + (long long)kvh * p.head_stride;

  load_tile<D>(sQ, p.q + (long long)(tok0 + row0) * p.q_stride + (long long)head * D, p.q_stride,
               64, rows_valid);
  {
    const long long off = (long long)pages[0] * p.page_stride;
    load_tile<D>(sK, kbase + off, D, 64, 64);
    load_tile<D>(sV, vbase + off, D, 64, 64);
  }
  cp_async_commit();

  uint32_t qf[KT][4];
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int qpos_lo = pos0 + warp * 16 + g;  // position of row g; row g + 8 is 8 further

  for (int pg = 0; pg < n_pages; ++pg) {
    const int st = pg & 1;
    if (pg + 1 < n_pages) {
      const long long off = (long long)pages[pg + 1] * p.page_stride;
      load_tile<D>(sK + (st ^ 1) * 64 * D, kbase + off, D, 64, 64);
      load_tile<D>(sV + (st ^ 1) * 64 * D, vbase + off, D, 64, 64);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (pg == 0) {
#pragma unroll
      for (int k = 0; k < KT; ++k)
        ldsm_x4(qf[k], smem_u32(sQ + Swz<D>::off(warp * 16 + (lane & 15), k * 16 + (lane >> 4) * 8)));
    }
    const int key0 = pg * FB_PAGE;
    // a warp whose every query lies before this page has nothing to add
    if (key0 <= pos0 + warp * 16 + 15) {
      const __nv_bfloat16* tK = sK + st * 64 * D;
      const __nv_bfloat16* tV = sV + st * 64 * D;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {  // two n-tiles (16 keys) per ldmatrix.x4
          uint32_t b[4];
          ldsm_x4(b, smem_u32(tK + Swz<D>::off(n2 * 16 + (lane & 7) + (lane >> 4) * 8,
                                              k * 16 + ((lane >> 3) & 1) * 8)));
          mma_bf16(s[2 * n2], qf[k], b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], qf[k], b[2], b[3]);
        }
      }
      // scale, mask, online softmax (in the log2 domain)
      const bool need_mask = key0 + FB_PAGE - 1 > pos0 + warp * 16;
      float mx[2] = {m[0], m[1]};
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * p.scale_log2;
          if (need_mask) {
            const int key = key0 + n * 8 + 2 * t + (e & 1);
            const int qp = qpos_lo + (e >> 1) * 8;
            if (key > qp) v = -INFINITY;
          }
          s[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) corr[r] = exp2f(m[r] - mx[r]);  // 0 on the first page
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[n][e] - mx[e >> 1]);
          s[n][e] = pv;
          sum[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[r] = l[r] * corr[r] + sum[r];
        m[r] = mx[r];
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
      // O += P V: probabilities become the A operand, 16 keys per k-step
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          ldsm_x4_trans(b, smem_u32(tV + Swz<D>::off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                    n2 * 16 + (lane >> 4) * 8)));
          mma_bf16(o[2 * n2], a, b[0], b[1]);
          mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // the stage is refilled two iterations on
  }
  // every valid row saw key 0, so l > 0
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row < rows_valid) {
      const float inv = 1.0f / l[r];
      __nv_bfloat16* dst = p.out + (long long)(tok0 + row0 + row) * p.out_stride + (long long)head * D;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) =
            pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
  }
}

// ---------------------------------------------------------------------- decode
// Called by every CTA of a (sequence, kv head) after it has written its partial
// result. The CTA whose count completes the set reads all partial results and
// writes the heads' outputs; it then puts the counter back to zero for the next
// call. Publishing follows the usual pattern: writes, fence, barrier, one atomic
// add; the reader fences after seeing the full count and reads around L1.
template <int D>
__device__ void merge_if_last(const AttnParams& p, int seq, int kvh, int token, int G) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int before = atomicAdd(&p.counters[seq * p.Kh + kvh], 1);
    s_last = before == p.splits - 1;  // every CTA of the pair arrives once
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const size_t base = (size_t)(seq * p.Kh + kvh) * p.parts;
  for (int idx = threadIdx.x; idx < G * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    // four parts at a time, their twelve loads on the way together
    float M = -INFINITY, L = 0.f, acc = 0.f;
    for (int s0 = 0; s0 < p.parts; s0 += 4) {
      float ms[4], ls[4], os[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool there = s0 + j < p.parts;
        const size_t s = base + (there ? s0 + j : 0);
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + s * 32 + 2 * row));
        os[j] = __ldcg(p.ws_o + (s * 16 + row) * D + d);
        ms[j] = there ? ml.x : -INFINITY;
        ls[j] = ml.y;
      }
      const float Mn = fmaxf(fmaxf(M, fmaxf(ms[0], ms[1])), fmaxf(ms[2], ms[3]));
      if (Mn == -INFINITY) continue;
      const float keep = M == -INFINITY ? 0.f : exp2f(M - Mn);
      L *= keep;
      acc *= keep;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (ms[j] == -INFINITY) continue;  // an empty range: nothing was written for it
        const float f = exp2f(ms[j] - Mn);
        L += ls[j] * f;
        acc += os[j] * f;
      }
      M = Mn;
    }
    p.out[(long long)token * p.out_stride + (long long)(kvh * G + row) * D + d] =
        __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
  if (threadIdx.x == 0) p.counters[seq * p.Kh + kvh] = 0;
}

// ---- the same merge inside a thread-block cluster: the CTAs of a (sequence,
// kv head) form one cluster, each leaves its partial (max, sum, output) in its
// own shared memory, and after a cluster barrier every CTA reads its peers'
// shared memory for its share of the output elements. No workspace in global
// memory, no counters. Every CTA of the cluster calls this exactly once (also
// one whose range is empty): the two barriers need all of them.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer(const float* mine, unsigned rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(mine)), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
constexpr int MAX_CLUSTER = 8;  // portable cluster size

// cO [16][D], cM [16], cL [16]: this CTA's partial result, at the same shared
// memory offset in every CTA of the cluster. With one cluster per pair the
// merged result is the output; with several (parts > 1) it is the cluster's
// partial result, which goes to the workspace where the pair's last CTA merges
// the clusters' results.
template <int D>
__device__ void merge_in_cluster(const AttnParams& p, const float* cO, const float* cM,
                                 const float* cL, int seq, int kvh, int token, int G) {
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  __syncthreads();
  cluster_sync_all();
  const int S = p.cluster;
  const int total = G * D, share = (total + S - 1) / S;
  const int end = min(total, (int)(rank + 1) * share);
  const size_t slot = (size_t)(seq * p.Kh + kvh) * p.parts + blockIdx.z / S;
  for (int idx = rank * share + threadIdx.x; idx < end; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float ms[MAX_CLUSTER], ls[MAX_CLUSTER], os[MAX_CLUSTER];
#pragma unroll
    for (int s = 0; s < MAX_CLUSTER; ++s) {
      ms[s] = -INFINITY; ls[s] = 0.f; os[s] = 0.f;
      if (s < S) {
        ms[s] = ld_peer(cM + row, s);
        ls[s] = ld_peer(cL + row, s);
        // an empty range left no output behind; its sum is zero
        os[s] = ms[s] == -INFINITY ? 0.f : ld_peer(cO + row * D + d, s);
      }
    }
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < MAX_CLUSTER; ++s) M = fmaxf(M, ms[s]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_CLUSTER; ++s) {
      if (ms[s] == -INFINITY) continue;
      const float f = exp2f(ms[s] - M);
      L += ls[s] * f;
      acc += os[s] * f;
    }
    if (p.parts > 1) {
      p.ws_o[(slot * 16 + row) * D + d] = acc;
      if (d == 0) { p.ws_ml[slot * 32 + 2 * row] = M; p.ws_ml[slot * 32 + 2 * row + 1] = L; }
    } else {
      p.out[(long long)token * p.out_stride + (long long)(kvh * G + row) * D + d] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
  }
  cluster_sync_all();  // peers may have been reading this CTA's memory until here
  if (p.parts > 1) merge_if_last<D>(p, seq, kvh, token, G);
}

// NARROW (at most 8 query heads per kv head): the keys are the 16 rows of the
// tensor-core instruction and the query heads its 8 columns, S^T = K Q^T and
// O^T = V^T P^T, half the instructions of the 16-query-row form, of whose rows
// a grouping of 3 or 4 uses a quarter. P^T reaches the second product's operand
// layout by a transposition inside the warp (movmatrix).
template <int D, int ST, bool CLUSTER, bool NARROW>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const AttnParams p) {
  constexpr int KT = D / 16, NT = D / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  // ST page buffers: ST - 1 pages are on their way while one is multiplied. A
  // CTA's speed is pages in flight / memory latency, and the kernel has nothing
  // else to hide that latency behind; more buffers mean fewer CTAs per SM.
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);  // [16][D]
  __nv_bfloat16* sK = sQ + 16 * D;                              // [ST][64][D]
  __nv_bfloat16* sV = sK + ST * 64 * D;                         // [ST][64][D]
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.A / p.Kh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // The step's description (token offsets, lengths, page table) is uploaded
  // before the step's first kernel, so it is read before the wait for the
  // previous kernel; so are cache pages that were full before this step: the
  // step's own keys lie in the pages from `fresh` on.
  const int token = p.cu_tokens[seq];
  const int kv_len = p.kv_lens[seq];
  const int n_pages = (kv_len + FB_PAGE - 1) / FB_PAGE;
  const int per = (n_pages + p.splits - 1) / p.splits;  // a range: 1/splits of the pages
  const int pg0 = split * per;
  const int pg1 = min(n_pages, pg0 + per);
  const int fresh = max(kv_len - (p.cu_tokens[seq + 1] - token), 0) / FB_PAGE;

  // without clusters every CTA's result is a part of its own
  float* ws_o = p.ws_o + ((size_t)(seq * p.Kh + kvh) * p.parts + split) * 16 * D;
  float* ws_ml = p.ws_ml + ((size_t)(seq * p.Kh + kvh) * p.parts + split) * 16 * 2;
  constexpr int DP = D + 8;                                     // padded row of the warps' merge
  float* cO = reinterpret_cast<float*>(sK) + 4 * 16 * DP + 128;  // [16][D] (cluster merge)
  float* cM = cO + 16 * D;                                      // [16]
  float* cL = cM + 16;                                          // [16]
  if (pg0 >= pg1) {  // nothing in this range (or a padding row: kv_len == 0)
    fb_pdl_wait();
    fb_prefetch_l2_slice(p.next, p.next_bytes);
    if (CLUSTER) {
      for (int i = threadIdx.x; i < 16; i += THREADS) { cM[i] = -INFINITY; cL[i] = 0.f; }
      merge_in_cluster<D>(p, cO, cM, cL, seq, kvh, token, G);
    } else if (p.splits > 1) {
      for (int i = threadIdx.x; i < G; i += THREADS) { ws_ml[2 * i] = -INFINITY; ws_ml[2 * i + 1] = 0.f; }
      merge_if_last<D>(p, seq, kvh, token, G);
    } else {
      for (int i = threadIdx.x; i < G * D; i += THREADS)
        p.out[(long long)token * p.out_stride + (long long)(kvh * G) * D + i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int* pages = p.page_table + (size_t)seq * p.max_pages;
  const __nv_bfloat16* kbase = p.k_cache + (long long)kvh * p.head_stride;
  const __nv_bfloat16* vbase = p.v_cache + (long long)kvh * p.head_stride;

  // Every warp streams its own 16 keys (and values) of each page into its own rows
  // of the page buffers and waits for nobody else's: no block barrier in the loop.
  auto load_rows = [&](int buffer, int page) {
    const long long off = (long long)page * p.page_stride;
    constexpr int CH = D / 8;
    for (int id = lane; id < 16 * CH; id += 32) {
      const int r = warp * 16 + id / CH, c = id % CH;
      const int so = buffer * 64 * D + Swz<D>::off(r, c * 8);
      cp_async16(smem_u32(sK + so), kbase + off + r * D + c * 8, true);
      cp_async16(smem_u32(sV + so), vbase + off + r * D + c * 8, true);
    }
  };
  // old pages of the first ST - 1 go out now; they complete with the first group
#pragma unroll
  for (int ahead = 0; ahead < ST - 1; ++ahead)
    if (pg0 + ahead < min(pg1, fresh)) load_rows(ahead, pages[pg0 + ahead]);
  fb_pdl_wait();
  // rows 0..G-1 of the tile are this kv head's query heads, consecutive in q
  load_tile<D>(sQ, p.q + (long long)token * p.q_stride + (long long)(kvh * G) * D, D, 16, G);
#pragma unroll
  for (int ahead = 0; ahead < ST - 1; ++ahead) {
    if (pg0 + ahead < pg1 && pg0 + ahead >= fresh) load_rows(ahead, pages[pg0 + ahead]);
    cp_async_commit();  // one group per page, empty when there is no page
  }

  // wide form: Q as the 16-row operand of S = Q K^T; o is O [16 queries, D].
  // narrow form: Q as the 8-column operand of S^T = K Q^T; o is O^T [D, 8 queries].
  constexpr int OT = NARROW ? KT : NT;
  uint32_t qf[KT][4];
  float o[OT][4];
#pragma unroll
  for (int n = 0; n < OT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  // wide: rows g, g + 8; narrow: queries 2t, 2t + 1 (the same in all lanes of a t)
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  int next_page = pg0 + ST - 1 < pg1 ? pages[pg0 + ST - 1] : 0;
  for (int pg = pg0; pg < pg1; ++pg) {
    const int st = (pg - pg0) % ST;
    __syncwarp();  // every lane has read the rows that the refill overwrites
    // The page number of the refill was read an iteration ago: a warp issues in
    // order, and a page-table read in front of the copies would hold up the whole
    // iteration for a trip to L2.
    const int refill_page = next_page;
    if (pg + ST < pg1) next_page = pages[pg + ST];
    // The buffer that the previous iteration finished with is refilled once this
    // page's score products have been issued: a warp issues in order, and the
    // copies' address arithmetic then runs while the tensor cores work instead of
    // in front of them.
    auto refill = [&]() {
      if (pg + ST - 1 < pg1) load_rows((pg - pg0 + ST - 1) % ST, refill_page);
      cp_async_commit();
    };
    cp_async_wait<ST - 2>();  // all but the newest ST - 2 groups: page `pg` has landed
    if (pg == pg0) __syncthreads();  // the queries came from all warps
    else __syncwarp();               // the page's rows from this warp's lanes
    if (pg == pg0) {
      if constexpr (NARROW) {
        // 8 x 8 matrices of Q: rows = queries 0..7, columns = 8 consecutive elements;
        // a lane then holds (query g; elements 2t, 2t + 1), the B operand's layout
        if constexpr (KT == 1) {
          uint32_t r[2];
          ldsm_x2(r, smem_u32(sQ + Swz<D>::off(lane & 7, ((lane >> 3) & 1) * 8)));
          qf[0][0] = r[0]; qf[0][1] = r[1];
        } else {
#pragma unroll
          for (int k2 = 0; k2 < KT / 2; ++k2) {
            uint32_t r[4];
            ldsm_x4(r, smem_u32(sQ + Swz<D>::off(lane & 7, k2 * 32 + (lane >> 3) * 8)));
            qf[2 * k2][0] = r[0]; qf[2 * k2][1] = r[1];
            qf[2 * k2 + 1][0] = r[2]; qf[2 * k2 + 1][1] = r[3];
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < KT; ++k)
          ldsm_x4(qf[k], smem_u32(sQ + Swz<D>::off(lane & 15, k * 16 + (lane >> 4) * 8)));
      }
    }
    const int key0 = pg * FB_PAGE + warp * 16;  // this warp's 16 keys of the page
    if (key0 < kv_len) {
      const __nv_bfloat16* tK = sK + st * 64 * D;
      const __nv_bfloat16* tV = sV + st * 64 * D;
      if constexpr (NARROW) {
        // S^T [16 keys, 8 queries]: up to four accumulators take the k steps in
        // turn, so that no product waits for more than one before it
        constexpr int NS = KT >= 4 ? 4 : KT;
        float sp[NS][4];
#pragma unroll
        for (int i = 0; i < NS; ++i) sp[i][0] = sp[i][1] = sp[i][2] = sp[i][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
          uint32_t a[4];
          ldsm_x4(a, smem_u32(tK + Swz<D>::off(warp * 16 + (lane & 15), k * 16 + (lane >> 4) * 8)));
          mma_bf16(sp[k % NS], a, qf[k][0], qf[k][1]);
        }
        refill();
        // s[e]: key g + 8 (e >> 1), query 2t + (e & 1)
        float s[4];
        float mx[2] = {m[0], m[1]};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sp[0][e];
#pragma unroll
          for (int i = 1; i < NS; ++i) v += sp[i][e];
          v *= p.scale_log2;
          if (key0 + g + (e >> 1) * 8 >= kv_len) v = -INFINITY;
          s[e] = v;
          mx[e & 1] = fmaxf(mx[e & 1], v);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
        }
        // key0 < kv_len: the warp's first key is visible, so mx is finite
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) corr[r] = exp2f(m[r] - mx[r]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[e] - mx[e & 1]);
          s[e] = pv;
          sum[e & 1] += pv;
        }
        // l stays this lane's share of the sum (its own keys); the lanes' shares
        // meet once, after the last page
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          l[r] = l[r] * corr[r] + sum[r];
          m[r] = mx[r];
        }
#pragma unroll
        for (int n = 0; n < OT; ++n) {
          o[n][0] *= corr[0]; o[n][1] *= corr[1];
          o[n][2] *= corr[0]; o[n][3] *= corr[1];
        }
        // P^T as the B operand: (keys 2t, 2t + 1 and 2t + 8, 2t + 9; query g)
        const uint32_t b0 = movmatrix_trans(pack_bf16(s[0], s[1]));
        const uint32_t b1 = movmatrix_trans(pack_bf16(s[2], s[3]));
#pragma unroll
        for (int n = 0; n < OT; ++n) {
          // V^T [16 elements, 16 keys] from V [key][element], transposed on the way in
          uint32_t a[4];
          ldsm_x4_trans(a, smem_u32(tV + Swz<D>::off(warp * 16 + (lane & 7) + (lane >> 4) * 8,
                                                    n * 16 + ((lane >> 3) & 1) * 8)));
          mma_bf16(o[n], a, b0, b1);
        }
      } else {
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
          uint32_t b[4];
          ldsm_x4(b, smem_u32(tK + Swz<D>::off(warp * 16 + (lane & 7) + (lane >> 4) * 8,
                                              k * 16 + ((lane >> 3) & 1) * 8)));
          mma_bf16(s[0], qf[k], b[0], b[1]);
          mma_bf16(s[1], qf[k], b[2], b[3]);
        }
        refill();
        float mx[2] = {m[0], m[1]};
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = s[n][e] * p.scale_log2;
            if (key0 + n * 8 + 2 * t + (e & 1) >= kv_len) v = -INFINITY;
            s[n][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) corr[r] = exp2f(m[r] - mx[r]);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[n][e] - mx[e >> 1]);
            s[n][e] = pv;
            sum[e >> 1] += pv;
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {  // l: this lane's share of the sum, as in the narrow form
          l[r] = l[r] * corr[r] + sum[r];
          m[r] = mx[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[n][0] *= corr[0]; o[n][1] *= corr[0];
          o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          ldsm_x4_trans(b, smem_u32(tV + Swz<D>::off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                    n2 * 16 + (lane >> 4) * 8)));
          mma_bf16(o[2 * n2], a, b[0], b[1]);
          mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    } else {
      refill();
    }
  }
  cp_async_wait<0>();
  fb_prefetch_l2_slice(p.next, p.next_bytes);
  // this CTA's pages are in: where the caller says so, the next kernel's blocks may be
  // placed while the partial results are merged
  if (p.trigger_next) fb_pdl_launch();
  // the lanes' shares of the sums meet: over the keys' lanes (g in the narrow form, t in the wide)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if constexpr (NARROW) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 4);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 8);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 16);
    } else {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
  }
  __syncthreads();  // all warps are through with the page buffers

  // merge the four warps' (m, l, O) through shared memory (the page buffers are free now)
  float* sO = reinterpret_cast<float*>(sK);   // [4][16][DP], rows padded: fewer bank conflicts
  float* sM = sO + 4 * 16 * DP;               // [4][16]
  float* sL = sM + 4 * 16;                    // [4][16]
  if constexpr (NARROW) {
    // o[n][e]: element 16 n + g + 8 (e >> 1) of query 2t + (e & 1); rows 8..15 stay unused
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = 2 * t + r;
      if (g == 0) { sM[warp * 16 + row] = m[r]; sL[warp * 16 + row] = l[r]; }
#pragma unroll
      for (int n = 0; n < OT; ++n) {
        sO[(warp * 16 + row) * DP + n * 16 + g] = o[n][r];
        sO[(warp * 16 + row) * DP + n * 16 + g + 8] = o[n][2 + r];
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + r * 8;
      if (t == 0) { sM[warp * 16 + row] = m[r]; sL[warp * 16 + row] = l[r]; }
#pragma unroll
      for (int n = 0; n < OT; ++n) {
        *reinterpret_cast<float2*>(sO + (warp * 16 + row) * DP + n * 8 + 2 * t) =
            make_float2(o[n][2 * r], o[n][2 * r + 1]);
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sM[w * 16 + row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sM[w * 16 + row];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += sL[w * 16 + row] * f;
      acc += sO[(w * 16 + row) * DP + d] * f;
    }
    if (CLUSTER) {
      cO[row * D + d] = acc;
      if (d == 0) { cM[row] = M; cL[row] = L; }
    } else if (p.splits > 1) {
      ws_o[row * D + d] = acc;
      if (d == 0) { ws_ml[2 * row] = M; ws_ml[2 * row + 1] = L; }
    } else {
      p.out[(long long)token * p.out_stride + (long long)(kvh * G + row) * D + d] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
  }
  if (CLUSTER) merge_in_cluster<D>(p, cO, cM, cL, seq, kvh, token, G);
  else if (p.splits > 1) merge_if_last<D>(p, seq, kvh, token, G);
}

template <int D>
int launch_prefill(const AttnParams& p, int q_blocks, cudaStream_t stream) {
  const int bytes = (64 + 4 * 64) * D * 2;
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fb_fail(2, "attention_prefill: %s", cudaGetErrorString(e));
  }
  fb_launch(attn_prefill_kernel<D>, dim3(dim3(q_blocks, p.A)), dim3(THREADS), bytes, stream, p);
  return fb_check_launch("attention_prefill");
}

template <int D, int ST, bool CLUSTER, bool NARROW>
int launch_decode_as(const AttnParams& p, cudaStream_t stream) {
  int bytes = (16 + 2 * ST * 64) * D * 2;
  // the merge reuses the page buffers: four warps' outputs, their (max, sum),
  // and the CTA's own partial result for its cluster
  const int merge = 16 * D * 2 + (4 * 16 * (D + 8) + 128 + 16 * D + 32) * 4;
  if (merge > bytes) bytes = merge;
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, ST, CLUSTER, NARROW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fb_fail(2, "attention_decode: %s", cudaGetErrorString(e));
  }
  const dim3 grid(p.n_seqs, p.Kh, p.splits);
  if (CLUSTER)
    fb_launch_cluster(attn_decode_kernel<D, ST, CLUSTER, NARROW>, grid, dim3(THREADS), bytes, stream,
                      (unsigned)p.cluster, p);
  else
    fb_launch(attn_decode_kernel<D, ST, CLUSTER, NARROW>, grid, dim3(THREADS), bytes, stream, p);
  return fb_check_launch("attention_decode");
}

// Several CTAs per (sequence, kv head) merge inside clusters of p.cluster, and
// what is left (all of them when p.cluster is 1) through the workspace.
template <int D, int ST>
int launch_decode(const AttnParams& p, cudaStream_t stream) {
  const bool narrow = p.A / p.Kh <= 8;
  if (p.cluster > 1)
    return narrow ? launch_decode_as<D, ST, true, true>(p, stream)
                  : launch_decode_as<D, ST, true, false>(p, stream);
  return narrow ? launch_decode_as<D, ST, false, true>(p, stream)
                : launch_decode_as<D, ST, false, false>(p, stream);
}

int check_common(const char* what, int n_seqs, int A, int Kh, int D, long long q_stride,
                 long long out_stride, const void* q, const void* k, const void* v,
                 long long page_stride, long long head_stride) {
  FB_REQUIRE(n_seqs > 0 && A > 0 && Kh > 0 && A % Kh == 0, "%s: bad head counts A=%d Kh=%d", what, A, Kh);
  FB_REQUIRE(D == 16 || D == 32 || D == 64 || D == 128,
             "%s: head size %d is not built for the tensor-core kernel (16, 32, 64, 128)", what, D);
  FB_REQUIRE(A / Kh <= 16, "%s: %d query heads per kv head exceed the 16-row tile", what, A / Kh);
  FB_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && page_stride % 8 == 0 && head_stride % 8 == 0,
             "%s: strides must keep 16-byte alignment", what);
  FB_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0,
             "%s: pointers must be 16-byte aligned", what);
  return 0;
}

}  // namespace

// Prompts (or any mix of token counts): q [T, A*D] rows with stride q_stride.
// `q_blocks` bounds the number of 64-row query blocks: sum over sequences of
// ceil(q_len / 64); blocks beyond the real count return at once.
FB_API int fb_attention_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                const int* cu_tokens, const int* kv_lens, const int* page_table,
                                int max_pages, const void* k_cache, const void* v_cache,
                                long long page_stride, long long head_stride, int n_seqs,
                                int q_blocks, int A, int Kh, int D, float scale,
                                cudaStream_t stream) {
  int rc = check_common("attention_prefill", n_seqs, A, Kh, D, q_stride, out_stride, q, k_cache,
                        v_cache, page_stride, head_stride);
  if (rc) return rc;
  if (q_blocks <= 0) return 0;
  AttnParams p{};
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.cu_tokens = cu_tokens; p.kv_lens = kv_lens; p.page_table = page_table; p.max_pages = max_pages;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.page_stride = page_stride; p.head_stride = head_stride;
  p.n_seqs = n_seqs; p.A = A; p.Kh = Kh; p.scale_log2 = scale * LOG2E; p.splits = 1;
  switch (D) {
    case 16: return launch_prefill<16>(p, q_blocks, stream);
    case 32: return launch_prefill<32>(p, q_blocks, stream);
    case 64: return launch_prefill<64>(p, q_blocks, stream);
    default: return launch_prefill<128>(p, q_blocks, stream);
  }
}

// One token per sequence. `splits` CTAs share each (sequence, kv head).
// `cluster` of them (up to 8; a divisor of `splits`; 0 or 1 for none) form a
// thread-block cluster and merge their partial results through each other's
// shared memory. The splits / cluster results per pair that are left (`parts`;
// all of them without clusters) meet in the workspaces, which must hold
// n_seqs*Kh*parts*16*D and n_seqs*Kh*parts*32 floats, with `counters` of
// n_seqs*Kh ints that are zero when the call starts (the kernel leaves them zero
// again); with one part per pair they are not used and may be null. `stages`
// (2 or 3) is the number of page buffers per CTA. A sequence with kv_lens == 0
// is padding: its output rows are zeros. `trigger_next`: see AttnParams (it pays in
// front of the tcgen05 products and costs a third of the step in front of the
// weight-streaming one, whose blocks then crowd in beside the attention's).
FB_API int fb_attention_decode(const void* q, long long q_stride, void* out, long long out_stride,
                               const int* cu_tokens, const int* kv_lens, const int* page_table,
                               int max_pages, const void* k_cache, const void* v_cache,
                               long long page_stride, long long head_stride, int n_seqs, int A,
                               int Kh, int D, float scale, int splits, int stages, int cluster,
                               float* ws_o, float* ws_ml, int* counters,
                               const void* next, long long next_bytes, int trigger_next,
                               cudaStream_t stream) {
  FB_REQUIRE(next_bytes >= 0 && next_bytes % 16 == 0 && ((uintptr_t)next % 16) == 0,
             "attention_decode: the prefetch range must be 16-byte aligned and a multiple of 16 bytes");
  int rc = check_common("attention_decode", n_seqs, A, Kh, D, q_stride, out_stride, q, k_cache,
                        v_cache, page_stride, head_stride);
  if (rc) return rc;
  FB_REQUIRE(splits >= 1 && splits <= 65535, "attention_decode: bad split count %d", splits);
  if (cluster < 1) cluster = 1;
  FB_REQUIRE(cluster <= MAX_CLUSTER && splits % cluster == 0,
             "attention_decode: clusters of %d do not divide %d splits (or exceed %d)", cluster,
             splits, MAX_CLUSTER);
  const int parts = splits / cluster;
  FB_REQUIRE(parts == 1 || (ws_o && ws_ml && counters && ((uintptr_t)ws_ml % 8) == 0),
             "attention_decode: %d partial results per pair need workspaces (8-byte aligned) "
             "and counters", parts);
  AttnParams p{};
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.cu_tokens = cu_tokens; p.kv_lens = kv_lens; p.page_table = page_table; p.max_pages = max_pages;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.page_stride = page_stride; p.head_stride = head_stride;
  p.n_seqs = n_seqs; p.A = A; p.Kh = Kh; p.scale_log2 = scale * LOG2E;
  p.splits = splits; p.cluster = cluster; p.parts = parts;
  p.ws_o = ws_o; p.ws_ml = ws_ml; p.counters = counters;
  p.next = next; p.next_bytes = next_bytes;
  p.trigger_next = trigger_next ? 1 : 0;
  FB_REQUIRE(stages == 2 || stages == 3, "attention_decode: %d page buffers (2 or 3)", stages);
  if (stages == 2) {
    switch (D) {
      case 16: return launch_decode<16, 2>(p, stream);
      case 32: return launch_decode<32, 2>(p, stream);
      case 64: return launch_decode<64, 2>(p, stream);
      default: return launch_decode<128, 2>(p, stream);
    }
  }
  switch (D) {
    case 16: return launch_decode<16, 3>(p, stream);
    case 32: return launch_decode<32, 3>(p, stream);
    case 64: return launch_decode<64, 3>(p, stream);
    default: return launch_decode<128, 3>(p, stream);
  }
}

// ------------------------------------------------- the entry point that allocates nothing
// See attention_static.h for who calls it and why.
#include <mutex>

#include "attention_static.h"

// The splits' partial results live here instead of in a caller's workspace.
// In host code `g_static_scratch` is only a handle for the symbol: its device
// address must be asked for with cudaGetSymbolAddress before a kernel gets it.
static __device__ __align__(256) float g_static_scratch[FB_ATTENTION_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the scratch array on the current device; looked up once.
int static_scratch(float** addr) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fb_fail(2, "attention_decode_static: %s", cudaGetErrorString(e));
  if (device < 0 || device >= MAX_DEVICES)
    return fb_fail(1, "attention_decode_static: device %d is beyond the %d this library tracks",
                   device, MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[device] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fb_fail(2, "attention_decode_static: cudaGetSymbolAddress failed: %s",
                     cudaGetErrorString(e));
    g_static_scratch_addr[device] = ptr;
  }
  *addr = g_static_scratch_addr[device];
  return 0;
}
}  // namespace

FB_API int fb_attention_decode_static(const void* q, long long q_stride, void* out,
                                      long long out_stride, const int* cu_tokens,
                                      const int* kv_lens, const int* page_table, int max_pages,
                                      const void* k_cache, const void* v_cache,
                                      long long page_stride, long long head_stride, int n_seqs,
                                      int A, int Kh, int D, float scale, int splits,
                                      cudaStream_t stream) {
  FB_REQUIRE(n_seqs > 0 && Kh > 0 && D > 0 && splits >= 1,
             "attention_decode_static: bad sizes n_seqs=%d Kh=%d D=%d splits=%d", n_seqs, Kh, D,
             splits);
  const long long units = (long long)n_seqs * Kh * splits;
  const long long need = units * (16LL * D + 32) + ((long long)n_seqs * Kh + 63) / 64 * 64;
  FB_REQUIRE(need <= (long long)FB_ATTENTION_STATIC_SCRATCH_FLOATS,
             "attention_decode_static: %d sequences x %d kv heads x %d splits at head size %d need "
             "%lld floats of scratch, the built-in array holds %d; use fewer splits or "
             "fb_attention_decode with a workspace of your own",
             n_seqs, Kh, splits, D, need, FB_ATTENTION_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  // The arrival counters sit at the start of the array. They are the one part that
  // must be zero when a call starts: the array is zero when the library is loaded,
  // and the kernel puts every counter it used back to zero before it ends. Behind
  // them come the partial outputs and the (max, sum) pairs, which a call writes
  // before it reads them.
  int* counters = reinterpret_cast<int*>(scratch);
  const long long head = ((long long)n_seqs * Kh + 63) / 64 * 64;
  float* ws_o = scratch + head;
  float* ws_ml = ws_o + units * 16 * D;
  return fb_attention_decode(q, q_stride, out, out_stride, cu_tokens, kv_lens, page_table,
                             max_pages, k_cache, v_cache, page_stride, head_stride, n_seqs, A, Kh,
                             D, scale, splits, 3, 1, ws_o, ws_ml, counters, nullptr, 0, 0, stream);
}
