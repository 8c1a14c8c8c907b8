// Prompt attention on the 5th-generation tensor cores: causal grouped-query
// attention of a 128-row block of one sequence's queries, for one head, over the
// sequence's cache pages (64 keys each), with both products issued as
// tcgen05.mma and both accumulators in tensor memory.
//
// Formulas are the reference's (src/nn/attention.rs:23-60: head a reads kv head
// a / G; src/models/llama/attention.rs:56-58: scale 1/sqrt(D);
// src/nn/masking.rs:76-92: key j visible iff j <= query position;
// src/nn/activation.rs:30-40: softmax with a maximum subtracted). Scores and
// the output accumulate in 32-bit; probabilities are rounded to bfloat16 only as
// the operand of the P.V product.
//
// Roles of a CTA (192 threads):
//   warp 0     one lane issues TMA loads: the query tile once, then a ring of
//              two K pages and a ring of two V pages (a K page is free again
//              when its scores are computed, a V page one product later);
//   warp 1     allocates tensor memory; one lane issues S = Q K^T (M 128, N 64)
//              into one of two score buffers and O += P V one page behind, so
//              that the next page's scores are computed while this page's
//              softmax runs. P is the A operand of that product and comes from
//              tensor memory (V is read MN-major straight from its [key, d] page);
//   warps 2-5  softmax: thread r owns query row r. It reads its 64 scores from
//              tensor memory, masks, exponentiates against a reference maximum,
//              and stores the probabilities as bfloat16 pairs into the first 32
//              columns of the score buffer they came from. The reference maximum
//              only moves when the row's maximum has grown by more than 2^8; only
//              then does the warp wait for the running product and read the
//              output accumulator back, rescale and store it again.
//   At the end the softmax warps read O, divide by the row sums and store.
//
// With P in the score buffers there are two of them, so the softmax of page
// j + 1 never waits for the product of page j: an earlier version kept one P tile
// in shared memory, and a page then cost the whole chain P -> product -> commit ->
// softmax (2,700 cycles a page whatever the softmax did; taking its loads, exps
// and stores out changed nothing).
//
// Shared memory (96 KB at head size 128) and tensor memory (256 columns) are
// sized so that two CTAs share an SM: the second CTA's warps fill the gaps that
// a row's long dependent chain leaves on the schedulers and the tensor pipe.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the CTA's
// abort flag, all roles run out, tensor memory is freed, and the host can read
// the place from `fb_attention_tc_status`.
#include <mutex>
#include <unordered_map>

#define FB_STATUS_KERNEL 3
#include "tcgen05.cuh"

namespace {

constexpr int BQ = 128;        // query rows per CTA = lanes of tensor memory
constexpr int ST = 2;          // K stages, and V stages
constexpr int THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;  // the reference maximum moves in steps of 2^8 at least

struct FaParams {
  __nv_bfloat16* out;
  long long out_stride;
  const int* cu_tokens;
  const int* kv_lens;
  const int* page_table;
  int max_pages, n_seqs, A, Kh;
  float scale_log2;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct FaSmem {
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int PAGE_BYTES = FB_PAGE * D * 2;       // one K or V page of one head
  static constexpr int USED = Q_BYTES + 2 * ST * PAGE_BYTES + 256;
  // never three CTAs on an SM: they would need more tensor memory than it has
  static constexpr int BYTES = USED > 77 * 1024 ? USED : 77 * 1024;
  static_assert(BYTES <= (233472 - 2 * 1024) / 2, "two CTAs must fit an SM");
};

template <int D>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  constexpr int SUB = D / 64;                  // 64-element (128-byte) blocks along D
  constexpr int Q_SUB = BQ * 128;              // bytes of one query sub-tile
  constexpr int KV_SUB = FB_PAGE * 128;        // bytes of one K or V sub-tile
  constexpr int TMEM_COLS = 256;               // 2 x 64 score columns + D output columns
  constexpr uint32_t O_COL = 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];  // swizzled tiles start on 1,024 bytes
  uint8_t* base = smem_raw;
  uint8_t* sQ = base;
  uint8_t* sK = sQ + FaSmem<D>::Q_BYTES;                 // [ST][SUB][64 keys][64]
  uint8_t* sV = sK + ST * FaSmem<D>::PAGE_BYTES;         // [ST][SUB][64 keys][64]
  uint64_t* bars = (uint64_t*)(sV + ST * FaSmem<D>::PAGE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;         // [ST]
  uint64_t* v_full = k_full + ST;      // [ST]
  uint64_t* k_empty = v_full + ST;     // [ST]
  uint64_t* v_empty = k_empty + ST;    // [ST]
  uint64_t* s_full = v_empty + ST;     // [2]: the scores of a page are in buffer b
  uint64_t* p_full = s_full + 2;       // [2]: its probabilities have replaced them
  uint64_t* pv_done = p_full + 2;      // completes once per P.V product
  uint64_t* o_final = pv_done + 1;     // completes once, after the last one
  uint32_t* tmem_slot = (uint32_t*)(o_final + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* s_info = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    // Later blocks of a sequence walk more pages: they are handed out first, and
    // the heads are the fast grid index, so that the long blocks of every head
    // start before any short one.
    int b = (int)(gridDim.y - 1 - blockIdx.y), s = 0;
    for (; s < p.n_seqs; ++s) {
      const int nb = (p.cu_tokens[s + 1] - p.cu_tokens[s] + BQ - 1) / BQ;
      if (b < nb) break;
      b -= nb;
    }
    s_info[0] = s < p.n_seqs ? s : -1;
    s_info[1] = b;
    mbar_init(q_full, 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);  // one arrival per softmax warp
    }
    mbar_init(pv_done, 1);
    mbar_init(o_final, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int seq = s_info[0];
  if (seq < 0) return;  // a block beyond the real count: nothing allocated yet
  if (smem_u32(base) & 1023u) {  // the tiles' swizzle pattern assumes this alignment
    if (threadIdx.x == 0)
      record_failure(20, (int)(blockIdx.x + gridDim.x * blockIdx.y), (int)(smem_u32(base) & 1023u));
    return;
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

  const int row0 = s_info[1] * BQ;
  const int head = blockIdx.x, kvh = head / (p.A / p.Kh);
  const int tok0 = p.cu_tokens[seq], q_len = p.cu_tokens[seq + 1] - tok0;
  const int kv_len = p.kv_lens[seq];
  const int pos0 = kv_len - q_len + row0;  // position of this block's first query
  const int rows_valid = min(BQ, q_len - row0);
  const int n_pages = (pos0 + rows_valid - 1) / FB_PAGE + 1;
  const int* pages = p.page_table + (size_t)seq * p.max_pages;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      fb_pdl_wait();  // the queries and this step's keys and values come from earlier kernels
      mbar_expect_tx(q_full, FaSmem<D>::Q_BYTES);
#pragma unroll
      for (int sb = 0; sb < SUB; ++sb)
        tma_load_2d(sQ + sb * Q_SUB, &map_q, q_full, head * D + sb * 64, tok0 + row0);
      for (int j = 0; j < n_pages; ++j) {
        const int s = j % ST;
        const uint32_t parity = (uint32_t)((j / ST) & 1) ^ 1u;
        const int page = pages[j];
        if (!mbar_wait(&k_empty[s], parity, abort_flag, 11, j)) break;
        mbar_expect_tx(&k_full[s], FaSmem<D>::PAGE_BYTES);
#pragma unroll
        for (int sb = 0; sb < SUB; ++sb)
          tma_load_3d(sK + s * FaSmem<D>::PAGE_BYTES + sb * KV_SUB, &map_k, &k_full[s], sb * 64,
                      kvh * FB_PAGE, page);
        if (!mbar_wait(&v_empty[s], parity, abort_flag, 10, j)) break;
        mbar_expect_tx(&v_full[s], FaSmem<D>::PAGE_BYTES);
#pragma unroll
        for (int sb = 0; sb < SUB; ++sb)
          tma_load_3d(sV + s * FaSmem<D>::PAGE_BYTES + sb * KV_SUB, &map_v, &v_full[s], sb * 64,
                      kvh * FB_PAGE, page);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BQ, FB_PAGE);
      constexpr uint32_t idesc_pv = make_idesc_b_mn(BQ, D);
      bool ok = mbar_wait(q_full, 0, abort_flag, 12, 0);
      for (int j = 0; j <= n_pages && ok; ++j) {
        if (j < n_pages) {
          // S[j & 1] = Q K_j^T. The buffer held P of page j - 2, whose product was
          // issued in the previous iteration: the tensor pipe runs them in order.
          const int s = j % ST, b = j & 1;
          ok = mbar_wait(&k_full[s], (uint32_t)((j / ST) & 1), abort_flag, 13, j);
          if (!ok) break;
          tc_fence_after();
          const uint32_t q_addr = smem_u32(sQ);
          const uint32_t k_addr = smem_u32(sK + s * FaSmem<D>::PAGE_BYTES);
#pragma unroll
          for (int sb = 0; sb < SUB; ++sb)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma(tmem_base + (uint32_t)(b * FB_PAGE), make_desc(q_addr + sb * Q_SUB + k * 32),
                   make_desc(k_addr + sb * KV_SUB + k * 32), idesc_qk, (sb | k) != 0 ? 1u : 0u);
          tc_commit(&s_full[b]);
          tc_commit(&k_empty[s]);
        }
        if (j >= 1) {
          // O += P_{j-1} V_{j-1}, one page behind the scores; P from tensor memory
          const int jj = j - 1, s = jj % ST, b = jj & 1;
          ok = mbar_wait(&p_full[b], (uint32_t)((jj >> 1) & 1), abort_flag, 15, jj) &&
               mbar_wait(&v_full[s], (uint32_t)((jj / ST) & 1), abort_flag, 9, jj);
          if (!ok) break;
          tc_fence_after();
          const uint32_t v_addr = smem_u32(sV + s * FaSmem<D>::PAGE_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 keys per instruction: 8 columns of P, 16 rows of V
            umma_a_tmem(tmem_base + O_COL, tmem_base + (uint32_t)(b * FB_PAGE + k * 8),
                        make_desc_mn(v_addr + k * 16 * 128, KV_SUB), idesc_pv,
                        (jj | k) != 0 ? 1u : 0u);
          tc_commit(&v_empty[s]);
          tc_commit(pv_done);
          if (jj == n_pages - 1) tc_commit(o_final);
        }
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qpos = pos0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    fb_pdl_wait();
    for (int j = 0; j < n_pages && ok; ++j) {
      const int b = j & 1;
      ok = mbar_wait(&s_full[b], (uint32_t)((j >> 1) & 1), abort_flag, 16, j);
      if (!ok) break;
      tc_fence_after();
      float sc[FB_PAGE];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * FB_PAGE), r0);
        tmem_ld32(tmem_base + lane_base + (uint32_t)(b * FB_PAGE + 32), r1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sc[e] = __uint_as_float(r0[e]);
          sc[32 + e] = __uint_as_float(r1[e]);
        }
      }

      const int key0 = j * FB_PAGE;
      const bool diagonal = key0 + FB_PAGE - 1 > pos0 + quarter * 32;  // some key may be masked
      if (diagonal) {
#pragma unroll
        for (int e = 0; e < FB_PAGE; ++e)
          if (key0 + e > qpos) sc[e] = -INFINITY;
      }
      // the row maximum of the raw scores, by four independent chains; the scale is
      // positive, so it can be applied to the maximum afterwards
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < FB_PAGE; e += 4) {
        mx4[0] = fmaxf(mx4[0], sc[e]);
        mx4[1] = fmaxf(mx4[1], sc[e + 1]);
        mx4[2] = fmaxf(mx4[2], sc[e + 2]);
        mx4[3] = fmaxf(mx4[3], sc[e + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const bool grow = mx > m_ref + RESCALE_STEP;  // also the first page (m_ref = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float corr = grow ? exp2f(m_ref - mx) : 1.0f;  // 0 on the first page
        if (j > 0) {
          // the accumulator must be at rest: wait for the product of page j - 1
          ok = mbar_wait(pv_done, (uint32_t)((j - 1) & 1), abort_flag, 18, j);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_base + O_COL + (uint32_t)c, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
            tmem_st32(tmem_base + lane_base + O_COL + (uint32_t)c, r);
          }
          tmem_st_wait();
        }
        l *= corr;
        if (grow) m_ref = mx;
      }
      // probabilities against the reference maximum (at most 2^8), rounded to bfloat16
      // and packed two keys to a column: the A operand of the product, in the first 32
      // columns of this page's score buffer
      const float neg_ref = -m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        // 2^(s * scale - m_ref): one multiply-add and one ex2; the result is at most 2^8
        // and is rounded to bfloat16 next, so the approximate ex2 costs no accuracy
        const float p0 = fast_exp2(fmaf(sc[2 * c], p.scale_log2, neg_ref));
        const float p1 = fast_exp2(fmaf(sc[2 * c + 1], p.scale_log2, neg_ref));
        sum4[c & 1] += p0;
        sum4[2 + (c & 1)] += p1;
        const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        packed[c] = *reinterpret_cast<const uint32_t*>(&h);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_st32(tmem_base + lane_base + (uint32_t)(b * FB_PAGE), packed);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }
    // O / l
    if (ok) ok = mbar_wait(o_final, 0, abort_flag, 19, n_pages);
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;  // every valid row saw key 0
      __nv_bfloat16* dst =
          p.out + (long long)(tok0 + row0 + row) * p.out_stride + (long long)head * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_base + O_COL + (uint32_t)c, r);
        tmem_ld_wait();
        if (row < rows_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2);
            pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + c + e) = pk;
          }
        }
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

// bf16 tensor of rank 2 or 3, innermost dimension contiguous, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int rank, const long long* dims,
             const long long* strides_elems, const int* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fb_fail(3, "attention_tc: cuTensorMapEncodeTiled is not available");
  cuuint64_t d[3], s[2];
  cuuint32_t b[3], e[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = (cuuint64_t)dims[i]; b[i] = (cuuint32_t)box[i]; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = (cuuint64_t)strides_elems[i] * 2;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d,
                  s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fb_fail(3, "attention_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& p,
           int q_blocks, cudaStream_t stream) {
  static bool configured[64] = {};
  if (fb_first_use_on_device(configured)) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FaSmem<D>::BYTES);
    if (e != cudaSuccess) return fb_fail(2, "attention_tc: %s", cudaGetErrorString(e));
  }
  fb_launch(attn_prefill_tc_kernel<D>, dim3(p.A, q_blocks), dim3(THREADS), FaSmem<D>::BYTES, stream,
            mq, mk, mv, p);
  return fb_check_launch("attention_prefill_tc");
}

}  // namespace

// Prompt attention on tcgen05. q: [T, A*D] bf16 rows with stride q_stride (all
// heads of a token contiguous); k_cache / v_cache: one cache entry's views
// [n_pages, Kh, 64, D] with strides (page_stride, 64*D, D, 1). `q_blocks` bounds
// the number of 128-row query blocks: the sum over sequences of ceil(q_len / 128).
// Head sizes 64 and 128.
FB_API int fb_attention_prefill_tc(const void* q, long long q_stride, int T, void* out,
                                   long long out_stride, const int* cu_tokens, const int* kv_lens,
                                   const int* page_table, int max_pages, const void* k_cache,
                                   const void* v_cache, long long page_stride,
                                   long long head_stride, int n_pages, int n_seqs, int q_blocks,
                                   int A, int Kh, int D, float scale, cudaStream_t stream) {
  FB_REQUIRE(D == 64 || D == 128, "attention_tc: head size %d is not built (64, 128)", D);
  FB_REQUIRE(n_seqs > 0 && A > 0 && Kh > 0 && A % Kh == 0 && T > 0 && n_pages > 0,
             "attention_tc: bad sizes");
  FB_REQUIRE(head_stride == (long long)FB_PAGE * D, "attention_tc: the heads of a page must be contiguous");
  FB_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && page_stride % 8 == 0 &&
                 ((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                 ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0,
             "attention_tc: pointers and strides must keep 16-byte alignment");
  if (q_blocks <= 0) return 0;
  bind_status_mirror(stream);
  CUtensorMap mq, mk, mv;
  {
    const long long dims[2] = {(long long)A * D, T}, strides[1] = {q_stride};
    const int box[2] = {64, BQ};
    int rc = make_map(&mq, q, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const long long dims[3] = {D, (long long)Kh * FB_PAGE, n_pages};
    const long long strides[2] = {D, page_stride};
    const int box[3] = {64, FB_PAGE, 1};
    int rc = make_map(&mk, k_cache, 3, dims, strides, box);
    if (rc) return rc;
    rc = make_map(&mv, v_cache, 3, dims, strides, box);
    if (rc) return rc;
  }
  FaParams p;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.cu_tokens = cu_tokens; p.kv_lens = kv_lens; p.page_table = page_table;
  p.max_pages = max_pages; p.n_seqs = n_seqs; p.A = A; p.Kh = Kh;
  p.scale_log2 = scale * LOG2E;
  return D == 64 ? launch<64>(mq, mk, mv, p, q_blocks, stream)
                 : launch<128>(mq, mk, mv, p, q_blocks, stream);
}

// As fb_gemm_tc_status, for the attention kernel of this file.
FB_API int fb_attention_tc_status(int* detail) {
  int host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(host, g_status, sizeof(host));
  if (e != cudaSuccess) return fb_fail(2, "attention_tc_status: %s", cudaGetErrorString(e));
  if (detail) { detail[0] = host[1]; detail[1] = host[2]; detail[2] = host[3]; }
  if (host[0]) {
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_status, zero, sizeof(zero));
  }
  return host[0] ? host[1] : 0;
}
