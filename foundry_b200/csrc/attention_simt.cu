// Causal grouped-query attention over the paged cache on the CUDA cores, in
// 32-bit arithmetic: the attention of the 32-bit path (prompts and single
// tokens alike) and the plain check of the tensor-core kernels.
//
// Formulas (reference, by its path in stratorys/foundry):
//   query head a reads key-value head a / (A / Kh)       (src/nn/attention.rs:40-44)
//   s[j] = (q . k_j) * 1/sqrt(D)                          (src/nn/attention.rs:45-55,
//                                                          src/models/llama/attention.rs:56-58)
//   key j is visible to the query at position p iff j <= p (src/nn/masking.rs:76-92)
//   p = softmax(s) with the maximum subtracted, in 32-bit  (src/nn/activation.rs:30-40)
//   o = sum_j p[j] * v_j                                   (src/nn/attention.rs:56-59)
// The reference materialises the score matrix and rounds scores and
// probabilities to 16 bits; here the softmax runs online over 32-key chunks and
// nothing between q.k and the output is rounded below 32 bits.
//
// One warp per (token, query head). A token's keys are the cache rows
// [lo, p] of its own sequence, lo = max(0, p - window + 1) when the layer group
// has a window. Each lane scores one key of a chunk; for the weighted sum the
// lanes own head elements lane, lane+32, ...
// Queries, keys and values are read with coherent (L2) loads: the kernel that
// wrote this step's rows may have overlapped this kernel's start.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* q, long long q_stride, T* __restrict__ out,
                      long long out_stride, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ page_table,
                      int max_pages, const T* k_cache, const T* v_cache,
                      long long page_stride, long long head_stride, int ring_pages, int window,
                      int A, int Kh, int D, float scale) {
  fb_pdl_wait();
  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int a = blockIdx.y * WARPS + warp;
  if (a >= A) return;
  const int seq = seq_of_token[t];
  T* o = out + (size_t)t * out_stride + (size_t)a * D;
  if (seq < 0) {  // padding token: defined output, no cache access
    for (int d = lane; d < D; d += 32) o[d] = fb_from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int kvh = a / (A / Kh);
  const T* qrow = q + (size_t)t * q_stride + (size_t)a * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = fb_load_coherent<T>(qrow + d);
  __syncwarp();

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* pages = page_table + (size_t)seq * max_pages;
  const T* kbase = k_cache + (long long)kvh * head_stride;
  const T* vbase = v_cache + (long long)kvh * head_stride;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    long long row_off = 0;
    if (j <= pos) {
      int lp = j / FB_PAGE;
      if (ring_pages > 0) lp %= ring_pages;
      row_off = (long long)pages[lp] * page_stride + (long long)(j % FB_PAGE) * D;
      const T* krow = kbase + row_off;
      float dot = 0.f;
      for (int d = 0; d < D; d += 8) {
        float kv[8];
        load8<T>(krow + d, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qs[warp][d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, fb_warp_max(s));
    const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first chunk
    const float p = (j <= pos) ? expf(s - m_new) : 0.f;
    l = l * corr + fb_warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
    const int n = min(32, pos - j0 + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long off = __shfl_sync(0xffffffffu, row_off, jj);
      const T* vrow = vbase + off;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, fb_load_coherent<T>(vrow + d), acc[i]);
      }
    }
  }
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) o[d] = fb_from_float<T>(acc[i] * inv_l);
  }
}
}  // namespace

FB_API int fb_attention_simt(const void* q, long long q_stride, void* out, long long out_stride,
                             int dtype, const int* positions, const int* seq_of_token,
                             const int* page_table, int max_pages, const void* k_cache,
                             const void* v_cache, long long page_stride, long long head_stride,
                             int ring_pages, int window, int T, int A, int Kh, int D, float scale,
                             cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && A > 0 && Kh > 0 && D > 0, "attention: bad sizes T=%d A=%d Kh=%d D=%d", T, A,
             Kh, D);
  FB_REQUIRE(A % Kh == 0, "attention: %d query heads are not a multiple of %d key-value heads", A,
             Kh);
  FB_REQUIRE(D % 16 == 0 && D <= MAX_D,
             "attention: head size %d is not a multiple of 16 up to %d", D, MAX_D);
  FB_REQUIRE(q_stride >= (long long)A * D && out_stride >= (long long)A * D,
             "attention: a row stride is too small");
  FB_REQUIRE(T <= 0x7fffffff / 1 && max_pages > 0, "attention: bad page table");
  if (T == 0) return 0;
  dim3 grid(T, (A + WARPS - 1) / WARPS);
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_simt_kernel<E>, dim3(grid), dim3(WARPS * 32), 0, stream, 
      (const E*)q, q_stride, (E*)out, out_stride, positions, seq_of_token, page_table, max_pages,
      (const E*)k_cache, (const E*)v_cache, page_stride, head_stride, ring_pages, window, A, Kh, D,
      scale)));
  return fb_check_launch("attention_simt");
}
