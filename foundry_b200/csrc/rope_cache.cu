// Rotary position encoding of queries and keys, fused with the write of the
// new keys and values into the paged cache.
//
// Formulas (reference, by its path in stratorys/foundry):
//   angle[p, i] = p * inv_freq[i], the position taken as a 32-bit float and the
//   product rounded once to 32 bits (src/models/llama/rotary_emb.rs:113-133);
//   rotate_half(x) = cat(-x[D/2:], x[:D/2]); x' = x*cos + rotate_half(x)*sin,
//   so element i pairs with i + D/2 (rotary_emb.rs:62-85); the pairing is a
//   parameter: `interleaved` turns elements (2i, 2i + 1) by frequency i instead,
//   the other convention in use for this encoding;
//   cache write K[slot, :, p, :] = k', V[...] = v (src/nn/kv_cache.rs:73-74).
// The reference rounds cos and sin to 16 bits in a table; here they are
// computed in 32-bit from the angle, in the kernel.
//
// Layout: the fused projection output is [T, (A + 2*Kh) * D]: A query heads,
// then Kh key heads, then Kh value heads.
// A cache page of one head is FB_PAGE rows of D elements; the page of position
// p is page_table[seq, (p / FB_PAGE) % ring] (ring = pages per sequence for a
// windowed group, else unbounded).
#include "common.cuh"

// `src` is the fused projection output: T elements, or float32 when it is
// `planes` partial results of a split-K product (summed here in plane order).
// Rotated queries go to `q_out` (row stride q_stride), which may be `src`
// itself when the types agree.
template <typename TS, typename T>
__global__ void rope_kv_write_kernel(const TS* src, long long src_stride, int planes,
                                     long long plane_stride, T* __restrict__ q_out,
                                     long long q_stride, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int max_pages,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     long long page_stride, long long head_stride, int ring_pages,
                                     int A, int Kh, int D, int write_cache, int interleaved) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float s_cos[128], s_sin[128];  // rotary_dim / 2 <= 128 (head sizes up to 256)
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) return;  // padding token
  const int pos = positions[t];
  const TS* row = src + (size_t)t * src_stride;
  T* qrow = q_out + (size_t)t * q_stride;
  const int half = rotary_dim >> 1;
  const float fpos = (float)pos;
  // the angles depend on the position only: computed once, used by every head
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = fpos * inv_freq[i];
    sincosf(angle, &s_sin[i], &s_cos[i]);
  }
  __syncthreads();
  // sums the planes of two elements; the loads of a group of planes are issued together
  auto load2 = [&](int i0, int i1, float& a, float& b) {
    a = 0.f;
    b = 0.f;
    for (int s0 = 0; s0 < planes; s0 += 4) {
      float pa[4], pb[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const bool ok = s0 + s < planes;
        pa[s] = ok ? fb_to_float<TS>(row[(size_t)(s0 + s) * plane_stride + i0]) : 0.f;
        pb[s] = ok ? fb_to_float<TS>(row[(size_t)(s0 + s) * plane_stride + i1]) : 0.f;
      }
#pragma unroll
      for (int s = 0; s < 4; ++s) { a += pa[s]; b += pb[s]; }
    }
  };

  long long cache_row = 0;
  if (write_cache) {
    int lp = pos / FB_PAGE;
    if (ring_pages > 0) lp %= ring_pages;
    const int page = page_table[(size_t)seq * max_pages + lp];
    cache_row = (long long)page * page_stride + (long long)(pos % FB_PAGE) * D;
  }

  // One index space over everything a token needs: rotated pairs of the query
  // and key heads, then pairs of value elements, then the elements beyond the
  // rotary part. The blocks of a token (gridDim.y) stride through it.
  const int rot_heads = A + (write_cache ? Kh : 0);
  const int n_rot = rot_heads * half;
  const int n_val = write_cache ? Kh * (D / 2) : 0;
  const int tail = D - rotary_dim;
  const bool copy_q_tail = tail > 0 && ((const void*)src != (const void*)q_out || planes > 1);
  const int n_tail = (tail / 2) * ((copy_q_tail ? A : 0) + (write_cache ? Kh : 0));
  const int total = n_rot + n_val + n_tail;
  for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < total;
       idx += gridDim.y * blockDim.x) {
    if (idx < n_rot) {
      const int h = idx / half, i = idx - h * half;
      const float s = s_sin[i], c = s_cos[i];
      // the pair that frequency i turns: (i, i + half), or (2i, 2i + 1) when interleaved
      const int e1 = interleaved ? 2 * i : i, e2 = interleaved ? 2 * i + 1 : i + half;
      float x1, x2;
      load2(h * D + e1, h * D + e2, x1, x2);
      const float y1 = x1 * c - x2 * s;
      const float y2 = x2 * c + x1 * s;
      if (h < A) {
        qrow[h * D + e1] = fb_from_float<T>(y1);
        qrow[h * D + e2] = fb_from_float<T>(y2);
      } else {
        T* dst = k_cache + cache_row + (long long)(h - A) * head_stride;
        dst[e1] = fb_from_float<T>(y1);
        dst[e2] = fb_from_float<T>(y2);
      }
    } else if (idx < n_rot + n_val) {
      const int j = idx - n_rot;
      const int h = j / (D / 2), i = 2 * (j - h * (D / 2));
      float a, b;
      load2((A + Kh + h) * D + i, (A + Kh + h) * D + i + 1, a, b);
      T* dst = v_cache + cache_row + (long long)h * head_stride + i;
      dst[0] = fb_from_float<T>(a);
      dst[1] = fb_from_float<T>(b);
    } else {
      const int j = idx - n_rot - n_val;
      int h = j / (tail / 2);
      const int i = rotary_dim + 2 * (j - h * (tail / 2));
      if (!copy_q_tail) h += A;  // only key heads have tails to move
      float a, b;
      load2(h * D + i, h * D + i + 1, a, b);
      if (h < A) {
        qrow[h * D + i] = fb_from_float<T>(a);
        qrow[h * D + i + 1] = fb_from_float<T>(b);
      } else {
        T* dst = k_cache + cache_row + (long long)(h - A) * head_stride + i;
        dst[0] = fb_from_float<T>(a);
        dst[1] = fb_from_float<T>(b);
      }
    }
  }
}

// The common prompt case, vectorised: bfloat16 source rotated in place, no
// planes, rotary width == head size, head size a multiple of 16. A thread moves
// 8 consecutive elements of the first half and the 8 they pair with (16 bytes
// each way), or, with interleaved pairs, 8 consecutive elements that are four
// pairs of their own; or 8 consecutive value elements.
template <bool INTERLEAVED>
__global__ void rope_kv_write_bf16_kernel(__nv_bfloat16* __restrict__ qkv, long long stride,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ seq_of_token,
                                          const int* __restrict__ page_table, int max_pages,
                                          const float* __restrict__ inv_freq,
                                          __nv_bfloat16* __restrict__ k_cache,
                                          __nv_bfloat16* __restrict__ v_cache,
                                          long long page_stride, long long head_stride,
                                          int ring_pages, int A, int Kh, int D, int write_cache) {
  __shared__ float s_cos[128], s_sin[128];
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int half = D >> 1;
  const float fpos = (float)pos;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(fpos * inv_freq[i], &s_sin[i], &s_cos[i]);
  __syncthreads();
  __nv_bfloat16* row = qkv + (size_t)t * stride;
  long long cache_row = 0;
  if (write_cache) {
    int lp = pos / FB_PAGE;
    if (ring_pages > 0) lp %= ring_pages;
    const int page = page_table[(size_t)seq * max_pages + lp];
    cache_row = (long long)page * page_stride + (long long)(pos % FB_PAGE) * D;
  }
  const int groups = (INTERLEAVED ? D : half) / 8;   // work items per rotated head
  const int n_rot = (A + (write_cache ? Kh : 0)) * groups;
  const int n_val = write_cache ? Kh * (D / 8) : 0;  // 8-element groups of the value heads
  for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < n_rot + n_val;
       idx += gridDim.y * blockDim.x) {
    if (idx < n_rot) {
      const int h = idx / groups, i0 = (idx - h * groups) * 8;
      __nv_bfloat16* x = row + (size_t)h * D + i0;
      __nv_bfloat16* dst = h < A ? x : k_cache + cache_row + (long long)(h - A) * head_stride + i0;
      if constexpr (INTERLEAVED) {
        const uint4 in = *reinterpret_cast<const uint4*>(x);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&in);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {  // elements i0 + 2e, i0 + 2e + 1 turn by frequency i0 / 2 + e
          const float2 a = __bfloat1622float2(p2[e]);
          const float c = s_cos[(i0 >> 1) + e], sn = s_sin[(i0 >> 1) + e];
          o2[e] = __floats2bfloat162_rn(a.x * c - a.y * sn, a.y * c + a.x * sn);
        }
        *reinterpret_cast<uint4*>(dst) = o;
      } else {
        const uint4 lo = *reinterpret_cast<const uint4*>(x);
        const uint4 hi = *reinterpret_cast<const uint4*>(x + half);
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
        uint4 olo, ohi;
        __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&olo);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ohi);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(l2[e]), b = __bfloat1622float2(h2[e]);
          const float c0 = s_cos[i0 + 2 * e], s0 = s_sin[i0 + 2 * e];
          const float c1 = s_cos[i0 + 2 * e + 1], s1 = s_sin[i0 + 2 * e + 1];
          ol[e] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
          oh[e] = __floats2bfloat162_rn(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
        }
        *reinterpret_cast<uint4*>(dst) = olo;
        *reinterpret_cast<uint4*>(dst + half) = ohi;
      }
    } else {
      const int j = idx - n_rot;
      const int h = j / (D / 8), i0 = (j - h * (D / 8)) * 8;
      *reinterpret_cast<uint4*>(v_cache + cache_row + (long long)h * head_stride + i0) =
          *reinterpret_cast<const uint4*>(row + (size_t)(A + Kh + h) * D + i0);
    }
  }
}

// src_dtype / planes: see the kernel. dtype is the element type of q_out and the cache.
// interleaved: 0 pairs element i with i + rotary_dim / 2, 1 pairs 2i with 2i + 1.
FB_API int fb_rope_kv_write(const void* src, int src_dtype, long long src_stride, int planes,
                            long long plane_stride, void* q_out, int dtype, long long q_stride,
                            const int* positions, const int* seq_of_token, const int* page_table,
                            int max_pages, const float* inv_freq, int rotary_dim, void* k_cache,
                            void* v_cache, long long page_stride, long long head_stride,
                            int ring_pages, int T, int A, int Kh, int D, int write_cache,
                            int interleaved, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && A > 0 && Kh > 0 && D > 0, "rope_kv_write: bad sizes T=%d A=%d Kh=%d D=%d",
             T, A, Kh, D);
  FB_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 2 == 0,
             "rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, D);
  FB_REQUIRE(src_stride >= (long long)(A + 2 * Kh) * D && q_stride >= (long long)A * D,
             "rope_kv_write: a row stride is too small");
  FB_REQUIRE(planes >= 1 && (planes == 1 || src_dtype == FB_F32),
             "rope_kv_write: split planes are float32");
  FB_REQUIRE(src_dtype == dtype || src_dtype == FB_F32,
             "rope_kv_write: the source is the output type or float32");
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && max_pages > 0),
             "rope_kv_write: cache pointers missing");
  if (T == 0) return 0;
  FB_REQUIRE(D % 2 == 0 && rotary_dim <= 256,
             "rope_kv_write: head_dim %d must be even and the rotary width %d at most 256", D,
             rotary_dim);
  // few tokens: several blocks per token so that the step's latency is one round trip
  const int work = (A + 2 * Kh) * D / 2;
  int per_token = T >= 256 ? 1 : (work + 255) / 256;
  if (per_token > 16) per_token = 16;
  dim3 grid(T, per_token);
  if (dtype == FB_BF16 && src_dtype == FB_BF16 && planes == 1 && src == q_out &&
      rotary_dim == D && D % 16 == 0 && src_stride % 8 == 0 && ((uintptr_t)src % 16) == 0 &&
      page_stride % 8 == 0 && head_stride % 8 == 0 && ((uintptr_t)k_cache % 16) == 0 &&
      ((uintptr_t)v_cache % 16) == 0) {
    const int vec_work = (A + 2 * Kh) * D / 16;
    int blocks_y = T >= 256 ? 1 : (vec_work + 127) / 128;
    if (blocks_y > 16) blocks_y = 16;
    if (interleaved)
      fb_launch(rope_kv_write_bf16_kernel<true>, dim3(T, blocks_y), dim3(128), 0, stream,
                (__nv_bfloat16*)q_out, src_stride, positions, seq_of_token, page_table, max_pages,
                inv_freq, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_stride,
                head_stride, ring_pages, A, Kh, D, write_cache);
    else
      fb_launch(rope_kv_write_bf16_kernel<false>, dim3(T, blocks_y), dim3(128), 0, stream,
                (__nv_bfloat16*)q_out, src_stride, positions, seq_of_token, page_table, max_pages,
                inv_freq, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_stride,
                head_stride, ring_pages, A, Kh, D, write_cache);
    return fb_check_launch("rope_kv_write");
  }
#define FB_ROPE_LAUNCH(TS, TT)                                                                  \
  fb_launch(rope_kv_write_kernel<TS, TT>, dim3(grid), dim3(128), 0, stream,                                        \
      (const TS*)src, src_stride, planes, plane_stride, (TT*)q_out, q_stride, positions,        \
      seq_of_token, page_table, max_pages, inv_freq, rotary_dim, (TT*)k_cache, (TT*)v_cache,    \
      page_stride, head_stride, ring_pages, A, Kh, D, write_cache, interleaved ? 1 : 0)
  if (dtype == FB_F32) {
    FB_ROPE_LAUNCH(float, float);
  } else if (dtype == FB_BF16 && src_dtype == FB_BF16) {
    FB_ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else if (dtype == FB_BF16) {
    FB_ROPE_LAUNCH(float, __nv_bfloat16);
  } else {
    return fb_fail(1, "rope_kv_write: unknown element type code %d", dtype);
  }
#undef FB_ROPE_LAUNCH
  return fb_check_launch("rope_kv_write");
}

// ---------------------------------------------------------------- the angles of a step
// cs[i, t] = (cos, sin) of positions[t] * inv_freq[i], the product rounded once to 32
// bits as above: what a product kernel that rotates in its epilogue reads instead of
// computing the same angles once per head and layer. The positions are the same for
// every layer of a step, so one table serves them all.
__global__ void rope_table_kernel(const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int T, int half,
                                  float2* __restrict__ cs) {
  fb_pdl_launch();
  fb_pdl_wait();
  const long long n = (long long)T * half;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx / T), t = (int)(idx - (long long)i * T);  // tokens run fastest
    float sn, c;
    sincosf((float)positions[t] * inv_freq[i], &sn, &c);
    cs[idx] = make_float2(c, sn);
  }
}

FB_API int fb_rope_table(const int* positions, const float* inv_freq, int T, int half, void* cs,
                         cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && half >= 0, "rope_table: bad sizes T=%d half=%d", T, half);
  FB_REQUIRE(((uintptr_t)cs % 8) == 0, "rope_table: the table must be 8-byte aligned");
  if (T == 0 || half == 0) return 0;
  const long long n = (long long)T * half;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  fb_launch(rope_table_kernel, dim3(blocks), dim3(256), 0, stream, positions, inv_freq, T, half,
            (float2*)cs);
  return fb_check_launch("rope_table");
}
