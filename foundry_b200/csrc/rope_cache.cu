// Rotary position encoding of queries and keys, fused with the write of the
// new keys and values into the paged cache.
//
// Formulas (reference, by its path in stratorys/foundry):
//   angle[p, i] = p * inv_freq[i], the position taken as a 32-bit float and the
//   product rounded once to 32 bits (src/models/llama/rotary_emb.rs:113-133);
//   rotate_half(x) = cat(-x[D/2:], x[:D/2]); x' = x*cos + rotate_half(x)*sin,
//   so element i pairs with i + D/2 (rotary_emb.rs:62-85);
//   cache write K[slot, :, p, :] = k', V[...] = v (src/nn/kv_cache.rs:73-74).
// The reference rounds cos and sin to 16 bits in a table; here they are
// computed in 32-bit from the angle, in the kernel.
//
// Layout: `qkv` is [T, (A + 2*Kh) * D] with row stride `qkv_stride`: A query
// heads, then Kh key heads, then Kh value heads. Queries are rotated in place.
// A cache page of one head is FB_PAGE rows of D elements; the page of position
// p is page_table[seq, (p / FB_PAGE) % ring] (ring = pages per sequence for a
// windowed group, else unbounded).
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long long qkv_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int max_pages,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     long long page_stride, long long head_stride, int ring_pages,
                                     int A, int Kh, int D, int write_cache) {
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) return;  // padding token
  const int pos = positions[t];
  T* row = qkv + (size_t)t * qkv_stride;
  const int half = rotary_dim >> 1;
  const float fpos = (float)pos;

  long long cache_row = 0;
  if (write_cache) {
    int lp = pos / FB_PAGE;
    if (ring_pages > 0) lp %= ring_pages;
    const int page = page_table[(size_t)seq * max_pages + lp];
    cache_row = (long long)page * page_stride + (long long)(pos % FB_PAGE) * D;
  }

  // rotated pairs of the query and key heads
  const int rot_heads = A + (write_cache ? Kh : 0);
  for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const float angle = fpos * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    T* x = row + (size_t)h * D;
    const float x1 = fb_to_float<T>(x[i]), x2 = fb_to_float<T>(x[i + half]);
    const float y1 = x1 * c - x2 * s;
    const float y2 = x2 * c + x1 * s;
    if (h < A) {
      x[i] = fb_from_float<T>(y1);
      x[i + half] = fb_from_float<T>(y2);
    } else {
      T* dst = k_cache + cache_row + (long long)(h - A) * head_stride;
      dst[i] = fb_from_float<T>(y1);
      dst[i + half] = fb_from_float<T>(y2);
    }
  }
  if (!write_cache) return;
  // key elements beyond the rotary part pass through unchanged
  const int tail = D - rotary_dim;
  for (int idx = threadIdx.x; idx < Kh * tail; idx += blockDim.x) {
    const int h = idx / tail, i = rotary_dim + (idx - h * tail);
    k_cache[cache_row + (long long)h * head_stride + i] = row[(size_t)(A + h) * D + i];
  }
  // values
  for (int idx = threadIdx.x; idx < Kh * D; idx += blockDim.x) {
    const int h = idx / D, i = idx - h * D;
    v_cache[cache_row + (long long)h * head_stride + i] = row[(size_t)(A + Kh + h) * D + i];
  }
}

FB_API int fb_rope_kv_write(void* qkv, int dtype, long long qkv_stride, const int* positions,
                            const int* seq_of_token, const int* page_table, int max_pages,
                            const float* inv_freq, int rotary_dim, void* k_cache, void* v_cache,
                            long long page_stride, long long head_stride, int ring_pages, int T,
                            int A, int Kh, int D, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && A > 0 && Kh > 0 && D > 0, "rope_kv_write: bad sizes T=%d A=%d Kh=%d D=%d",
             T, A, Kh, D);
  FB_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 2 == 0,
             "rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, D);
  FB_REQUIRE(qkv_stride >= (long long)(A + 2 * Kh) * D, "rope_kv_write: row stride too small");
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && max_pages > 0),
             "rope_kv_write: cache pointers missing");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (rope_kv_write_kernel<E><<<T, 256, 0, stream>>>(
      (E*)qkv, qkv_stride, positions, seq_of_token, page_table, max_pages, inv_freq, rotary_dim,
      (E*)k_cache, (E*)v_cache, page_stride, head_stride, ring_pages, A, Kh, D, write_cache)));
  return fb_check_launch("rope_kv_write");
}
