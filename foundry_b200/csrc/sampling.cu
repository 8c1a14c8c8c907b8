// Token selection on the device: greedy argmax and temperature sampling.
//
// Greedy: the index of the largest logit; among equal logits the lowest index
// wins (src/generate/mod.rs:192-204, src/metal/kernels/reduce.metal:42-78).
// The reference samples in no other way. Temperature sampling is added with the
// Gumbel-max rule: argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)), which
// draws from softmax(logits / T) without a cumulative sum. u_i is a pure
// function of (seed, sequence key, step, i), so a sequence's draws do not depend
// on the batch it runs in, and the host can restate them.
#include "common.cuh"

namespace {
__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  // the SplitMix64 finaliser (src/bench/rng.rs:21-27 uses the same constants)
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  return z ^ (z >> 31);
}
constexpr unsigned long long GOLDEN = 0x9e3779b97f4a7c15ULL;

// `stream` is mix64(seed + GOLDEN * (key + 1)), formed on the host once per
// sequence, so that no launch argument changes from step to step.
__device__ __forceinline__ float uniform24(unsigned long long stream, unsigned long long step,
                                           unsigned long long i) {
  unsigned long long z = mix64(stream + GOLDEN * (step + 1));
  z = mix64(z + GOLDEN * (i + 1));
  return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1), exact in 32-bit
}

// temperature[r] == 0 selects greedily. streams/steps may be null when every
// temperature is 0. Block (r, c) scans chunk c of row r and leaves its best
// (score, index); with one chunk per row it writes the token itself.
__global__ void __launch_bounds__(1024)
select_tokens_kernel(const float* logits, long long row_stride, int V, int chunk,
                     const float* __restrict__ temperature,
                     const long long* __restrict__ streams, const long long* __restrict__ steps,
                     float* __restrict__ part_val, int* __restrict__ part_idx,
                     int* __restrict__ out) {
  fb_pdl_wait();
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int r = blockIdx.x, c = blockIdx.y, chunks = gridDim.y;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature ? temperature[r] : 0.f;
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.f : 1.0f / temp;
  const unsigned long long stream = (!greedy && streams) ? (unsigned long long)streams[r] : 0ULL;
  const unsigned long long step = (!greedy && steps) ? (unsigned long long)steps[r] : 0ULL;
  const int lo = c * chunk, hi = min(V, lo + chunk);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  // a thread's next eight values are asked for together, then compared in order
  constexpr int AHEAD = 8;
  for (int i0 = lo + threadIdx.x; i0 < hi; i0 += blockDim.x * AHEAD) {
    float got[AHEAD];
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int i = i0 + a * (int)blockDim.x;
      got[a] = i < hi ? row[i] : 0.f;
    }
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int i = i0 + a * (int)blockDim.x;
      if (i >= hi) break;
      float v = got[a];
      if (!greedy) {
        const float u = uniform24(stream, step, (unsigned long long)i);
        v = v * inv_t - logf(-logf(u));
      }
      // indices ascend within a thread, so `>` keeps the first of equal values;
      // a NaN compares false and never wins
      if (v == v && (bi == 0x7fffffff || v > bv)) { bv = v; bi = i; }
    }
  }
  // reduce (value, index): larger value, then lower index
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
      bv = ov; bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    bv = lane < nwarps ? best_v[lane] : -INFINITY;
    bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov; bi = oi;
      }
    }
    if (lane == 0) {
      if (chunks == 1) {
        out[r] = (bi == 0x7fffffff) ? 0 : bi;
      } else {
        part_val[(size_t)r * chunks + c] = bv;
        part_idx[(size_t)r * chunks + c] = bi;
      }
    }
  }
}

// One warp per row merges the chunk results (chunks <= 1024).
__global__ void select_merge_kernel(const float* part_val,
                                    const int* part_idx, int chunks,
                                    int* __restrict__ out) {
  fb_pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < chunks; c += 32) {
    const float ov = part_val[(size_t)r * chunks + c];
    const int oi = part_idx[(size_t)r * chunks + c];
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
      bv = ov; bi = oi;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
      bv = ov; bi = oi;
    }
  }
  if (lane == 0) out[r] = (bi == 0x7fffffff) ? 0 : bi;
}
}  // namespace

// `chunks` blocks share each row; with chunks > 1 the two workspaces hold
// n * chunks entries and a second small kernel merges them.
FB_API int fb_select_tokens(const float* logits, long long row_stride, int n, int V,
                            const float* temperature, const long long* streams,
                            const long long* steps, int* out, int chunks, float* part_val,
                            int* part_idx, cudaStream_t stream) {
  FB_REQUIRE(n >= 0 && V > 0 && row_stride >= V, "select_tokens: bad sizes n=%d V=%d", n, V);
  FB_REQUIRE(chunks >= 1 && chunks <= 1024 && (chunks == 1 || (part_val && part_idx)),
             "select_tokens: bad chunk count %d or missing workspaces", chunks);
  if (n == 0) return 0;
  const int chunk = (V + chunks - 1) / chunks;
  const int threads = chunk >= 8192 ? 1024 : 256;
  fb_launch(select_tokens_kernel, dim3(dim3(n, chunks)), dim3(threads), 0, stream, 
      logits, row_stride, V, chunk, temperature, streams, steps, part_val, part_idx, out);
  int rc = fb_check_launch("select_tokens");
  if (rc || chunks == 1) return rc;
  fb_launch(select_merge_kernel, dim3(n), dim3(32), 0, stream, part_val, part_idx, chunks, out);
  return fb_check_launch("select_merge");
}
