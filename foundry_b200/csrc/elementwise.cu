// Row-wise kernels around the matrix products: token embedding gather,
// residual add fused with RMS normalisation, SiLU(gate) * up, row gather.
//
// Formulas (reference file:line, by its path in stratorys/foundry):
//   embedding  x[t,:] = E[ids[t],:]; an id outside the table gives a zero row
//              (src/nn/linear.rs:54-69, src/metal/kernels/index_select.metal:23-26)
//   RMS norm   r = 1/sqrt(sum(x^2) * (1/H) + eps); y = x * r * w, in 32-bit
//              (src/nn/norm.rs:31-51)
//   residual   h = x + delta (src/models/llama/model.rs:272, 277); here the sum
//              is kept in 32-bit and never rounded to 16 bits
//   SiLU       a = g / (1 + exp(-g)) in 32-bit, then a * u
//              (src/nn/activation.rs:18-27, src/models/llama/mlp.rs:56)
#include "common.cuh"

// Four consecutive elements as float32.
template <typename TD>
__device__ __forceinline__ float4 load4(const TD* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V) {
  fb_pdl_launch();  // a few small blocks: the norm behind them may be placed at once
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + (size_t)id * H;
  if (H % 4 == 0 && (((uintptr_t)src | (uintptr_t)dst) % 16) == 0) {
    // groups of four elements; a thread's loads all go out before its first store
    constexpr int AHEAD = 4;
    for (int i0 = threadIdx.x * 4; i0 < H; i0 += blockDim.x * 4 * AHEAD) {
      float4 v[AHEAD];
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int i = i0 + a * blockDim.x * 4;
        if (i < H) v[a] = load4<T>(src + i);
      }
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int i = i0 + a * blockDim.x * 4;
        if (i < H) *reinterpret_cast<float4*>(dst + i) = v[a];
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = fb_to_float<T>(src[i]);
}

FB_API int fb_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T,
                           int H, int V, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
  if (T == 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  FB_DISPATCH_DTYPE(table_dtype, E, (fb_launch(embed_gather_kernel<E>, dim3(T), dim3(threads), 0, stream, 
                                        (const E*)table, ids, out, H, V)));
  return fb_check_launch("embed_gather");
}

// ------------------------------------------------- residual add + RMS norm
// resid[t,:] += delta[t,:] (if delta), then out[t,:] = resid * r * w.
// `delta` may be `planes` float32 partial results of a split-K product
// ([planes, T, H], `plane_stride` elements apart); they are summed in plane
// order, then added. One block per row; the row is re-read from `resid`, which
// the same thread wrote, so no synchronisation is needed between the passes.
// Each thread owns up to ITEMS groups of four consecutive elements; all loads of
// a group (the residual and every plane) are issued before any is used, so a
// row costs one round trip to memory, one block reduction and one store.
// Four elements as they lie in memory (bfloat16: two registers instead of four
// while they wait for their use), and their float32 values.
template <typename TD> struct Raw4;
template <> struct Raw4<float> { float4 bits; };
template <> struct Raw4<__nv_bfloat16> { uint2 bits; };
template <typename TD>
__device__ __forceinline__ Raw4<TD> load_raw4(const TD* p) {
  Raw4<TD> r;
  r.bits = *reinterpret_cast<const decltype(r.bits)*>(p);
  return r;
}
__device__ __forceinline__ float4 widen(const Raw4<float>& r) { return r.bits; }
__device__ __forceinline__ float4 widen(const Raw4<__nv_bfloat16>& r) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.bits.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.bits.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename TO>
__device__ __forceinline__ void store4(TO* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TD, typename TO, int ITEMS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* delta,
                                       int planes, long long plane_stride,
                                       const float* __restrict__ weight, TO* __restrict__ out,
                                       int H, float eps, float inv_h) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float scratch[32];
  const size_t row = (size_t)blockIdx.x * H;
  float* x = resid + row;
  float4 v[ITEMS];
  float ss = 0.f;
  if (delta != nullptr && planes == 1) {
    // One plane (every prompt step): the loads of all of a thread's groups go out
    // before the first store. `delta` is not known to be another buffer than
    // `resid`, so inside one loop a group's store would hold back the next group's
    // loads, and a row would cost a round trip to memory per group.
    Raw4<TD> raw[ITEMS];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int i = (threadIdx.x + it * blockDim.x) * 4;
      v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < H) {
        v[it] = load4<float>(x + i);
        raw[it] = load_raw4<TD>(delta + row + i);
      }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int i = (threadIdx.x + it * blockDim.x) * 4;
      if (i < H) {
        const float4 add = widen(raw[it]);
        v[it].x += add.x; v[it].y += add.y; v[it].z += add.z; v[it].w += add.w;
        store4<float>(x + i, v[it]);
        ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
      }
    }
  } else {
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < H) {
      v[it] = load4<float>(x + i);
      if (delta != nullptr) {
        const TD* d = delta + row + i;
        for (int s0 = 0; s0 < planes; s0 += 8) {
          float4 part[8];
#pragma unroll
          for (int s = 0; s < 8; ++s)
            part[s] = (s0 + s < planes) ? load4<TD>(d + (size_t)(s0 + s) * plane_stride)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
          float4 add = part[0];
#pragma unroll
          for (int s = 1; s < 8; ++s) {
            add.x += part[s].x; add.y += part[s].y; add.z += part[s].z; add.w += part[s].w;
          }
          v[it].x += add.x; v[it].y += add.y; v[it].z += add.z; v[it].w += add.w;
        }
        store4<float>(x + i, v[it]);
      }
      ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
    }
  }
  }
  ss = fb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss * inv_h + eps);
  if (out != nullptr) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int i = (threadIdx.x + it * blockDim.x) * 4;
      if (i < H) {
        const float4 w = load4<float>(weight + i);
        store4<TO>(out + row + i, make_float4(v[it].x * r * w.x, v[it].y * r * w.y,
                                              v[it].z * r * w.z, v[it].w * r * w.w));
      }
    }
  }
}

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* delta,
                                   int planes, long long plane_stride,
                                   const float* __restrict__ weight, TO* __restrict__ out, int H,
                                   float eps, float inv_h) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float scratch[32];
  const size_t row = (size_t)blockIdx.x * H;
  float* x = resid + row;
  float ss = 0.f;
  if (delta != nullptr) {
    const TD* d = delta + row;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float add = fb_to_float<TD>(d[i]);
      for (int s = 1; s < planes; ++s) add += fb_to_float<TD>(d[(size_t)s * plane_stride + i]);
      const float v = x[i] + add;
      x[i] = v;
      ss += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = x[i];
      ss += v * v;
    }
  }
  ss = fb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss * inv_h + eps);
  if (out != nullptr) {
    TO* y = out + row;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      y[i] = fb_from_float<TO>(x[i] * r * weight[i]);
  }
}

FB_API int fb_add_rmsnorm(float* resid, const void* delta, int delta_dtype, int planes,
                          long long plane_stride, const float* weight, float eps, void* out,
                          int out_dtype, int T, int H, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0, "add_rmsnorm: bad sizes T=%d H=%d", T, H);
  FB_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
  FB_REQUIRE(planes >= 1 && (planes == 1 || delta_dtype == FB_F32),
             "add_rmsnorm: split planes are float32");
  if (T == 0) return 0;
  const float inv_h = 1.0f / (float)H;
  // vector path: rows of whole float4 groups on 16-byte boundaries, at most 4 groups a thread
  const bool aligned = H % 4 == 0 && ((uintptr_t)resid % 16) == 0 && ((uintptr_t)weight % 16) == 0 &&
                       ((uintptr_t)delta % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                       plane_stride % 4 == 0;
  if (aligned && H <= 4 * 4 * 1024) {
    const int groups = H / 4;
    // few rows: wide blocks make a row's latency short; many rows: narrower blocks
    // with more loads in flight per thread keep more rows resident per SM
    // (the block width decides the order of a row's sum: "many" begins above 512 rows,
    // the largest step that is also run padded to a bucket, so that a step and its
    // padded form take the same width)
    int threads = groups <= 128 ? 128 : groups <= 512 ? 256 : groups <= 1024 ? 512 : 1024;
    if (T > 512 && groups <= 1024) threads = groups <= 512 ? 128 : 256;
    const int items = (groups + threads - 1) / threads;
#define FB_NORM_LAUNCH(N)                                                                     \
    FB_DISPATCH_DTYPE(delta_dtype, TD, FB_DISPATCH_DTYPE(out_dtype, TO, (                     \
        fb_launch(add_rmsnorm_vec_kernel<TD, TO, N>, dim3(T), dim3(threads), 0, stream,                          \
            resid, (const TD*)delta, planes, plane_stride, weight, (TO*)out, H, eps, inv_h))))
    if (items <= 1) { FB_NORM_LAUNCH(1); }
    else if (items == 2) { FB_NORM_LAUNCH(2); }
    else { FB_NORM_LAUNCH(4); }
#undef FB_NORM_LAUNCH
    return fb_check_launch("add_rmsnorm");
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  FB_DISPATCH_DTYPE(delta_dtype, TD, FB_DISPATCH_DTYPE(out_dtype, TO, (
      fb_launch(add_rmsnorm_kernel<TD, TO>, dim3(T), dim3(threads), 0, stream, 
          resid, (const TD*)delta, planes, plane_stride, weight, (TO*)out, H, eps, inv_h))));
  return fb_check_launch("add_rmsnorm");
}

// ------------------------------------------------- a deferred norm's row scale
// out[t, i] = values[t, i] / sqrt(sum_c shares[c * stride + t] / dim + eps): the
// plain tensor of a norm whose scale the weight-streaming products would have
// applied themselves (gemm_skinny.cu), for a consumer that is none of them.
__global__ void apply_row_scale_kernel(const __nv_bfloat16* values, long long ld,
                                       const float* shares, int count, int stride, float inv_dim,
                                       float eps, __nv_bfloat16* __restrict__ out, long long ldo,
                                       int H) {
  fb_pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float sum = 0.f;
  for (int c = threadIdx.x; c < count; c += blockDim.x) sum += shares[(size_t)c * stride + t];
  sum = fb_block_sum(sum, scratch);
  const float r = 1.0f / sqrtf(sum * inv_dim + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[t * ldo + i] = __float2bfloat16_rn(__bfloat162float(values[t * ld + i]) * r);
}

FB_API int fb_apply_row_scale(const void* values, long long ld, const float* shares, int count,
                              int stride, int dim, float eps, void* out, long long ldo, int T,
                              int H, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && count > 0 && stride >= T && dim > 0 && eps > 0.f,
             "apply_row_scale: bad sizes T=%d H=%d count=%d stride=%d", T, H, count, stride);
  if (T == 0) return 0;
  fb_launch(apply_row_scale_kernel, dim3(T), dim3(256), 0, stream,
            (const __nv_bfloat16*)values, ld, shares, count, stride, 1.0f / (float)dim, eps,
            (__nv_bfloat16*)out, ldo, H);
  return fb_check_launch("apply_row_scale");
}

// Every token's 1 / sqrt(mean square + eps) from the shares of its sum of squares
// that the product in front of a norm left: out[t] for t < T. For products of many
// rows, whose epilogues would otherwise add the shares up again for every tile.
__global__ void row_scales_kernel(const float* shares, int count, int stride, float inv_dim,
                                  float eps, float* __restrict__ out, int T) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float sum = 0.f;
  int c = 0;
  for (; c + 8 <= count; c += 8) {  // eight loads on their way together, added in order
    float part[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) part[e] = __ldcg(shares + (size_t)(c + e) * stride + t);
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += part[e];
  }
  for (; c < count; ++c) sum += __ldcg(shares + (size_t)c * stride + t);
  out[t] = 1.0f / sqrtf(sum * inv_dim + eps);
}

FB_API int fb_row_scales(const float* shares, int count, int stride, int dim, float eps,
                         float* out, int T, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && count > 0 && stride >= T && dim > 0 && eps > 0.f,
             "row_scales: bad sizes T=%d count=%d stride=%d", T, count, stride);
  if (T == 0) return 0;
  fb_launch(row_scales_kernel, dim3((T + 127) / 128), dim3(128), 0, stream, shares, count, stride,
            1.0f / (float)dim, eps, out, T);
  return fb_check_launch("row_scales");
}

// ------------------------------------------------------------- SiLU(g) * u
// gate_up is [T, 2I]. Plain layout: columns [0, I) hold the gate, [I, 2I) the
// up projection. Interleaved layout: column 2i holds gate i, column 2i+1 up i
// (the layout the fused product epilogue uses).
template <typename T>
__global__ void silu_mul_kernel(const T* gate_up, T* __restrict__ out, int I,
                                size_t total, int interleaved) {
  fb_pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const T* row = gate_up + t * 2 * I;
    const float g = fb_to_float<T>(interleaved ? row[2 * i] : row[i]);
    const float u = fb_to_float<T>(interleaved ? row[2 * i + 1] : row[I + i]);
    const float a = g / (1.0f + expf(-g));
    out[idx] = fb_from_float<T>(a * u);
  }
}

FB_API int fb_silu_mul(const void* gate_up, void* out, int dtype, int T, int I, int interleaved,
                       cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && I > 0, "silu_mul: bad sizes T=%d I=%d", T, I);
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(silu_mul_kernel<E>, dim3(blocks), dim3(threads), 0, stream, 
                                  (const E*)gate_up, (E*)out, I, total, interleaved)));
  return fb_check_launch("silu_mul");
}

// ---------------------------------------------------------------- row gather
// dst[r,:] = src[rows[r],:]; a negative row index gives a zero row.
template <typename T>
__global__ void gather_rows_kernel(const T* src, const int* __restrict__ rows,
                                   T* __restrict__ dst, int H) {
  fb_pdl_wait();
  const int r = blockIdx.x;
  const int s = rows[r];
  T* d = dst + (size_t)r * H;
  if (s < 0) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = fb_from_float<T>(0.f);
    return;
  }
  const T* p = src + (size_t)s * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = p[i];
}

FB_API int fb_gather_rows(const void* src, int dtype, const int* rows, void* dst, int n, int H,
                          cudaStream_t stream) {
  FB_REQUIRE(n >= 0 && H > 0, "gather_rows: bad sizes n=%d H=%d", n, H);
  if (n == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(gather_rows_kernel<E>, dim3(n), dim3(256), 0, stream, 
                                  (const E*)src, rows, (E*)dst, H)));
  return fb_check_launch("gather_rows");
}

// ----------------------------------------------------------------------- cast
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* in, TO* __restrict__ out, size_t n) {
  fb_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = fb_from_float<TO>(fb_to_float<TI>(in[i]));
}

FB_API int fb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                   cudaStream_t stream) {
  FB_REQUIRE(n >= 0, "cast: negative count");
  if (n == 0) return 0;
  const size_t want = ((size_t)n + 255) / 256;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, TO, (
      fb_launch(cast_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)in, (TO*)out, (size_t)n))));
  return fb_check_launch("cast");
}

// ------------------------------------------------------- sum of split-K planes
// out[i] = sum_s planes[s * plane_stride + i], planes in float32, summed in
// plane order (a fixed order: the result does not depend on timing).
template <typename TO>
__global__ void sum_planes_kernel(const float* planes, int S, long long n,
                                  long long plane_stride, TO* __restrict__ out) {
  fb_pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float acc = planes[i];
    for (int s = 1; s < S; ++s) acc += planes[(long long)s * plane_stride + i];
    out[i] = fb_from_float<TO>(acc);
  }
}

FB_API int fb_sum_planes(const float* planes, int S, long long n, long long plane_stride,
                         void* out, int out_dtype, cudaStream_t stream) {
  FB_REQUIRE(S >= 1 && n >= 0, "sum_planes: bad sizes S=%d n=%lld", S, n);
  if (n == 0) return 0;
  const long long want = (n + 255) / 256;
  const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
  FB_DISPATCH_DTYPE(out_dtype, TO, (fb_launch(sum_planes_kernel<TO>, dim3(blocks), dim3(256), 0, stream, 
                                       planes, S, n, plane_stride, (TO*)out)));
  return fb_check_launch("sum_planes");
}
