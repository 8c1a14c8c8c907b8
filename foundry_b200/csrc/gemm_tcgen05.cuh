// What the tcgen05 product kernels share (gemm_tcgen05.cu: one tile per CTA and
// the persistent form; gemm_tcgen05_pair.cu: two SMs per tile): tile constants,
// the launch parameters, the epilogue's store, and the host's tensor maps.
#pragma once

#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

// What a product whose A rows are tokens (stride_b == 1) may do beyond storing:
// apply the row scale of an input that is a norm's output without it, and, in
// front of a norm (epilogue 2), add its result to the float32 residual rows,
// leave resid * gamma in bfloat16 and every token's share of the sum of squares
// over this tile's features (gemm_skinny.cu has the same two for few rows).
struct FbRowExtras {
  const float* scale_ss;  // [scale_count, scale_stride] shares of the tokens' sums of squares;
                          // with scale_count == 0: the tokens' scales themselves; null: none
  int scale_count, scale_stride;
  float scale_inv_dim, scale_eps;
  float* resid;           // [rows_a, rows_b] float32, row stride ldr
  long long ldr;
  const float* gamma;     // [rows_b]
  __nv_bfloat16* xg;      // [rows_a, rows_b], row stride ldxg
  long long ldxg;
  float* ss_out;          // [feature tiles, ss_stride]
  int ss_stride;
};

// Epilogue 3, for the fused q/k/v projection with tokens as the A rows: feature
// j is element j % D of head j / D (A query heads, Kh key heads, Kh value
// heads). Queries and keys are rotated over neighbouring features (2i, 2i + 1)
// by frequency i with the cos and sin of `cs`; queries go to `q_out`, keys and
// values into the paged cache (rope_cache.cu has the formulas and the layout).
struct FbRopeExtras {
  const float2* cs;        // [half, rows_a]: (cos, sin) of frequency and token (a warp's 32
                           // tokens read one frequency's angles as 256 contiguous bytes)
  int half;                // rotary width / 2
  const int* positions;    // [rows_a]
  const int* seq_of_token; // [rows_a], -1: padding (nothing is written for it)
  const int* page_table;   // [sequences, max_pages]
  int max_pages, ring_pages;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  long long page_stride, head_stride;
  int A, Kh, D, write_cache;
  __nv_bfloat16* q_out;    // [rows_a, A * D], row stride ldq
  long long ldq;
};

struct FbGemmParams {
  int rows_a, rows_b, K;
  int kblocks_per_split;      // K blocks of BK each CTA of a tile walks
  long long stride_a, stride_b;  // out[i * stride_a + j * stride_b]
  long long split_stride;        // elements between split-K planes
  void* out;
  int out_f32;                // 1: float32 output, 0: bfloat16
  int constant_operand;       // 1: A holds constants (weights), 2: B does, 0: neither
  int epilogue;               // 0: store D; 1: SiLU(gate) * up over interleaved feature pairs;
                              // 2: residual add in front of a norm (`rows`)
                              // 3: rotation and cache write of a q/k/v projection (`rope`)
  FbRowExtras rows;
  FbRopeExtras rope;
  // paired form only: the tiles of the last, partly filled round are shared along K
  int full_tiles;             // tiles [0, full_tiles) are computed whole
  int tail_splits;            // K shares of every later tile (1: whole too)
  int tail_kblocks;           // K blocks per share
  float* partial;             // float32 partial sums of the shares (layout: see the kernel)
  int* tail_counters;         // [tail tile][8]: shares delivered per (CTA of the pair, epilogue warp)
};

// The paired form (gemm_tcgen05_pair.cu), called by fb_gemm_tc.
int fb_gemm_tc_pair(const void* a, long long lda, int rows_a, const void* b, long long ldb,
                    int rows_b, int bn, const FbGemmParams& p, void* workspace,
                    long long workspace_bytes, int* counters, int counters_len,
                    int share_min_kblocks, cudaStream_t stream);

namespace {

constexpr int BM = 128;            // rows of A per tile = instruction M
constexpr int BK = 64;             // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;         // K of one tcgen05.mma for 16-bit inputs
constexpr int THREADS = 192;       // 6 warps
using GemmParams = FbGemmParams;

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

// 1 / sqrt(mean square + eps) of token `i` from the shares the product in front left.
__device__ __forceinline__ float token_scale(const GemmParams& p, long long i) {
  if (p.rows.scale_ss == nullptr || i >= p.rows_a) return 1.f;
  if (p.rows.scale_count == 0) return __ldcg(p.rows.scale_ss + i);
  float sum = 0.f;
  for (int c = 0; c < p.rows.scale_count; ++c)
    sum += __ldcg(p.rows.scale_ss + (size_t)c * p.rows.scale_stride + i);
  return 1.0f / sqrtf(sum * p.rows.scale_inv_dim + p.rows.scale_eps);
}

// Epilogue 2 for CHUNK consecutive features (j0 ..) of token i: resid += v,
// xg = bf16(resid * gamma); returns the chunk's sum of resid^2.
template <int CHUNK>
__device__ __forceinline__ float sink_chunk(const GemmParams& p, const float (&v)[CHUNK],
                                            long long i, long long j0) {
  if (i >= p.rows_a) return 0.f;
  float* rp = p.rows.resid + i * p.rows.ldr + j0;
  __nv_bfloat16* xp = p.rows.xg + i * p.rows.ldxg + j0;
  const float* gp = p.rows.gamma + j0;
  float ss = 0.f;
  const bool vec = j0 + CHUNK <= p.rows_b && (((uintptr_t)rp | (uintptr_t)gp) % 16) == 0 &&
                   ((uintptr_t)xp % 8) == 0;
  if (vec) {
    float4 old[CHUNK / 4];
#pragma unroll
    for (int e = 0; e < CHUNK / 4; ++e) old[e] = __ldcg(reinterpret_cast<const float4*>(rp) + e);
#pragma unroll
    for (int e = 0; e < CHUNK / 4; ++e) {
      const float4 g = *(reinterpret_cast<const float4*>(gp) + e);
      float4 r;
      r.x = old[e].x + v[4 * e]; r.y = old[e].y + v[4 * e + 1];
      r.z = old[e].z + v[4 * e + 2]; r.w = old[e].w + v[4 * e + 3];
      *(reinterpret_cast<float4*>(rp) + e) = r;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x * g.x, r.y * g.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(r.z * g.z, r.w * g.w);
      uint2 pk;
      pk.x = *reinterpret_cast<const uint32_t*>(&lo);
      pk.y = *reinterpret_cast<const uint32_t*>(&hi);
      *(reinterpret_cast<uint2*>(xp) + e) = pk;
      ss += (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w);
    }
  } else {
#pragma unroll
    for (int e = 0; e < CHUNK; ++e) {
      if (j0 + e < p.rows_b) {
        const float r = __ldcg(rp + e) + v[e];
        rp[e] = r;
        xp[e] = __float2bfloat16_rn(r * gp[e]);
        ss += r * r;
      }
    }
  }
  return ss;
}

// Epilogue 3 for CHUNK consecutive features (j0 ..) of token i. The launcher
// makes sure that a chunk lies inside one head (D is a multiple of CHUNK) and
// that every store is 16 bytes on a 16-byte boundary.
template <int CHUNK>
__device__ __forceinline__ void rope_chunk(const GemmParams& p, float (&v)[CHUNK], long long i,
                                           long long j0) {
  const FbRopeExtras& r = p.rope;
  if (i >= p.rows_a || j0 >= p.rows_b) return;
  const int seq = r.seq_of_token[i];
  if (seq < 0) return;  // padding token
  const int head = (int)(j0 / r.D), e0 = (int)(j0 - (long long)head * r.D);
  if (head >= r.A && !r.write_cache) return;  // keys and values are not wanted
  if (head < r.A + r.Kh && e0 < 2 * r.half) {
    // pairs (e0 + 2q, e0 + 2q + 1) turn by frequency e0 / 2 + q while they lie inside the rotary width
    const float2* cs = r.cs + (size_t)(e0 >> 1) * p.rows_a + i;
    float2 c[CHUNK / 2];
#pragma unroll
    for (int q = 0; q < CHUNK / 2; ++q)  // all loads go out before the first is used
      c[q] = e0 + 2 * q < 2 * r.half ? __ldg(cs + (size_t)q * p.rows_a) : make_float2(1.f, 0.f);
#pragma unroll
    for (int q = 0; q < CHUNK / 2; ++q) {
      const float a = v[2 * q], b = v[2 * q + 1];
      v[2 * q] = a * c[q].x - b * c[q].y;
      v[2 * q + 1] = b * c[q].x + a * c[q].y;
    }
  }
  __nv_bfloat16* dst;
  if (head < r.A) {
    dst = r.q_out + i * r.ldq + j0;
  } else {
    const int pos = r.positions[i];
    int lp = pos / FB_PAGE;
    if (r.ring_pages > 0) lp %= r.ring_pages;
    const long long row = (long long)r.page_table[(size_t)seq * r.max_pages + lp] * r.page_stride +
                          (long long)(pos % FB_PAGE) * r.D + e0;
    dst = head < r.A + r.Kh ? r.k_cache + (long long)(head - r.A) * r.head_stride + row
                            : r.v_cache + (long long)(head - r.A - r.Kh) * r.head_stride + row;
  }
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
    *reinterpret_cast<uint4*>(dst + e) = pk;
  }
}

// A chunk of a tile's epilogue with the row extras: scale, then sink or store.
// Returns what the chunk adds to the token's sum of squares (epilogue 2, else 0).
template <int CHUNK>
__device__ __forceinline__ float finish_chunk(const GemmParams& p, float (&v)[CHUNK], float scale,
                                              long long i_global, long long j0, int lane,
                                              float* out_f, __nv_bfloat16* out_h) {
  if (p.rows.scale_ss != nullptr) {
#pragma unroll
    for (int e = 0; e < CHUNK; ++e) v[e] *= scale;
  }
  if (p.epilogue == 2) return sink_chunk<CHUNK>(p, v, i_global, j0);
  if (p.epilogue == 3) {
    rope_chunk<CHUNK>(p, v, i_global, j0);
    return 0.f;
  }
  store_chunk<CHUNK>(p, v, i_global, j0, lane, out_f, out_h);
  return 0.f;
}
// After a tile's last chunk: the token's share over this tile's features.
__device__ __forceinline__ void finish_tile(const GemmParams& p, float ss, long long i_global,
                                            int tile_b) {
  if (p.epilogue == 2 && i_global < p.rows_a)
    p.rows.ss_out[(size_t)tile_b * p.rows.ss_stride + i_global] = ss;
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

}  // namespace
