// bfloat16 product for a handful of tokens (up to 16): out[t, n] = sum_k x[t,k] w[n,k].
//
// With so few tokens a projection (src/nn/linear.rs:19-36) is a stream of
// weights through the chip: every weight byte is used once, for `tokens`
// multiply-adds. This kernel is shaped for that. A CTA owns 16 weight rows;
// its warps split K among themselves; every thread pulls 32 contiguous bytes
// from each of its two rows per 64-element chunk, straight from global memory
// into the registers of the tensor-core instruction's A operand
// (mma.sync.m16n8k16, bf16 -> f32), several chunks in flight. The tokens are
// the instruction's narrow N. The K index inside a chunk is permuted so that a
// thread's 16 consecutive weights are what the instruction expects from it;
// the same permutation is applied to x, so the sum is unchanged. At the end the
// warps' partial sums meet in shared memory and the CTA writes its 16 output
// features for every token (optionally as SiLU(gate) * up over row pairs).
// No shared-memory staging of weights, no barriers in the main loop, no
// workspace in global memory.
//
// A third epilogue serves the fused q/k/v projection of an attention layer: it
// rotates the query and key heads by the position encoding and writes the new
// keys and values straight into their cache pages (what rope_cache.cu does as
// a kernel of its own for longer steps; formulas and layout are described
// there). For that a CTA's 16 rows are 8 rows of a head and the 8 rows they
// pair with in the rotation, so that a thread's two accumulator rows are a
// rotation pair and nothing crosses CTAs.
//
// Larger token counts run on the tcgen05 kernel (gemm_tcgen05.cu).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) {
  uint4 v;
  // Not the non-coherent path: the kernel that writes x may still have been
  // running when this kernel's blocks were placed (dependent launch), and a
  // non-coherent load may then return what the address held before.
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int CHUNK = 64;   // K elements per step of a warp

// What the rotary epilogue needs; unused (zeros) for the other epilogues.
struct RopeWrite {
  const int* positions;     // [T]
  const int* seq_of_token;  // [T], -1 = padding
  const int* page_table;    // [n_seqs, max_pages]
  int max_pages;
  const float* inv_freq;    // [rotary_dim / 2]
  int rotary_dim;           // a multiple of 16, at most D
  __nv_bfloat16* q_out;     // [T, A * D], row stride q_stride
  long long q_stride;
  __nv_bfloat16* k_cache;   // pages [*, Kh, FB_PAGE, D]
  __nv_bfloat16* v_cache;
  long long page_stride, head_stride;
  int ring_pages;           // pages per sequence of a windowed group, else 0
  int A, Kh, D;             // weight rows are A query, Kh key, Kh value heads of D
  int write_cache;          // 0: keys and values are not computed at all
};
struct NoRope {};
template <bool ROPE> struct RopeArg { using type = NoRope; };
template <> struct RopeArg<true> { using type = RopeWrite; };

// NT: token tiles of 8 (1 or 2). WARPS: warps per CTA, each with a K range.
// UNROLL: chunks whose loads are in flight together.
// No register cap beyond the block size: the compiler's own choice (128
// registers with four chunks in flight, so four CTAs of 4 warps on an SM) was
// the fastest on the 3B decode step. Capped to 96 registers (five CTAs) the
// 1,024 CTAs of the gate/up product run as 740 and a thin 284, which was slower.
template <int NT, int WARPS, int UNROLL, bool ROPE>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* x, long long ldx,
                   const __nv_bfloat16* __restrict__ w, long long ldw, void* __restrict__ out,
                   long long ldo, int out_f32, int T, int N, int K, int epilogue,
                   const void* next, long long next_bytes, long long plane_stride,
                   const typename RopeArg<ROPE>::type rw) {
  __shared__ float red[WARPS][16][8 * NT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);  // rows past N are discarded
  // rotary epilogue: this CTA's head, and its rows' first elements inside the head
  int head = 0, e_lo = 0, e_hi = 0;
  bool rotated = false;
  if constexpr (ROPE) {
    const int per_head = rw.D >> 4, half = rw.rotary_dim >> 1;
    head = blockIdx.x / per_head;
    const int c = blockIdx.x - head * per_head;
    if (head >= rw.A && !rw.write_cache) return;  // keys and values are not wanted
    rotated = c < (half >> 3) && head < rw.A + rw.Kh;
    if (c < (half >> 3)) { e_lo = 8 * c; e_hi = e_lo + half; }
    else { e_lo = rw.rotary_dim + 16 * (c - (half >> 3)); e_hi = e_lo + 8; }
    r0 = head * rw.D + e_lo + g;
    r1 = head * rw.D + e_hi + g;
  }
  // gridDim.y CTAs share a row group's K; each writes its own float32 plane
  const int chunks = (K + CHUNK - 1) / CHUNK;
  const int share = (chunks + (int)gridDim.y - 1) / (int)gridDim.y;
  const int s0 = blockIdx.y * share, s1 = min(chunks, s0 + share);
  const int per = (max(s1 - s0, 0) + WARPS - 1) / WARPS;
  const int c0 = s0 + warp * per, c1 = min(s1, c0 + per);

  // A thread's 16 elements of a 64-element chunk are [8t, 8t+8) and [32+8t, 32+8t+8):
  // the four threads of a row group read 64 contiguous bytes per load instruction.
  const __nv_bfloat16* w0 = w + (size_t)r0 * ldw + t * 8;
  const __nv_bfloat16* w1 = w + (size_t)r1 * ldw + t * 8;
  const __nv_bfloat16* xr[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int tok = j * 8 + g;
    xok[j] = tok < T;
    xr[j] = x + (size_t)(xok[j] ? tok : 0) * ldx + t * 8;  // a padding row reads row 0, unused
  }
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  // The thread's 16 elements feed four instructions; instruction s takes
  // elements 4s..4s+3 as its k slots (2t, 2t+1, 2t+8, 2t+9).
  auto multiply = [&](const uint4 (&a)[4], const uint4 (&b)[NT][2]) {
    const uint32_t* a0 = reinterpret_cast<const uint32_t*>(&a[0]);  // row r0: 8 words
    const uint32_t* a1 = reinterpret_cast<const uint32_t*>(&a[2]);  // row r1: 8 words
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint32_t* bx = reinterpret_cast<const uint32_t*>(&b[j][0]);
        const uint32_t b0 = xok[j] ? bx[2 * s] : 0u, b1 = xok[j] ? bx[2 * s + 1] : 0u;
        mma_bf16(acc[j], a0[2 * s], a1[2 * s], a0[2 * s + 1], a1[2 * s + 1], b0, b1);
      }
    }
  };

  // whole chunks, UNROLL at a time: every load is issued before the first use
  // The weights are constants: their first loads go out before this kernel
  // waits for the one that produces x.
  const int full_end = min(c1, K / CHUNK);  // chunks that lie entirely inside K
  int c = c0;
  bool waited = false;
  for (; c + UNROLL <= full_end; c += UNROLL) {
    uint4 a[UNROLL][4];
    uint4 b[UNROLL][NT][2];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const size_t off = (size_t)(c + u) * CHUNK;
      a[u][0] = ld_stream(w0 + off);
      a[u][1] = ld_stream(w0 + off + 32);
      a[u][2] = ld_stream(w1 + off);
      a[u][3] = ld_stream(w1 + off + 32);
    }
    if (!waited) {
      fb_pdl_wait();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const size_t off = (size_t)(c + u) * CHUNK;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        b[u][j][0] = ld_cached(xr[j] + off);
        b[u][j][1] = ld_cached(xr[j] + off + 32);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) multiply(a[u], b[u]);
  }
  if (!waited) fb_pdl_wait();
  // the rest: single chunks, the last of which may reach beyond K
  for (; c < c1; ++c) {
    const size_t off = (size_t)c * CHUNK;
    const int k = c * CHUNK + t * 8;
    const bool lo = k + 8 <= K, hi = k + 32 + 8 <= K;
    uint4 a[4];
    uint4 b[NT][2];
    a[0] = lo ? ld_stream(w0 + off) : zero;
    a[1] = hi ? ld_stream(w0 + off + 32) : zero;
    a[2] = lo ? ld_stream(w1 + off) : zero;
    a[3] = hi ? ld_stream(w1 + off + 32) : zero;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      b[j][0] = lo ? ld_cached(xr[j] + off) : zero;
      b[j][1] = hi ? ld_cached(xr[j] + off + 32) : zero;
    }
    multiply(a, b);
  }
  // this block's weights are in; the kernel after this one can have its own on the way
  fb_prefetch_l2_slice(next, next_bytes);
  // acc[j][0..1]: row g, tokens j*8 + 2t, 2t+1; acc[j][2..3]: row g + 8
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][g][j * 8 + 2 * t] = acc[j][0];
    red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  float* out_f = reinterpret_cast<float*>(out) + (size_t)blockIdx.y * plane_stride;
  __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(out);
  if constexpr (ROPE) {
    // rows p and p + 8 are elements e_lo + p and e_hi + p of the head
    for (int idx = threadIdx.x; idx < 8 * T; idx += WARPS * 32) {
      const int p = idx & 7, tok = idx >> 3;
      const int seq = rw.seq_of_token[tok];
      if (seq < 0) continue;  // padding token
      float x1 = 0.f, x2 = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) {
        x1 += red[wi][p][tok];
        x2 += red[wi][p + 8][tok];
      }
      const int pos = rw.positions[tok];
      if (rotated) {
        float sn, cs;
        sincosf((float)pos * rw.inv_freq[e_lo + p], &sn, &cs);
        const float y1 = x1 * cs - x2 * sn;
        x2 = x2 * cs + x1 * sn;
        x1 = y1;
      }
      __nv_bfloat16* dst;
      if (head < rw.A) {
        dst = rw.q_out + (size_t)tok * rw.q_stride + (size_t)head * rw.D;
      } else {
        int lp = pos / FB_PAGE;
        if (rw.ring_pages > 0) lp %= rw.ring_pages;
        const long long page = rw.page_table[(size_t)seq * rw.max_pages + lp];
        const bool key = head < rw.A + rw.Kh;
        dst = (key ? rw.k_cache : rw.v_cache) + page * rw.page_stride +
              (long long)(head - rw.A - (key ? 0 : rw.Kh)) * rw.head_stride +
              (long long)(pos % FB_PAGE) * rw.D;
      }
      dst[e_lo + p] = __float2bfloat16_rn(x1);
      dst[e_hi + p] = __float2bfloat16_rn(x2);
    }
  } else {
    if (epilogue == 0) {
      for (int idx = threadIdx.x; idx < 16 * T; idx += WARPS * 32) {
        const int row = idx & 15, tok = idx >> 4;
        if (n0 + row >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v += red[wi][row][tok];
        const size_t o = (size_t)tok * ldo + n0 + row;
        if (out_f32) out_f[o] = v;
        else out_h[o] = __float2bfloat16_rn(v);
      }
    } else {
      // rows 2p and 2p+1 hold gate p and up p: out[t, n0/2 + p] = silu(gate) * up
      for (int idx = threadIdx.x; idx < 8 * T; idx += WARPS * 32) {
        const int p = idx & 7, tok = idx >> 3;
        if (n0 + 2 * p + 1 >= N) continue;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) {
          gate += red[wi][2 * p][tok];
          up += red[wi][2 * p + 1][tok];
        }
        out_h[(size_t)tok * ldo + (n0 >> 1) + p] =
            __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
      }
    }
  }
}

int launch_skinny(const void* x, long long ldx, const void* w, long long ldw, void* out,
                  long long ldo, int out_f32, int T, int N, int K, int epilogue, const void* next,
                  long long next_bytes, int ksplit, long long plane_stride, int warps,
                  const RopeWrite& rw, cudaStream_t stream) {
  FB_REQUIRE(next_bytes >= 0 && next_bytes % 16 == 0 && ((uintptr_t)next % 16) == 0,
             "gemm_skinny: the prefetch range must be 16-byte aligned and a multiple of 16 bytes");
  FB_REQUIRE(T > 0 && T <= 16 && N > 0 && K > 0, "gemm_skinny: bad sizes T=%d N=%d K=%d", T, N, K);
  FB_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)x % 16) == 0 &&
                 ((uintptr_t)w % 16) == 0,
             "gemm_skinny: K, the row strides and the pointers must keep 16-byte alignment");
  FB_REQUIRE(epilogue != 1 || (!out_f32 && N % 2 == 0),
             "gemm_skinny: the SiLU-mul epilogue needs a bf16 output and an even row count");
  FB_REQUIRE(ksplit >= 1 && ksplit <= 64 && (ksplit == 1 || (out_f32 && epilogue == 0 &&
                                                             plane_stride >= (long long)T * ldo)),
             "gemm_skinny: %d K shares need float32 planes and the plain epilogue", ksplit);
  FB_REQUIRE(warps == 0 || warps == 4 || warps == 8 || warps == 16,
             "gemm_skinny: %d warps per CTA (4, 8 or 16)", warps);
  const int blocks = (N + 15) / 16;
  // Warps per CTA: as many as still let every CTA of the grid be resident at
  // once (one CTA of 16 warps, two of 8 or five of 4 fit an SM). A second, thin
  // round of CTAs costs a whole round's latency: measured on the 3B decode step,
  // 192 CTAs of 16 warps (148 + 44) were 4 us a call slower than 192 of 8.
  const int chunks = ((K + CHUNK - 1) / CHUNK + ksplit - 1) / ksplit;
  if (warps == 0) {
    const long long ctas = (long long)blocks * ksplit;
    warps = ctas <= 148 ? 16 : ctas <= 296 ? 8 : 4;
    while (warps > 4 && chunks / warps < 2) warps /= 2;
  }
  const int per = (chunks + warps - 1) / warps;
  const int unroll = per >= 4 ? 4 : per >= 3 ? 3 : 2;
#define FB_SKINNY_R(NT, W, U, R, EXTRA)                                                       \
  fb_launch(gemm_skinny_kernel<NT, W, U, R>, dim3(blocks, ksplit), dim3(W * 32), 0, stream,    \
            (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, ldw, out, ldo, out_f32, T, N, \
            K, epilogue, next, next_bytes, plane_stride, EXTRA)
#define FB_SKINNY(NT, W, U)                                   \
  do {                                                        \
    if (epilogue == 2) FB_SKINNY_R(NT, W, U, true, rw);       \
    else FB_SKINNY_R(NT, W, U, false, NoRope{});              \
  } while (0)
#define FB_SKINNY_U(NT, W)                                    \
  do {                                                        \
    if (unroll == 4) FB_SKINNY(NT, W, 4);                     \
    else if (unroll == 3) FB_SKINNY(NT, W, 3);                \
    else FB_SKINNY(NT, W, 2);                                 \
  } while (0)
#define FB_SKINNY_W(NT)                                       \
  do {                                                        \
    if (warps == 4) FB_SKINNY_U(NT, 4);                       \
    else if (warps == 8) FB_SKINNY_U(NT, 8);                  \
    else FB_SKINNY_U(NT, 16);                                 \
  } while (0)
  if (T <= 8) FB_SKINNY_W(1); else FB_SKINNY_W(2);
#undef FB_SKINNY_W
#undef FB_SKINNY_U
#undef FB_SKINNY
#undef FB_SKINNY_R
  return fb_check_launch("gemm_skinny");
}

}  // namespace

// x: [T, K] bf16 (row stride ldx), w: [N, K] bf16 (row stride ldw), T <= 16.
// epilogue 0: out[T, N] (bf16 or float32, row stride ldo).
// epilogue 1: w's rows are (gate, up) pairs; out[T, N / 2] bf16 = SiLU(gate) * up.
// next / next_bytes: optional constant data (the next kernel's weights) to be
// brought into L2 as this kernel's blocks finish their own loads; 0 bytes = none.
// ksplit > 1: K is shared by ksplit CTAs per row group and out is ksplit float32
// planes [T, N], plane_stride elements apart, for a consumer that sums them
// (epilogue 0 only). warps: 4, 8 or 16 per CTA, or 0 to have it chosen here.
FB_API int fb_gemm_skinny(const void* x, long long ldx, const void* w, long long ldw, void* out,
                          long long ldo, int out_f32, int T, int N, int K, int epilogue,
                          const void* next, long long next_bytes, int ksplit,
                          long long plane_stride, int warps, cudaStream_t stream) {
  FB_REQUIRE(epilogue == 0 || epilogue == 1, "gemm_skinny: epilogue %d", epilogue);
  return launch_skinny(x, ldx, w, ldw, out, ldo, out_f32, T, N, K, epilogue, next, next_bytes,
                       ksplit, plane_stride, warps, RopeWrite{}, stream);
}

// The fused q/k/v projection of up to 16 tokens with the rotary epilogue:
// w is [(A + 2 Kh) * D, K] (query, key, value heads); rotated queries go to
// q_out [T, A * D], rotated keys and the values into the cache pages of each
// token's position (page_table[seq, position / FB_PAGE], modulo ring_pages when
// that is > 0). Tokens with seq_of_token < 0 are padding and write nothing;
// with write_cache == 0 only the queries are computed.
FB_API int fb_gemm_skinny_rope(const void* x, long long ldx, const void* w, long long ldw, int T,
                               int K, const int* positions, const int* seq_of_token,
                               const int* page_table, int max_pages, const float* inv_freq,
                               int rotary_dim, void* q_out, long long q_stride, void* k_cache,
                               void* v_cache, long long page_stride, long long head_stride,
                               int ring_pages, int A, int Kh, int D, int write_cache,
                               const void* next, long long next_bytes, int warps,
                               cudaStream_t stream) {
  FB_REQUIRE(A > 0 && Kh > 0 && D > 0 && D % 16 == 0,
             "gemm_skinny_rope: head size %d is not a multiple of 16", D);
  FB_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 16 == 0,
             "gemm_skinny_rope: rotary width %d must be a multiple of 16 up to the head size %d",
             rotary_dim, D);
  FB_REQUIRE(q_stride >= (long long)A * D && max_pages > 0 && ring_pages >= 0,
             "gemm_skinny_rope: bad strides or page counts");
  RopeWrite rw{};
  rw.positions = positions; rw.seq_of_token = seq_of_token; rw.page_table = page_table;
  rw.max_pages = max_pages; rw.inv_freq = inv_freq; rw.rotary_dim = rotary_dim;
  rw.q_out = (__nv_bfloat16*)q_out; rw.q_stride = q_stride;
  rw.k_cache = (__nv_bfloat16*)k_cache; rw.v_cache = (__nv_bfloat16*)v_cache;
  rw.page_stride = page_stride; rw.head_stride = head_stride; rw.ring_pages = ring_pages;
  rw.A = A; rw.Kh = Kh; rw.D = D; rw.write_cache = write_cache;
  return launch_skinny(x, ldx, w, ldw, q_out, q_stride, 0, T, (A + 2 * Kh) * D, K, 2, next,
                       next_bytes, 1, 0, warps, rw, stream);
}
