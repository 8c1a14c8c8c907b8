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
// Two more pieces take the RMS norm between two projections out of the step
// as a kernel of its own (y = x / sqrt(mean(x^2) + eps) * g, src/nn/norm.rs:31-51).
// The projection BEFORE the norm adds its result to the float32 residual rows
// in its epilogue, writes resid * g in bfloat16 for the next projection, and
// leaves each CTA's share of the rows' sums of squares ("residual sink"). The
// projection AFTER the norm sums those shares (in a fixed order) and multiplies
// its accumulators by 1 / sqrt(mean + eps): the product is linear in the row
// scale, so scaling after the sum over K is the same normalisation, with the one
// rounding to bfloat16 made before the scale instead of after it.
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
  int interleaved;          // rotation pairs are elements (2i, 2i + 1) instead of (i, i + rotary_dim / 2)
};
struct NoRope {};

// Most shares of a row scale (rows of 64 bytes in the consumer's shared memory,
// within the 48 KB a kernel has without opting in for more, beside its own).
constexpr int FB_SKINNY_MAX_SHARES = 384;

// Row scale of the input: token t's accumulators are multiplied by
// 1 / sqrt(sum_c ss[c * stride + t] * inv_dim + eps). ss == nullptr: no scale.
struct RowScale {
  const float* ss;
  int count, stride;
  float inv_dim, eps;
};
// Residual sink (epilogue 3): resid[t, n] += out[t, n]; xg[t, n] = bf16(resid * gamma[n]);
// ss_out[blockIdx.x * ss_stride + t] = this CTA's sum over its rows of resid^2.
struct ResidualSink {
  float* resid;
  long long ldr;
  const float* gamma;
  __nv_bfloat16* xg;
  long long ldxg;
  float* ss_out;
  int ss_stride;
};
template <bool ROPE> struct RopeArg { using type = NoRope; };
template <> struct RopeArg<true> { using type = RopeWrite; };
struct NoSink {};
template <bool SINK> struct SinkArg { using type = NoSink; };
template <> struct SinkArg<true> { using type = ResidualSink; };
// what a kernel instance ends with
constexpr int MODE_PLAIN = 0;  // store, or SiLU(gate) * up
constexpr int MODE_ROPE = 1;   // rotate and write queries, keys, values
constexpr int MODE_SINK = 2;   // add into the residual rows in front of a norm

// NT: token tiles of 8 (1 or 2). WARPS: warps per CTA, each with a K range.
// UNROLL: chunks whose loads are in flight together.
// Registers are capped at 128 (four chunks of weights in flight; four CTAs of 4
// warps on an SM), the fastest on the 3B decode step: at 130 the gate/up product
// of 8 tokens ran three CTAs to an SM and took 3 us longer; capped to 96 (five
// CTAs) its 1,024 CTAs run as 740 and a thin 284, which was slower too. With 16
// tokens the cap holds only because x is fetched one chunk ahead instead of all
// chunks at once.
constexpr int min_blocks(int warps) { return 16 / warps; }
template <int NT, int WARPS, int UNROLL, int MODE>
__global__ void __launch_bounds__(WARPS * 32, min_blocks(WARPS))
gemm_skinny_kernel(const __nv_bfloat16* x, long long ldx,
                   const __nv_bfloat16* __restrict__ w, long long ldw, void* __restrict__ out,
                   long long ldo, int out_f32, int T, int N, int K, int epilogue,
                   const void* next, long long next_bytes, long long plane_stride,
                   int late_trigger, int early_from,
                   const typename RopeArg<MODE == MODE_ROPE>::type rw,
                   const RowScale scale,
                   const typename SinkArg<MODE == MODE_SINK>::type sink) {
  constexpr bool ROPE = MODE == MODE_ROPE, SINK = MODE == MODE_SINK;
  __shared__ float red[WARPS][16][8 * NT + 1];
  __shared__ float scale_part[4][16];
  extern __shared__ __align__(16) float shares[];  // [scale.count][16] when there is a row scale
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  // The CTAs that are placed last let the next kernel's blocks be placed as they
  // start: no CTA of this kernel waits for room any more, and what room there is
  // (a thin last round, SMs with one CTA of two) goes to blocks that ask for their
  // first weights while this kernel still streams. The other CTAs say so when their
  // main loop is through (below). Measured on the 3B decode step at batch 8 with
  // the last half round starting so, that was the fastest (a whole round and a quarter lost).
  if (late_trigger && (int)(blockIdx.x + blockIdx.y * gridDim.x) >= early_from) fb_pdl_launch();
  int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);  // rows past N are discarded
  // rotary epilogue: this CTA's head, and its rows' first elements inside the head
  // (accumulator rows p and p + 8 are elements e_lo + p * e_step and e_hi + p * e_step
  // of the head, a rotation pair with frequency f_lo + p where the CTA rotates)
  int head = 0, e_lo = 0, e_hi = 0, e_step = 1, f_lo = 0;
  bool rotated = false;
  if constexpr (ROPE) {
    const int per_head = rw.D >> 4, half = rw.rotary_dim >> 1;
    head = blockIdx.x / per_head;
    const int c = blockIdx.x - head * per_head;
    if (head >= rw.A && !rw.write_cache) return;  // keys and values are not wanted
    rotated = c < (half >> 3) && head < rw.A + rw.Kh;
    if (c < (half >> 3)) {
      f_lo = 8 * c;
      if (rw.interleaved) { e_lo = 16 * c; e_hi = e_lo + 1; e_step = 2; }
      else { e_lo = 8 * c; e_hi = e_lo + half; }
    } else {
      e_lo = rw.rotary_dim + 16 * (c - (half >> 3));
      e_hi = e_lo + 8;
    }
    r0 = head * rw.D + e_lo + g * e_step;
    r1 = head * rw.D + e_hi + g * e_step;
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
  // What the epilogue needs from the kernel before this one is asked for as soon
  // as that kernel is through, so that nothing is fetched at the end: the shares
  // of the row scale go to shared memory behind the weight stream (cp.async), a
  // thread's old residual values and norm weights into registers.
  constexpr int SINK_ITEMS = SINK ? (16 * 8 * NT + WARPS * 32 - 1) / (WARPS * 32) : 1;
  float old_resid[SINK_ITEMS], gamma[SINK_ITEMS];
  auto after_wait = [&]() {
    fb_pdl_wait();
    if (scale.ss != nullptr) {
      // Every CTA of the grid wants the same few lines: through L1 (.ca), so that
      // the CTAs of an SM ask L2 once, and only the T floats of a row that count.
      const int pieces = (T + 3) >> 2;  // 16-byte pieces of a 64-byte row
      for (int i = threadIdx.x; i < scale.count * pieces; i += WARPS * 32) {
        const int off = (i / pieces) * 16 + (i % pieces) * 4;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(shares + off);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(scale.ss + off)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if constexpr (SINK) {
#pragma unroll
      for (int it = 0; it < SINK_ITEMS; ++it) {
        const int idx = threadIdx.x + it * WARPS * 32;
        const int row = idx & 15, tok = idx >> 4;
        const bool live = tok < T && n0 + row < N;
        old_resid[it] = live ? *reinterpret_cast<const volatile float*>(
                                   sink.resid + (size_t)tok * sink.ldr + n0 + row) : 0.f;
        gamma[it] = live ? sink.gamma[n0 + row] : 0.f;
      }
    }
  };
  // The row scales, in a fixed order and in few instructions. Called once by every
  // thread, right after the first loads of x have gone out, so that waiting for
  // the shares costs nothing beyond waiting for x (at the end of the kernel, where
  // every CTA of an SM arrives together and nothing else hides it, the same work
  // cost the gate/up product of 8 tokens 1.5 us, and 5 us as a loop of whole warps
  // over the tokens). Of the first 128 threads, thread i sums every GROUPS-th share
  // of token i % TOKS; the groups of a warp meet by shuffles, the four warps' sums
  // in shared memory, where every thread of the epilogue adds its token's four and
  // takes the root.
  auto finish_scale = [&]() {
    if (scale.ss == nullptr) return;
    constexpr int TOKS = 8 * NT, GROUPS = 128 / TOKS;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 128) {
      const int tok = threadIdx.x & (TOKS - 1);
      float sum = 0.f;
      for (int c0 = threadIdx.x / TOKS; c0 < scale.count; c0 += GROUPS) sum += shares[c0 * 16 + tok];
#pragma unroll
      for (int o = TOKS; o < 32; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane < TOKS) scale_part[warp][lane] = sum;
    }
  };
  for (; c + UNROLL <= full_end; c += UNROLL) {
    uint4 a[UNROLL][4];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const size_t off = (size_t)(c + u) * CHUNK;
      a[u][0] = ld_stream(w0 + off);
      a[u][1] = ld_stream(w0 + off + 32);
      a[u][2] = ld_stream(w1 + off);
      a[u][3] = ld_stream(w1 + off + 32);
    }
    const bool first = !waited;
    if (first) {
      after_wait();
      waited = true;
    }
    auto load_x = [&](uint4 (&b)[NT][2], int u) {
      const size_t off = (size_t)(c + u) * CHUNK;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        b[j][0] = ld_cached(xr[j] + off);
        b[j][1] = ld_cached(xr[j] + off + 32);
      }
    };
    if constexpr (NT == 1) {
      uint4 b[UNROLL][NT][2];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) load_x(b[u], u);
      if (first) finish_scale();
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) multiply(a[u], b[u]);
    } else {
      // 16 tokens: x comes from L1 or L2, the weights from DRAM. One chunk's x at a
      // time, the next chunk's on its way, leaves the registers to the weights in
      // flight (with all chunks' x held at once the kernel wanted 134 registers
      // and ran three CTAs to an SM, or spilled under the cap).
      uint4 b[2][NT][2];
      load_x(b[0], 0);
      if (first) finish_scale();
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        if (u + 1 < UNROLL) load_x(b[(u + 1) & 1], u + 1);
        multiply(a[u], b[u & 1]);
      }
    }
  }
  if (!waited) {
    after_wait();
    finish_scale();
  }
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
  // ... and its blocks may be placed as this kernel's leave: the weights' last bytes
  // are on their way, what is left is the epilogue. (At the start of the kernel the
  // same instruction lost: the next kernel's blocks then take the room of this one's.
  // In front of an attention over a long context it lost too, so the caller decides.)
  if (late_trigger) fb_pdl_launch();
  // acc[j][0..1]: row g, tokens j*8 + 2t, 2t+1; acc[j][2..3]: row g + 8
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][g][j * 8 + 2 * t] = acc[j][0];
    red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
    red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
    red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  // token `tok`'s scale, by whoever needs it (no barrier more for a shared copy)
  auto row_scale = [&](int tok) {
    if (scale.ss == nullptr) return 1.f;
    const float sum = (scale_part[0][tok] + scale_part[1][tok]) +
                      (scale_part[2][tok] + scale_part[3][tok]);
    return 1.0f / sqrtf(sum * scale.inv_dim + scale.eps);
  };
  float* out_f = reinterpret_cast<float*>(out) + (size_t)blockIdx.y * plane_stride;
  __nv_bfloat16* out_h = reinterpret_cast<__nv_bfloat16*>(out);
  if constexpr (ROPE) {
    // rows p and p + 8 are elements e_lo + p * e_step and e_hi + p * e_step of the head
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
      const float rs = row_scale(tok);
      x1 *= rs;
      x2 *= rs;
      const int pos = rw.positions[tok];
      if (rotated) {
        float sn, cs;
        sincosf((float)pos * rw.inv_freq[f_lo + p], &sn, &cs);
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
      dst[e_lo + p * e_step] = __float2bfloat16_rn(x1);
      dst[e_hi + p * e_step] = __float2bfloat16_rn(x2);
    }
  } else if constexpr (SINK) {
    // 16 consecutive lanes hold a token's 16 rows of this CTA
#pragma unroll
    for (int it = 0; it < SINK_ITEMS; ++it) {
      const int idx = threadIdx.x + it * WARPS * 32;
      if (idx < 16 * 8 * NT) {  // whole warps are in or out
        const int row = idx & 15, tok = idx >> 4;
        const bool live = tok < T && n0 + row < N;
        float v = 0.f;
        if (live) {
#pragma unroll
          for (int wi = 0; wi < WARPS; ++wi) v += red[wi][row][tok];
          v = old_resid[it] + v * row_scale(tok);
          sink.resid[(size_t)tok * sink.ldr + n0 + row] = v;
          sink.xg[(size_t)tok * sink.ldxg + n0 + row] = __float2bfloat16_rn(v * gamma[it]);
        }
        float sq = v * v;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (row == 0 && tok < T) sink.ss_out[(size_t)blockIdx.x * sink.ss_stride + tok] = sq;
      }
    }
  } else {
    if (epilogue == 0) {
      for (int idx = threadIdx.x; idx < 16 * T; idx += WARPS * 32) {
        const int row = idx & 15, tok = idx >> 4;
        if (n0 + row >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v += red[wi][row][tok];
        v *= row_scale(tok);
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
        const float rs = row_scale(tok);
        gate *= rs;
        up *= rs;
        out_h[(size_t)tok * ldo + (n0 >> 1) + p] =
            __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
      }
    }
  }
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

int launch_skinny(const void* x, long long ldx, const void* w, long long ldw, void* out,
                  long long ldo, int out_f32, int T, int N, int K, int epilogue, const void* next,
                  long long next_bytes, int ksplit, long long plane_stride, int warps,
                  int late_trigger, const RopeWrite& rw, const RowScale& scale,
                  const ResidualSink& sink, cudaStream_t stream) {
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
  FB_REQUIRE(scale.ss == nullptr || (scale.count > 0 && scale.count <= FB_SKINNY_MAX_SHARES &&
                                     scale.stride == 16 && ((uintptr_t)scale.ss % 16) == 0 &&
                                     scale.inv_dim > 0.f && scale.eps > 0.f),
             "gemm_skinny: the row scale needs 1..%d shares in 16-byte aligned rows of 16 floats "
             "and a positive eps", FB_SKINNY_MAX_SHARES);
  const size_t shares_bytes = scale.ss != nullptr ? (size_t)scale.count * 64 : 0;
  FB_REQUIRE(epilogue != 3 || (sink.resid && sink.gamma && sink.xg && sink.ss_out &&
                               sink.ldr >= N && sink.ldxg >= N && sink.ss_stride >= T),
             "gemm_skinny: the residual sink needs its four arrays, rows of %d and shares of %d",
             N, T);
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
  // CTAs from this one on are the last half round of the grid (16 / warps CTAs fit an SM)
  const int early_from = blocks * ksplit - (16 / warps) * (sm_count() / 2);
#define FB_SKINNY_R(NT, W, U, MODE, ROPE_ARG, SINK_ARG)                                        \
  do {                                                                                         \
  fb_launch(gemm_skinny_kernel<NT, W, U, MODE>, dim3(blocks, ksplit), dim3(W * 32),            \
            shares_bytes, stream, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, ldw,   \
            out, ldo, out_f32, T, N, K, epilogue, next, next_bytes, plane_stride,               \
            late_trigger, early_from, ROPE_ARG, scale, SINK_ARG); } while (0)
#define FB_SKINNY(NT, W, U)                                                      \
  do {                                                                           \
    if (epilogue == 2) FB_SKINNY_R(NT, W, U, MODE_ROPE, rw, NoSink{});            \
    else if (epilogue == 3) FB_SKINNY_R(NT, W, U, MODE_SINK, NoRope{}, sink);     \
    else FB_SKINNY_R(NT, W, U, MODE_PLAIN, NoRope{}, NoSink{});                   \
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
// scale_ss (or null): x is resid * g of a norm whose 1 / sqrt(mean + eps) is
// still missing; token t's results are multiplied by
// 1 / sqrt(sum_c scale_ss[c * scale_stride + t] / scale_dim + scale_eps), c < scale_count.
FB_API int fb_gemm_skinny(const void* x, long long ldx, const void* w, long long ldw, void* out,
                          long long ldo, int out_f32, int T, int N, int K, int epilogue,
                          const void* next, long long next_bytes, int ksplit,
                          long long plane_stride, int warps, const float* scale_ss,
                          int scale_count, int scale_stride, int scale_dim, float scale_eps,
                          cudaStream_t stream) {
  FB_REQUIRE(epilogue == 0 || epilogue == 1, "gemm_skinny: epilogue %d", epilogue);
  const RowScale scale{scale_ss, scale_count, scale_stride,
                       scale_dim > 0 ? 1.0f / (float)scale_dim : 0.f, scale_eps};
  return launch_skinny(x, ldx, w, ldw, out, ldo, out_f32, T, N, K, epilogue, next, next_bytes,
                       ksplit, plane_stride, warps, 1, RopeWrite{}, scale, ResidualSink{}, stream);
}

// The projection in front of a norm (see the top of the file): resid [T, N]
// float32 (row stride ldr) += x w^T; xg [T, N] bf16 (row stride ldxg) =
// resid * gamma; ss_out[c * ss_stride + t] = CTA c's share of token t's sum of
// squares of the new resid, c < ceil(N / 16); ss_stride must be 16 for the
// products behind the norm.
FB_API int fb_gemm_skinny_residual(const void* x, long long ldx, const void* w, long long ldw,
                                   int T, int N, int K, float* resid, long long ldr,
                                   const float* gamma, void* xg, long long ldxg, float* ss_out,
                                   int ss_stride, const void* next, long long next_bytes,
                                   int warps, cudaStream_t stream) {
  ResidualSink sink{resid, ldr, gamma, (__nv_bfloat16*)xg, ldxg, ss_out, ss_stride};
  return launch_skinny(x, ldx, w, ldw, resid, ldr, 1, T, N, K, 3, next, next_bytes, 1, 0, warps,
                       1, RopeWrite{}, RowScale{}, sink, stream);
}

// Most shares of a row scale that the products behind a norm take
// (fb_gemm_skinny_residual leaves one per 16 features).
FB_API int fb_gemm_skinny_max_shares() { return FB_SKINNY_MAX_SHARES; }

// The fused q/k/v projection of up to 16 tokens with the rotary epilogue:
// w is [(A + 2 Kh) * D, K] (query, key, value heads); rotated queries go to
// q_out [T, A * D], rotated keys and the values into the cache pages of each
// token's position (page_table[seq, position / FB_PAGE], modulo ring_pages when
// that is > 0). Tokens with seq_of_token < 0 are padding and write nothing;
// with write_cache == 0 only the queries are computed. interleaved: the rotation
// pairs elements (2i, 2i + 1) of the rotary part instead of (i, i + rotary_dim / 2).
// late_trigger: whether the
// kernel behind this one (the attention) may have its blocks placed as this
// one's main loops end. scale_*: as in fb_gemm_skinny.
FB_API int fb_gemm_skinny_rope(const void* x, long long ldx, const void* w, long long ldw, int T,
                               int K, const int* positions, const int* seq_of_token,
                               const int* page_table, int max_pages, const float* inv_freq,
                               int rotary_dim, void* q_out, long long q_stride, void* k_cache,
                               void* v_cache, long long page_stride, long long head_stride,
                               int ring_pages, int A, int Kh, int D, int write_cache,
                               int interleaved, const void* next, long long next_bytes, int warps,
                               int late_trigger, const float* scale_ss, int scale_count,
                               int scale_stride, int scale_dim, float scale_eps,
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
  rw.interleaved = interleaved ? 1 : 0;
  const RowScale scale{scale_ss, scale_count, scale_stride,
                       scale_dim > 0 ? 1.0f / (float)scale_dim : 0.f, scale_eps};
  return launch_skinny(x, ldx, w, ldw, q_out, q_stride, 0, T, (A + 2 * Kh) * D, K, 2, next,
                       next_bytes, 1, 0, warps, late_trigger, rw, scale, ResidualSink{}, stream);
}
