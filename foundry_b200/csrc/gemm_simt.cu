// out[M,N] = x[M,K] * w[N,K]^T on the CUDA cores, accumulating in IEEE 32-bit
// (FFMA; no tensor cores, no TF32). This is the matrix product of the 32-bit
// path of the whole model, and the plain check of the tensor-core products.
//
// A projection is `x * W^T` with W stored [out, in] row-major and no bias
// (src/nn/linear.rs:19-36); accumulation is 32-bit in the reference too
// (src/metal/kernels/matmul.metal:42-64). Every output element sums its K
// products in the same order whatever M is, so a row's result does not depend
// on what else is in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* x /* written by the kernel before: no read-only promise */,
                 const TI* __restrict__ w, TO* __restrict__ out, int M,
                 int N, int K, long long ldx, long long ldw, long long ldo) {
  fb_pdl_wait();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int lr = tid / 4;        // 0..63: tile row loaded by this thread
  const int lc = (tid % 4) * 4;  // 0,4,8,12: first of its four k columns
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lc + j;
      const int m = m0 + lr, n = n0 + lr;
      xs[lc + j][lr] = (m < M && k < K) ? fb_load_coherent<TI>(x + (size_t)m * ldx + k) : 0.f;
      ws[lc + j][lr] = (n < N && k < K) ? fb_to_float<TI>(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) out[(size_t)m * ldo + n] = fb_from_float<TO>(acc[i][j]);
    }
  }
}
}  // namespace

FB_API int fb_gemm_simt(const void* x, const void* w, void* out, int M, int N, int K,
                        long long ldx, long long ldw, long long ldo, int in_dtype, int out_dtype,
                        cudaStream_t stream) {
  FB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  FB_REQUIRE(ldx >= K && ldw >= K && ldo >= N, "gemm_simt: a leading dimension is too small");
  if (M == 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  FB_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d exceeds the grid limit", M);
  FB_DISPATCH_DTYPE(in_dtype, TI, FB_DISPATCH_DTYPE(out_dtype, TO, (
      fb_launch(gemm_simt_kernel<TI, TO>, dim3(grid), dim3(256), 0, stream, 
          (const TI*)x, (const TI*)w, (TO*)out, M, N, K, ldx, ldw, ldo))));
  return fb_check_launch("gemm_simt");
}
