// Shared declarations of the kernel library: element types, the error channel
// and small device helpers. Every launcher is `extern "C"`, takes raw device
// pointers and a stream, validates its arguments on the host, returns 0 on
// success and a non-zero code with a message in `fb_last_error()` otherwise.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <utility>

#define FB_API extern "C" __attribute__((visibility("default")))

// Element types as the Python side names them.
enum FbDType : int { FB_F32 = 0, FB_BF16 = 1 };

// Tokens per cache page: the unit in which sequences take and give back cache
// memory. Kernels index a key at position p as page_table[p / 64], row p % 64.
constexpr int FB_PAGE = 64;

int fb_fail(int code, const char* fmt, ...);  // records the message, returns code
int fb_check_launch(const char* what);        // cudaGetLastError -> code

// True the first time it is called with this table on the current device: for
// per-kernel set-up (shared-memory opt-in, occupancy queries) that CUDA keeps
// per device. `seen` is a static table of the call site. Devices beyond the
// table are set up on every call, which is slower and still right.
inline bool fb_first_use_on_device(bool (&seen)[64]) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return true;
  if (seen[device]) return false;
  seen[device] = true;
  return true;
}

#define FB_REQUIRE(cond, ...)                      \
  do {                                             \
    if (!(cond)) return fb_fail(1, __VA_ARGS__);   \
  } while (0)

// ------------------------------------------------------------------ launching
// Every kernel of the library is launched through `fb_launch`, which marks the
// launch for programmatic dependent launch: the kernel's blocks may be placed on
// the SMs as the blocks of the kernel before it in the stream retire, without
// waiting for that kernel's memory to be flushed first. In return every kernel
// calls `fb_pdl_wait()` before it reads anything an earlier kernel wrote and
// before it writes anything an earlier kernel may still read (only constants
// such as weights may be touched before; the products request their first
// weight tiles there). When a kernel lets its successor's blocks be placed
// (griddepcontrol.launch_dependents) decides whether that helps: the short
// kernels of few blocks (norm, rotary) do it at once; the single-token
// products when a block's main loop is through (the CTAs of the grid's last
// half round as they start, when no CTA of the kernel waits for room any
// more); the single-token attention and the tcgen05 products not at all, and
// no long kernel at its start (the successor's blocks would sit on the SMs
// holding registers and shared memory that this kernel's next blocks need).
// Every kernel reads what an earlier kernel wrote with ordinary (coherent)
// loads only: pointers to such data carry no `__restrict__` read-only promise
// and no `ld.global.nc`, because after an early trigger the writer may still
// have been running when the reader's blocks were placed, and a non-coherent
// load was seen to return the address's previous contents then. Only weights
// and the step's description, which no kernel writes, keep the promise.
// `fb_set_pdl(0)` switches the mark off: launches then serialise as usual and
// the device calls do nothing.
extern int g_fb_pdl;

template <typename... KArgs, typename... Args>
inline cudaError_t fb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_fb_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The same launch with the grid's z extent grouped into thread-block clusters of
// `cluster_z` CTAs (distributed shared memory between the CTAs of a cluster).
template <typename... KArgs, typename... Args>
inline cudaError_t fb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, unsigned cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = cluster_z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_fb_pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void fb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel's blocks be placed as soon as every block of this kernel
// has said so or ended (see the notes on launching above for where to call it).
__device__ __forceinline__ void fb_pdl_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Asks the memory system to bring [p, p + bytes) into L2; nothing waits for it.
// The blocks of a grid share the range in pieces, each block's first warp asks
// for its pieces. A kernel calls this once its own loads are issued, with the
// constant data (weights) that the NEXT kernel streams first: DRAM then keeps
// working through this kernel's tail and the next one's start.
// p must be 16-byte aligned and bytes a multiple of 16.
__device__ __forceinline__ void fb_prefetch_l2_slice(const void* p, long long bytes) {
  constexpr long long PIECE = 8192;
  if (bytes <= 0 || threadIdx.x >= 32) return;
  const long long nblk = (long long)gridDim.x * gridDim.y * gridDim.z;
  const long long bid = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
  const long long pieces = (bytes + PIECE - 1) / PIECE;
  for (long long i = bid + nblk * threadIdx.x; i < pieces; i += nblk * 32) {
    const long long left = bytes - i * PIECE;
    const unsigned size = (unsigned)(left < PIECE ? left : PIECE);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;"
                 :: "l"(reinterpret_cast<const char*>(p) + i * PIECE), "r"(size) : "memory");
  }
}
#endif

// ---------------------------------------------------------------- device side
template <typename T>
__device__ __forceinline__ float fb_to_float(T v);
template <>
__device__ __forceinline__ float fb_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float fb_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// A load that is never served by the non-coherent path: for data that the
// kernel before this one wrote (see the launching notes above).
template <typename T>
__device__ __forceinline__ float fb_load_coherent(const T* p);
template <>
__device__ __forceinline__ float fb_load_coherent<float>(const float* p) { return __ldcg(p); }
template <>
__device__ __forceinline__ float fb_load_coherent<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(__ldcg(p));
}

template <typename T>
__device__ __forceinline__ T fb_from_float(float v);
template <>
__device__ __forceinline__ float fb_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 fb_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float fb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float fb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds 32 floats of shared memory. Every thread of
// the block must call it; the result is returned to all of them.
__device__ __forceinline__ float fb_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = fb_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = fb_warp_sum(t);
  return t;
}

// Dispatch a host-side dtype code to a template parameter.
#define FB_DISPATCH_DTYPE(code, T, ...)                                   \
  do {                                                                    \
    if ((code) == FB_F32) {                                               \
      using T = float;                                                    \
      __VA_ARGS__;                                                        \
    } else if ((code) == FB_BF16) {                                       \
      using T = __nv_bfloat16;                                            \
      __VA_ARGS__;                                                        \
    } else {                                                              \
      return fb_fail(1, "unknown element type code %d", (int)(code));    \
    }                                                                     \
  } while (0)
