// Inline-PTX faces of the Blackwell tensor-core path shared by the kernels that
// use it: mbarriers with bounded waits, TMA tile loads, tcgen05 MMA issue and
// commit, tensor-memory loads and stores, shared-memory matrix descriptors.
//
// Every wait is bounded: when the bound is hit the caller's `abort_flag` (in
// shared memory) is raised so that the CTA's other roles give up too, and the
// place is recorded twice: in a status word on the device (`fb_gemm_tc_status`
// and its siblings read and clear it) and in a record in pinned host memory
// that the host reads without a copy (`fb_status_mirror`), so that the engine
// can check it wherever it has just synchronised.
//
// A file that includes this header first defines FB_STATUS_KERNEL, the code
// under which its kernels report (1 the one-CTA products, 2 the paired
// product, 3 the prompt attention).
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

#ifndef FB_STATUS_KERNEL
#error "define FB_STATUS_KERNEL before including tcgen05.cuh"
#endif

int* fb_status_mirror_host();  // common.cu: the pinned record, or null

namespace {

constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ int g_status[4];  // [0] != 0: a wait ran out; [1] where; [2] block; [3] k-block
__device__ int* g_status_mirror;  // the host-visible record {kernel, where, block, k-block}

// The first failure of this file's kernels since the status was last cleared.
__device__ __forceinline__ void record_failure(int where, int block, int kb) {
  if (atomicCAS(&g_status[0], 0, 1) != 0) return;
  g_status[1] = where;
  g_status[2] = block;
  g_status[3] = kb;
  volatile int* mirror = g_status_mirror;
  if (mirror != nullptr && mirror[0] == 0) {
    mirror[1] = where;
    mirror[2] = block;
    mirror[3] = kb;
    __threadfence_system();
    mirror[0] = FB_STATUS_KERNEL;  // last, so that a host that sees it sees the rest
    __threadfence_system();
  }
}

// Points this file's kernels at the host-visible record, once per device.
// Launchers call it before their launch; a capturing stream puts it off (the
// copy to the symbol is no stream work), and a device beyond the table goes
// without the mirror: the status on the device is recorded either way.
inline void bind_status_mirror(cudaStream_t stream) {
  static std::mutex mu;
  static bool bound[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return;
  std::lock_guard<std::mutex> lock(mu);
  if (bound[device]) return;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess ||
      capturing != cudaStreamCaptureStatusNone)
    return;
  int* host = fb_status_mirror_host();
  int* mapped = nullptr;
  if (host != nullptr && cudaHostGetDevicePointer((void**)&mapped, host, 0) == cudaSuccess)
    cudaMemcpyToSymbol(g_status_mirror, &mapped, sizeof(mapped));
  bound[device] = true;
}

// ------------------------------------------------------------------ PTX faces
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait. Returns false when the bound was hit or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int where, int kb) {
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  record_failure(where, (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)), kb);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Makes shared-memory writes of this thread visible to the async proxy (TMA, MMA).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// swizzled in 128-byte mode: 8-row groups are 1024 bytes apart (stride byte
// offset); the leading byte offset is unused because one MMA's K extent
// (32 bytes) lies inside one swizzle row. Bits 46-47 carry the descriptor
// version of this architecture (1); bits 61-63 the swizzle mode (2 = 128 B).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// The same for an operand whose MN dimension is contiguous (a [K rows, MN
// columns] tile, rows of 128 bytes = 64 elements, 128-byte swizzle): 8-row
// groups along K are 1024 bytes apart (stride byte offset), and the next 64
// elements along MN start `mn_block_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16: D = float32 (bits 4-5 = 1), A and B =
// bfloat16 (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0),
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
// The same with B given MN-major (bit 16).
__host__ __device__ constexpr uint32_t make_idesc_b_mn(int m, int n) {
  return make_idesc(m, n) | (1u << 16);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                     uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same product with the A operand in tensor memory: lane = row of A, each
// 32-bit column two consecutive K elements (the lower half first); 16 K elements
// per instruction are 8 columns from `tmem_a` on.
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


}  // namespace
