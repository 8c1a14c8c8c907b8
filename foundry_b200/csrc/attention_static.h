// Declaration of the one entry point of this library that allocates nothing.
//
// It has no counterpart in the reference (stratorys/foundry), whose device
// code allocates a fresh buffer for every operation.
//
// Who needs it: callers that drive the kernels from a place where device
// memory cannot be requested: a host runtime that has handed all device memory
// to its own arena and forbids cudaMalloc afterwards, a plugin that runs inside
// another framework's stream callback or captured region, a real-time loop that
// must not take the allocator's lock. Such callers can pass inputs and outputs
// they already own, but split-KV decode attention also needs a place for the
// partial results of its splits. `fb_attention_decode_static` keeps that place
// inside the library: a fixed array in device memory that exists from the moment
// the library is loaded on a GPU until the process ends.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Floats of scratch the library holds on every GPU it is loaded on (8 MiB).
#define FB_ATTENTION_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Decode attention (one new token per sequence) over the paged bfloat16 cache,
// with the arguments and the result of `fb_attention_decode`, except that no
// workspace is passed (nor a page-buffer count or a cluster size: three buffers,
// no clusters): the partial results of the `splits` cache ranges go to the
// library's own scratch array, where the last CTA of a pair merges them.
//
//   needs  n_seqs * Kh * splits * (16 * D + 32) + n_seqs * Kh (rounded up to 64)
//          <= FB_ATTENTION_STATIC_SCRATCH_FLOATS, else it returns non-zero with a
//          message in fb_last_error() and launches nothing.
//   calls  no cudaMalloc, cudaFree or any allocating routine.
//   first call on a device: looks up the scratch array's device address (once
//          per device, with that device current). Make this first call before
//          any stream capture begins.
//   shared state: every call on a device uses the same array, which keeps what
//          the last call left. Only the arrival counters at its start must be
//          zero when a call begins: they are zero when the library is loaded and
//          the kernel clears each one it used before it ends; everything else a
//          call writes before it reads. Two calls that overlap on the GPU
//          (different streams, no ordering between them) race on the array;
//          order them, as calls on one stream are.
int fb_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                               const int* cu_tokens, const int* kv_lens, const int* page_table,
                               int max_pages, const void* k_cache, const void* v_cache,
                               long long page_stride, long long head_stride, int n_seqs, int A,
                               int Kh, int D, float scale, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
