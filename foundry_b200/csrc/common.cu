// The error channel of the kernel library.
#include "common.cuh"

#include <mutex>

static thread_local char g_error[1024] = "";

int fb_fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int fb_check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return fb_fail(2, "%s: %s", what, cudaGetErrorString(err));
  return 0;
}

// The host-visible record of a bounded wait that ran out (see tcgen05.cuh):
// four ints in pinned, mapped memory that every device of the process can
// write, {kernel code, where, block, k-block}; all zero while nothing failed.
// Allocated at the first request; null when the allocation fails (the status
// words on the device are kept either way).
int* fb_status_mirror_host() {
  static std::mutex mu;
  static int* record = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lock(mu);
  if (!tried) {
    tried = true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, 4 * sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) ==
        cudaSuccess) {
      record = static_cast<int*>(p);
      for (int i = 0; i < 4; ++i) record[i] = 0;
    } else {
      cudaGetLastError();  // the failure is reported by the null, not by the next launch
    }
  }
  return record;
}

// The record's host address for the caller to read (and to zero after a
// failure has been reported); null if it could not be made.
FB_API int* fb_status_mirror() { return fb_status_mirror_host(); }

int g_fb_pdl = 1;

// 1 (default): kernels are launched for programmatic dependent launch; 0: plain launches.
FB_API void fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; }

FB_API const char* fb_last_error() { return g_error; }

// Bumped whenever an exported signature changes; the Python side refuses a
// library of another version instead of calling it with the wrong arguments.
FB_API int fb_abi_version() { return 2; }
