// The error channel of the kernel library.
#include "common.cuh"

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

int g_fb_pdl = 1;

// 1 (default): kernels are launched for programmatic dependent launch; 0: plain launches.
FB_API void fb_set_pdl(int on) { g_fb_pdl = on ? 1 : 0; }

FB_API const char* fb_last_error() { return g_error; }

// Bumped whenever an exported signature changes; the Python side refuses a
// library of another version instead of calling it with the wrong arguments.
FB_API int fb_abi_version() { return 1; }
