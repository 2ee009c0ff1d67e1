// Host-side error plumbing shared by every library built from this folder.
// An entry point that refuses its arguments stores a message here and returns
// a negative code; the Python binding raises it.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[768] = "";

void tge_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

int tge_check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    tge_set_error("%s: launch failed: %s", what, cudaGetErrorString(err));
    return -2;
  }
  return 0;
}

bool tge_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* off = getenv("TGE_NO_PDL");
    enabled = (off != nullptr && off[0] != '\0') ? 0 : 1;
  }
  return enabled == 1;
}

int tge_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (count <= 0) count = 1;
  }
  return count;
}

TGE_API int tge_device_sm_count() { return tge_sm_count(); }

TGE_API const char* tge_last_error() { return g_error; }

TGE_API int tge_abi_version() { return 1; }
