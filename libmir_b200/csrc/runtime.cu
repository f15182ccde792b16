// Error text of the last failed call, and the check after each launch.
#include <cstdarg>
#include <cstdio>
#include "common.cuh"

static thread_local char g_error[512] = "";

void mir_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

int mir_check_launch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) return MIR_OK;
  mir_set_error("%s: %s", what, cudaGetErrorString(err));
  return MIR_CUDA_ERROR;
}

MIR_EXPORT const char* mir_last_error() { return g_error; }

MIR_EXPORT int mir_abi_version() { return 1; }
