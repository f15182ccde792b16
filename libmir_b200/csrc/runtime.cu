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

static bool g_pdl = false;   // measured: inside captured decode steps it costs more than it hides

bool mir_pdl_enabled() { return g_pdl; }

// 1: kernels are launched with programmatic stream serialization; 0 (the default): plainly.
MIR_EXPORT void mir_set_pdl(int enabled) { g_pdl = enabled != 0; }
MIR_EXPORT int mir_get_pdl() { return g_pdl ? 1 : 0; }
