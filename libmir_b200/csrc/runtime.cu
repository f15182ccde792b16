// Error text of the last failed call, and the check after each launch.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "common.cuh"

static thread_local char g_error[512] = "";

void mir_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

// How often each kernel was launched, by the name its launcher gives (launches recorded while a CUDA graph is
// captured count once, replays of the graph do not count).  Names are string literals: found by address first.
namespace {
constexpr int kMaxCounted = 96;
struct Counted { const char* name; long long count; };
Counted g_counted[kMaxCounted];
int g_counted_used = 0;
std::mutex g_counted_mutex;
}  // namespace

void mir_count_launch(const char* what) {
  std::lock_guard<std::mutex> lock(g_counted_mutex);
  for (int i = 0; i < g_counted_used; ++i)
    if (g_counted[i].name == what) { ++g_counted[i].count; return; }
  for (int i = 0; i < g_counted_used; ++i)
    if (strcmp(g_counted[i].name, what) == 0) { ++g_counted[i].count; return; }
  if (g_counted_used < kMaxCounted) g_counted[g_counted_used++] = Counted{what, 1};
}

// "name=count" lines into `text` (at most `size` bytes with the final zero); returns the bytes it needs.
MIR_EXPORT int mir_launch_counts(char* text, int size) {
  std::lock_guard<std::mutex> lock(g_counted_mutex);
  int needed = 1;
  if (size > 0) text[0] = 0;
  for (int i = 0; i < g_counted_used; ++i) {
    char line[160];
    const int length = snprintf(line, sizeof(line), "%s=%lld\n", g_counted[i].name, g_counted[i].count);
    if (needed + length <= size) memcpy(text + needed - 1, line, (size_t)length + 1);
    needed += length;
  }
  return needed;
}

MIR_EXPORT void mir_reset_launch_counts() {
  std::lock_guard<std::mutex> lock(g_counted_mutex);
  g_counted_used = 0;
}

int mir_check_launch(const char* what) {
  mir_count_launch(what);
  const cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) return MIR_OK;
  mir_set_error("%s: %s", what, cudaGetErrorString(err));
  return MIR_CUDA_ERROR;
}

MIR_EXPORT const char* mir_last_error() { return g_error; }

// Multiprocessors of the current device (148 on a B200; also the answer when the device cannot be asked).
int mir_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0, found = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&found, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && found > 0)
      count = found;
    else
      return 148;
  }
  return count;
}

MIR_EXPORT int mir_abi_version() { return 1; }

// 0 off, 1 every kernel, 2 only the kernels that stream weights before they wait.  Measured inside captured
// decode steps (Qwen3-4B sizes, batch 8): 3.37 ms off, 3.42 ms for every kernel, 3.25 ms for the streaming ones.
static int g_pdl = 2;

bool mir_pdl_enabled() { return g_pdl == 1; }
bool mir_pdl_for_streaming() { return g_pdl >= 1; }

// Which kernels are launched with programmatic stream serialization: see g_pdl.
MIR_EXPORT void mir_set_pdl(int mode) { g_pdl = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }
MIR_EXPORT int mir_get_pdl() { return g_pdl; }
