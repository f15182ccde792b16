// Timestamps from inside kernels, for looking at a captured decode step on a time line: where a kernel waits for
// the one before it, when its first data is there, how long its epilogue takes.  Compiled in only with -DMIR_TRACE
// (the library "bf16_trace" of build.py, which bench.py --phase trace loads); otherwise every macro here is empty
// and the kernels are exactly what they are without this file.
//
//   MIR_TRACE_DEFINE(name)            at file scope: the records of this file's kernels (16 x 64-bit each: up to 14
//                                     time stamps in ns of %globaltimer, [14] a value of the kernel's choice, [15] a
//                                     tag) and the exported reader mir_trace_read_<name>(host, capacity) -> records
//   MIR_TRACE_BEGIN(name, chosen, tag) in a kernel, by every thread, where the CTA is not yet split into roles: the
//                                     CTAs for which `chosen` holds (say the first and the last of the grid) take a
//                                     record; contains a __syncthreads()
//   MIR_TRACE_POINT(name, index)      by one thread: time stamp number `index` of this CTA's record
//   MIR_TRACE_VALUE(name, value)      by one thread: the record's free value
#pragma once
#include "common.cuh"

#ifdef MIR_TRACE
#define MIR_TRACE_RECORDS 4096
#define MIR_TRACE_DEFINE(name)                                                                                       \
  __device__ unsigned long long g_trace_##name[16 * MIR_TRACE_RECORDS];                                              \
  __device__ int g_trace_next_##name = 0;                                                                            \
  MIR_EXPORT int mir_trace_read_##name(unsigned long long* host, int capacity) {                                     \
    int count = 0;                                                                                                   \
    if (cudaDeviceSynchronize() != cudaSuccess ||                                                                    \
        cudaMemcpyFromSymbol(&count, g_trace_next_##name, sizeof(int)) != cudaSuccess)                               \
      return -1;                                                                                                     \
    count = count < MIR_TRACE_RECORDS ? count : MIR_TRACE_RECORDS;                                                   \
    count = count < capacity ? count : capacity;                                                                     \
    if (count > 0 && cudaMemcpyFromSymbol(host, g_trace_##name, sizeof(unsigned long long) * 16 * count) != cudaSuccess) \
      return -1;                                                                                                     \
    const int zero = 0;                                                                                              \
    cudaMemcpyToSymbol(g_trace_next_##name, &zero, sizeof(int));                                                     \
    return count;                                                                                                    \
  }
#define MIR_TRACE_NOW(result) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(result))
#define MIR_TRACE_BEGIN(name, chosen, tag)                                                                           \
  __shared__ int mir_trace_slot_shared;                                                                              \
  if (threadIdx.x == 0) {                                                                                            \
    mir_trace_slot_shared = -1;                                                                                      \
    if (chosen) {                                                                                                    \
      const int taken = atomicAdd(&g_trace_next_##name, 1);                                                          \
      if (taken < MIR_TRACE_RECORDS) {                                                                               \
        mir_trace_slot_shared = taken;                                                                               \
        for (int i = 0; i < 15; ++i) g_trace_##name[taken * 16 + i] = 0ull;                                          \
        g_trace_##name[taken * 16 + 15] = (unsigned long long)(tag);                                                 \
      }                                                                                                              \
    }                                                                                                                \
  }                                                                                                                  \
  __syncthreads();                                                                                                   \
  const int mir_trace_slot = mir_trace_slot_shared;
#define MIR_TRACE_POINT(name, index)                                                                                 \
  do {                                                                                                               \
    if (mir_trace_slot >= 0) {                                                                                       \
      unsigned long long now_;                                                                                       \
      MIR_TRACE_NOW(now_);                                                                                           \
      g_trace_##name[mir_trace_slot * 16 + (index)] = now_;                                                          \
    }                                                                                                                \
  } while (0)
#define MIR_TRACE_VALUE(name, value)                                                                                 \
  do {                                                                                                               \
    if (mir_trace_slot >= 0) g_trace_##name[mir_trace_slot * 16 + 14] = (unsigned long long)(value);                 \
  } while (0)
#else
#define MIR_TRACE_DEFINE(name)
#define MIR_TRACE_BEGIN(name, chosen, tag)
#define MIR_TRACE_POINT(name, index) do { } while (0)
#define MIR_TRACE_VALUE(name, value) do { } while (0)
#endif
