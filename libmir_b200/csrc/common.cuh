// Shared helpers of the sm_100a kernels: storage types, 32-bit loads and stores, warp reductions.
// Every kernel computes in float; T is only how a tensor is stored (float or __nv_bfloat16).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MIR_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes returned by every exported launcher.
enum MirStatus : int {
  MIR_OK = 0,
  MIR_BAD_ARGUMENT = 1,      // a size the kernel does not take; nothing was launched
  MIR_CUDA_ERROR = 2,        // the launch itself failed; mir_last_error() has the text
  MIR_LIBRARY_ERROR = 3,     // cuBLASLt or the driver API refused
};

void mir_set_error(const char* fmt, ...);
int mir_check_launch(const char* what);
int mir_sm_count();
void mir_count_launch(const char* what);   // launches that do not end in mir_check_launch (library products)

// Programmatic dependent launch: a kernel launched this way may be scheduled while the kernel before it in
// the stream is still draining.  Its CTAs run up to mir::grid_dependency_wait() (prefetching what does not
// depend on the earlier kernel, e.g. weights) and block there until the earlier kernel has completed and
// its writes are visible.  Every kernel launched through mir_launch calls grid_dependency_wait() before it
// reads an activation or writes anything, so the order of memory effects is the order of the stream.
bool mir_pdl_enabled();
bool mir_pdl_for_streaming();   // also true in the mode that launches only the weight-streaming kernels this way

template <typename... KernelArgs, typename... Args>
int mir_launch_cluster(bool programmatic, const char* what, void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                       size_t smem, cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = cluster.x;
    attributes[count].val.clusterDim.y = cluster.y;
    attributes[count].val.clusterDim.z = cluster.z;
    ++count;
  }
  if (programmatic) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  if (err != cudaSuccess) {
    mir_set_error("%s: launch failed: %s", what, cudaGetErrorString(err));
    return MIR_CUDA_ERROR;
  }
  return mir_check_launch(what);
}

template <typename... KernelArgs, typename... Args>
int mir_launch_with(bool programmatic, const char* what, void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                    size_t smem, cudaStream_t stream, int cluster_y, Args... args) {
  return mir_launch_cluster(programmatic, what, kernel, grid, block, smem, stream,
                            dim3(1, cluster_y > 0 ? (unsigned)cluster_y : 1u, 1), args...);
}

template <typename... KernelArgs, typename... Args>
int mir_launch(const char* what, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
               cudaStream_t stream, int cluster_y, Args... args) {
  return mir_launch_with(mir_pdl_enabled(), what, kernel, grid, block, smem, stream, cluster_y, args...);
}

namespace mir {
// Row stride (in tokens) of the arrays of partial sums of squares that an accumulating few-rows product leaves for
// the RMSNorm folded into the next product: [tiles of 16 columns][kNormStatStride tokens].
constexpr int kNormStatStride = 32;


// See mir_launch.  Both are no-ops in a kernel that was launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" :::); }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Eight consecutive elements starting at a 16-byte (bf16) or 32-byte (float) aligned address.
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads with a fixed tree: the result depends only on the
// values and on blockDim, never on timing.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = lane < warps ? scratch[lane] : 0.0f;
  total = warp_sum(total);
  return total;
}

}  // namespace mir
