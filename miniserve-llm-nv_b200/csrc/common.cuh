// Shared helpers of the kernel library: element types, error reporting, reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a
// CUDA stream, launches on that stream and returns 0, or a non-zero code after
// storing a message that `ms_last_error()` returns.  Nothing here allocates.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define MS_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python bindings.
enum : int { MS_F32 = 0, MS_BF16 = 1 };

namespace ms {

char* error_buffer();  // defined in runtime.cu

#define MS_FAIL(...)                                                  \
  do {                                                                \
    snprintf(ms::error_buffer(), 512, __VA_ARGS__);                   \
    return 1;                                                         \
  } while (0)

#define MS_REQUIRE(cond, ...)                                         \
  do {                                                                \
    if (!(cond)) MS_FAIL(__VA_ARGS__);                                \
  } while (0)

#define MS_CHECK_LAUNCH(name)                                         \
  do {                                                                \
    cudaError_t e_ = cudaGetLastError();                              \
    if (e_ != cudaSuccess) MS_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
  } while (0)

// Programmatic dependent launch.  Every kernel of this library is launched so that it may start
// while the kernel before it on the stream is still running; it must call `grid_dependency_wait()`
// before it reads anything an earlier kernel wrote and before it writes anything at all (the call
// returns once the earlier kernel has finished and its writes are visible).  What a kernel does before
// that call (fetching weights, which no kernel writes) overlaps with the tail of its predecessor.
// Every thread block calls it on every path, so that a kernel never finishes before its predecessor.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_launch() { asm volatile("griddepcontrol.launch_dependents;" ::); }

bool dependent_launch_enabled();  // defined in runtime.cu

template <typename... Params, typename... Args>
cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Loads element i of an array whose element type is only known at run time.
__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
  return dtype == MS_F32 ? reinterpret_cast<const float*>(p)[i]
                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
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

// Sum over a thread block in a fixed order (same result whatever else runs).
// `scratch` holds at least 32 floats; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < n_warps; ++w) total += scratch[w];
  return total;
}

}  // namespace ms
