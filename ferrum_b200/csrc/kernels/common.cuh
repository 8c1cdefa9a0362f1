// Shared helpers of the sm_100a kernels: storage types, warp/block reductions with a
// fixed tree shape, error reporting of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FERRUM_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum FerrumDType : int { FERRUM_F32 = 0, FERRUM_BF16 = 1 };

// Error text of the last failed entry point on this thread (see ferrum_last_error).
void ferrum_set_error(const char* fmt, ...);

#define FERRUM_CHECK_ARG(cond, ...)            \
  do {                                         \
    if (!(cond)) {                             \
      ferrum_set_error(__VA_ARGS__);           \
      return 1;                                \
    }                                          \
  } while (0)

#define FERRUM_CHECK_LAUNCH(name)                                                   \
  do {                                                                              \
    cudaError_t e__ = cudaGetLastError();                                           \
    if (e__ != cudaSuccess) {                                                       \
      ferrum_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__));     \
      return 2;                                                                     \
    }                                                                               \
  } while (0)

// ---- programmatic dependent launch
// A kernel launched through launch_kernel() may start while the kernel before it in the
// stream is still running.  pdl_wait() blocks until that kernel has completed and its writes
// are visible; nothing that an earlier kernel of the stream writes may be read, and nothing it
// reads may be written, before it.  pdl_launch() lets the next kernel of the stream begin its
// own prologue.  In a kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool ferrum_dependent_launch_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ferrum_dependent_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The tree is
// the same for every row, so a row's value does not depend on what else is in the grid.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? smem32[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
