// Shared helpers of the sm_100a kernels: storage types, warp/block reductions with a
// fixed tree shape, error reporting of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FERRUM_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum FerrumDType : int { FERRUM_F32 = 0, FERRUM_BF16 = 1, FERRUM_F16 = 2 };
inline bool ferrum_is_16bit(int dtype) { return dtype == FERRUM_BF16 || dtype == FERRUM_F16; }

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

// ---- kernel timeline (only in a build with -DFERRUM_TRACE, see ops/build.py)
// Block 0 of an instrumented kernel records three points of the GPU's global timer: entry,
// return from the dependency wait, exit.  Each translation unit has its own ring of records
// [kind, t_entry, t_waited, t_exit] and exports a reader.  Without the macro nothing is
// compiled in.
#ifdef FERRUM_TRACE
constexpr int TRACE_RECORDS = 8192;
static __device__ unsigned long long g_trace[TRACE_RECORDS * 4];
static __device__ unsigned int g_trace_n;
__device__ __forceinline__ unsigned long long trace_clock() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int trace_begin(int kind) {
  const unsigned i = atomicAdd(&g_trace_n, 1u) % TRACE_RECORDS;
  g_trace[i * 4 + 0] = (unsigned long long)kind;
  g_trace[i * 4 + 1] = trace_clock();
  g_trace[i * 4 + 2] = 0;
  g_trace[i * 4 + 3] = 0;
  return (int)i;
}
// `first` is true in the one thread of the grid that keeps the record
#define TRACE_BEGIN(first, kind) const int trace_slot_ = (first) ? trace_begin(kind) : -1
#define TRACE_MARK(field)                                              \
  do {                                                                 \
    if (trace_slot_ >= 0) g_trace[trace_slot_ * 4 + (field)] = trace_clock(); \
  } while (0)
#define FERRUM_TRACE_READER(name)                                                                  \
  FERRUM_API int name(unsigned long long* out, unsigned int* n) {                                 \
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;                                          \
    cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * TRACE_RECORDS * 4);            \
    cudaMemcpyFromSymbol(n, g_trace_n, sizeof(unsigned int));                                      \
    const unsigned int zero = 0;                                                                   \
    cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));                                            \
    return 0;                                                                                      \
  }
#else
#define TRACE_BEGIN(first, kind) ((void)0)
#define TRACE_MARK(field) ((void)0)
#define FERRUM_TRACE_READER(name)
#endif
constexpr int TRACE_WAITED = 2, TRACE_EXIT = 3;
// kinds: 1 product (+ output features / 64 * 16, + 8 for the two-product kernel), 2 norm, 3 rotary,
// 4 swiglu_reduce, 5 attention (mma.sync), 6 combine
constexpr int TRACE_GEMM = 1, TRACE_NORM = 2, TRACE_ROPE = 3, TRACE_SWIGLU_REDUCE = 4, TRACE_FLASH = 5, TRACE_COMBINE = 6;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Two float32 values rounded to the 16-bit type T and packed, the first in the low half.
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The bits of one float32 value rounded to bfloat16 (half = false) or to float16 (half = true),
// for epilogues whose 16-bit type is a run-time parameter.
__device__ __forceinline__ uint16_t bits16(float v, bool half) {
  return half ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ uint32_t pack2_bits(float lo, float hi, bool half) {
  return half ? pack2<__half>(lo, hi) : pack2<__nv_bfloat16>(lo, hi);
}

// Run `body` with T bound to the storage type of a dtype code (float, __nv_bfloat16, __half).
#define FERRUM_DISPATCH_DTYPE(dtype, T, ...)                      \
  do {                                                            \
    if ((dtype) == FERRUM_F32) { using T = float; __VA_ARGS__; }  \
    else if ((dtype) == FERRUM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == FERRUM_F16) { using T = __half; __VA_ARGS__; }         \
    else FERRUM_CHECK_ARG(false, "unknown dtype code %d", (int)(dtype));      \
  } while (0)
#define FERRUM_DISPATCH_16BIT(dtype, T, ...)                      \
  do {                                                            \
    if ((dtype) == FERRUM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == FERRUM_F16) { using T = __half; __VA_ARGS__; }    \
    else FERRUM_CHECK_ARG(false, "dtype code %d is not a 16-bit type", (int)(dtype)); \
  } while (0)

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
