/* An entry point of the kernel library for callers that must not allocate device memory.
 *
 * This has no counterpart in the reference (JustinA988/ferrum is CPU-only and allocates its
 * buffers with ordinary vectors); it exists for embedders of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- inside a host that has
 * already handed all device memory to its own pool allocator and forbids further driver
 * allocations, inside a real-time or safety-certified loop where allocation latency and
 * failure are not acceptable, or inside a plugin whose memory the host application owns.
 * Such callers can pass their own input and output buffers, but they cannot provide the
 * float32 partial-sum workspace and the tile counters that the tensor-core product needs
 * when several CTAs share an output tile.
 *
 * ferrum_gemm_tc_noalloc computes the same bfloat16 product as ferrum_gemm_tc,
 *     out[t, n] (op)= sum_k x[t, k] * w[n, k],
 * but keeps that scratch in a fixed array inside the library's device image instead of
 * taking it from the caller.  It calls no cudaMalloc, cudaFree or any allocating library
 * routine.
 *
 * Limits: the scratch array is FERRUM_NOALLOC_SCRATCH_BYTES (16 MiB) plus
 * FERRUM_NOALLOC_MAX_TILES counters, and every GPU that loads the library holds it until the
 * process exits.  A call whose shape needs more (roughly: more than 64 tokens, or more than
 * 32 with the SwiGLU epilogue, on a 148-SM part; or more than 4096 output tiles) is refused
 * with a non-zero return code and a message from ferrum_last_error(); nothing is launched.
 *
 * Set-up: the first call on a device looks up the array's device address (once per device,
 * with that device current).  Make that first call outside of any CUDA stream capture.
 *
 * Sharing: every call on a device uses the same array and the array keeps the last call's
 * contents.  The entry point clears the counters (the only part that must start at zero) on
 * the caller's stream before each launch.  Two calls that may run at the same time on one
 * GPU -- on different streams, or from different threads -- race on the array: serialise
 * them on one stream.
 *
 * Arguments are those of ferrum_gemm_tc without the workspace, counters and grid size:
 *   x [M, K] bfloat16 (row stride ldx), w [w_rows, K] bfloat16 (row stride ldw),
 *   out [M, ldo]: bfloat16 for epilogue 0 (store) and 3 (SwiGLU), float32 for 1 (store) and
 *   2 (out += product); dual_offset > 0 selects the SwiGLU epilogue's second weight rows;
 *   err_flag: one int32 in device memory that a kernel-side timeout sets non-zero.
 * Returns 0 on success.
 */
#pragma once
#include <cuda_runtime.h>

#define FERRUM_NOALLOC_SCRATCH_BYTES (16u << 20)
#define FERRUM_NOALLOC_MAX_TILES 4096

#ifdef __cplusplus
extern "C" {
#endif

int ferrum_gemm_tc_noalloc(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                           int w_rows, int epilogue, int dual_offset, int* err_flag, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
