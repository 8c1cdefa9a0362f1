// out[t, n] = sum_k x[t, k] * w[n, k] on the CUDA cores, float32 accumulation with FFMA.
//
// This is the true 32-bit matrix product of the engine (the tensor cores have no
// float32 input type; TF32 is not 32-bit), and the bfloat16 product for shapes the
// tcgen05 kernel refuses (rows that are not 16-byte multiples).  Every output element
// is one accumulator that walks k = 0..K-1 in order, so a token's result does not
// depend on how many other tokens are in the call.  The reference's product is the same
// left-to-right dot per output (crates/kernels/src/scalar.rs:221-241).
#include "common.cuh"

enum GemmEpilogue : int {
  EPI_STORE = 0,      // out (same dtype as the inputs) = acc
  EPI_STORE_F32 = 1,  // out (float32) = acc
  EPI_RESIDUAL = 2,   // out (float32) += acc        (the residual sum stays float32)
};

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out, int M, int N, int K,
                    int ldx, int ldw, int ldo) {
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per operand = 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      const int m = m0 + r, n = n0 + r;
      xs[kk][r] = (m < M && k < K) ? to_f32<T>(x[(size_t)m * ldx + k]) : 0.f;
      ws[kk][r] = (n < N && k < K) ? to_f32<T>(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const size_t o = (size_t)m * ldo + n;
      if (EPI == EPI_STORE) ((T*)out)[o] = from_f32<T>(acc[i][j]);
      else if (EPI == EPI_STORE_F32) ((float*)out)[o] = acc[i][j];
      else ((float*)out)[o] += acc[i][j];
    }
  }
}

template <typename T>
static int launch_generic(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                          int epilogue, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  FERRUM_CHECK_ARG(grid.y <= 65535, "gemm: too many row tiles (%u)", grid.y);
  switch (epilogue) {
    case EPI_STORE:
      gemm_generic_kernel<T, EPI_STORE><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, out, M, N, K, ldx, ldw, ldo);
      break;
    case EPI_STORE_F32:
      gemm_generic_kernel<T, EPI_STORE_F32><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, out, M, N, K, ldx, ldw, ldo);
      break;
    case EPI_RESIDUAL:
      gemm_generic_kernel<T, EPI_RESIDUAL><<<grid, 256, 0, stream>>>((const T*)x, (const T*)w, out, M, N, K, ldx, ldw, ldo);
      break;
    default:
      FERRUM_CHECK_ARG(false, "gemm: unknown epilogue %d", epilogue);
  }
  FERRUM_CHECK_LAUNCH("gemm_generic");
  return 0;
}

FERRUM_API int ferrum_gemm_generic(const void* x, const void* w, void* out, int dtype, int M, int N, int K, int ldx,
                                   int ldw, int ldo, int epilogue, cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  FERRUM_CHECK_ARG(ldx >= K && ldw >= K && ldo >= N, "gemm: a row stride is shorter than its row");
  if (M == 0) return 0;
  if (dtype == FERRUM_F32) return launch_generic<float>(x, w, out, M, N, K, ldx, ldw, ldo, epilogue, stream);
  if (dtype == FERRUM_BF16) return launch_generic<__nv_bfloat16>(x, w, out, M, N, K, ldx, ldw, ldo, epilogue, stream);
  FERRUM_CHECK_ARG(false, "gemm: unknown dtype code %d", dtype);
}
