// out[t, n] = sum_k x[t, k] * w[n, k] on the CUDA cores, float32 accumulation with FFMA.
//
// This is the true 32-bit matrix product of the engine (the tensor cores have no float32
// input type; TF32 is not 32-bit), and the 16-bit product for shapes the tcgen05 kernel
// refuses (rows that are not 16-byte multiples).  The reference's product is a left-to-right
// dot per output (crates/kernels/src/scalar.rs:221-241).  Two kernels:
//
// Tiled (more than 64 tokens): a CTA computes BM tokens x 128 features; both operands are
// K-major, so a thread fetches 16 bytes along K of one row, and the 16-wide k-slices go into
// shared memory transposed ([k][row]), double buffered: the loads of slice i + 1 are in flight
// while slice i is multiplied.  A thread owns BM/16 x 8 outputs in registers.  Every output is
// ONE accumulator that walks k = 0..K-1 in order.
//
// Skinny (up to 64 tokens: decoding): the product is a stream of the weights.  A CTA owns 8
// features; its 8 warps cut K into 8 contiguous ranges of whole 128-element blocks (a function
// of K alone); a lane walks its 4 elements of every block of its warp's range in order; the
// 32 lanes meet in a fixed shuffle tree and the 8 warps are added in warp order.  (Measured on
// Llama-3.1-8B shapes with 8 tokens: 43 to 60 % of the copy bandwidth, 65 % with one token; four
// features per CTA with the next block's weights requested ahead was no faster.)
//
// Stream (float32 with 16-byte aligned rows, up to 64 tokens in passes of 8: the decode steps of
// the 32-bit path; the skinny kernel remains for 16-bit types and unaligned rows):
// the skinny kernel keeps too few bytes on their way (its loads wait in registers for the
// multiplications before them: 22 % of the warp slots busy, 46 % of the copy bandwidth at 8
// tokens).  Here a CTA of 8 features brings 512-element slices of its weight rows and of the
// tokens' rows into a ring of three shared-memory stages with cp.async, two stages ahead of the
// arithmetic, and nothing passes through registers on the way.  A thread owns four consecutive k
// of every slice for 8 features x 4 tokens; at the end the 32 sums of a lane meet the other
// lanes' in a butterfly that halves the values at every step (31 shuffles), and the four warps
// of a token group are added in warp order.
//
// In all kernels the order of the sum of an output is a function of K only, so a token's
// result does not depend on how many other tokens are in the call or where it stands among
// them.  (Between the kernels the orders differ: a token decoded alone and the same token
// inside a larger batch agree to rounding, not bitwise.)
#include "common.cuh"

enum GemmEpilogue : int {
  EPI_STORE = 0,      // out (same dtype as the inputs) = acc
  EPI_STORE_F32 = 1,  // out (float32) = acc
  EPI_RESIDUAL = 2,   // out (float32) += acc        (the residual sum stays float32)
};

template <typename T>
__device__ __forceinline__ void epilogue_store(void* out, size_t o, float v, int epi) {
  if (epi == EPI_STORE) ((T*)out)[o] = from_f32<T>(v);
  else if (epi == EPI_STORE_F32) ((float*)out)[o] = v;
  else ((float*)out)[o] += v;
}

// ------------------------------------------------------------------ tiled kernel
constexpr int TBN = 128, TBK = 16;
constexpr int TLV = TBK / 8;      // 16-byte pieces of a slice that a thread brings per operand

// VEC: float32 operands whose rows start on 16-byte boundaries and K a multiple of 4.
template <typename T, int BM, bool VEC>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out, int M, int N, int K, int ldx,
                  int ldw, int ldo, int epi) {
  constexpr int TM = BM / 16;               // outputs per thread along the tokens
  constexpr int A_VECS = BM * 8 / 4;        // 16-byte pieces of eight k of a token slice (at most 256)
  __shared__ __align__(16) float xs[2][TBK][BM];
  __shared__ __align__(16) float ws[2][TBK][TBN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * TBN;
  // this thread's pieces of a slice: row lr, k offsets lk (0 or 4) + 8 q
  const int lr = tid >> 1, lk = (tid & 1) * 4;
  const bool a_loader = tid < A_VECS;
  const T* xrow = x + (size_t)min(m0 + lr, M - 1) * ldx;
  const T* wrow = w + (size_t)min(n0 + lr, N - 1) * ldw;
  const bool a_ok = a_loader && m0 + lr < M, b_ok = n0 + lr < N;

  float acc[TM][8];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float ra[TLV][4], rb[TLV][4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int q = 0; q < TLV; ++q) {
      const int k = k0 + q * 8 + lk;
      if (VEC) {
        const float4 za = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 a = (a_ok && k < K) ? *reinterpret_cast<const float4*>((const float*)xrow + k) : za;
        const float4 b = (b_ok && k < K) ? *reinterpret_cast<const float4*>((const float*)wrow + k) : za;
        ra[q][0] = a.x; ra[q][1] = a.y; ra[q][2] = a.z; ra[q][3] = a.w;
        rb[q][0] = b.x; rb[q][1] = b.y; rb[q][2] = b.z; rb[q][3] = b.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ra[q][i] = (a_ok && k + i < K) ? to_f32<T>(xrow[k + i]) : 0.f;
          rb[q][i] = (b_ok && k + i < K) ? to_f32<T>(wrow[k + i]) : 0.f;
        }
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int q = 0; q < TLV; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (a_loader) xs[buf][q * 8 + lk + i][lr] = ra[q][i];
        ws[buf][q * 8 + lk + i][lr] = rb[q][i];
      }
  };

  const int n_slices = (K + TBK - 1) / TBK;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int s = 0; s < n_slices; ++s) {
    const int buf = s & 1;
    if (s + 1 < n_slices) fetch((s + 1) * TBK);   // in flight during the arithmetic below
#pragma unroll
    for (int kk = 0; kk < TBK; ++kk) {
      float a[TM], b[8];
      if (TM >= 4) {
#pragma unroll
        for (int g = 0; g < TM / 4; ++g) {
          const float4 v = *reinterpret_cast<const float4*>(&xs[buf][kk][g * 64 + ty * 4]);
          a[g * 4] = v.x; a[g * 4 + 1] = v.y; a[g * 4 + 2] = v.z; a[g * 4 + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = xs[buf][kk][ty * TM + i];
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(&ws[buf][kk][g * 64 + tx * 4]);
        b[g * 4] = v.x; b[g * 4 + 1] = v.y; b[g * 4 + 2] = v.z; b[g * 4 + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (s + 1 < n_slices) {
      stash(buf ^ 1);      // the other buffer: nobody reads it during this slice
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + (TM >= 4 ? (i / 4) * 64 + ty * 4 + (i & 3) : ty * TM + i);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j / 4) * 64 + tx * 4 + (j & 3);
      if (n < N) epilogue_store<T>(out, (size_t)m * ldo + n, acc[i][j], epi);
    }
  }
}

// ------------------------------------------------------------------ skinny kernel
constexpr int SK_FEAT = 8;     // features per CTA
constexpr int SK_WARPS = 8;    // warps per CTA: K ranges
constexpr int SK_TOK = 8;      // tokens per pass
constexpr int SK_MAX_TOKENS = 64;   // in passes of SK_TOK tokens: the weights of the later passes come from the L2

template <typename T, bool VEC>
__global__ void __launch_bounds__(SK_WARPS * 32, 2)
gemm_skinny_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ out, int M, int N, int K, int ldx,
                   int ldw, int ldo, int epi) {
  __shared__ float part[SK_WARPS][SK_FEAT][SK_TOK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * SK_FEAT;
  const int n_blocks = (K + 127) / 128;
  const int b_begin = n_blocks * warp / SK_WARPS, b_end = n_blocks * (warp + 1) / SK_WARPS;
  const T* wr[SK_FEAT];
#pragma unroll
  for (int f = 0; f < SK_FEAT; ++f) wr[f] = w + (size_t)min(n0 + f, N - 1) * ldw;

  for (int m0 = 0; m0 < M; m0 += SK_TOK) {
    float acc[SK_FEAT][SK_TOK];
#pragma unroll
    for (int f = 0; f < SK_FEAT; ++f)
#pragma unroll
      for (int m = 0; m < SK_TOK; ++m) acc[f][m] = 0.f;
#pragma unroll 1
    for (int b = b_begin; b < b_end; ++b) {
      const int k = b * 128 + lane * 4;
      float wv[SK_FEAT][4];
      if (VEC) {
#pragma unroll
        for (int f = 0; f < SK_FEAT; ++f) {
          const float4 v = k < K ? __ldcs(reinterpret_cast<const float4*>((const float*)wr[f] + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
          wv[f][0] = v.x; wv[f][1] = v.y; wv[f][2] = v.z; wv[f][3] = v.w;
        }
      } else {
#pragma unroll
        for (int f = 0; f < SK_FEAT; ++f)
#pragma unroll
          for (int i = 0; i < 4; ++i) wv[f][i] = k + i < K ? to_f32<T>(wr[f][k + i]) : 0.f;
      }
#pragma unroll
      for (int m = 0; m < SK_TOK; ++m) {
        float xv[4] = {0.f, 0.f, 0.f, 0.f};
        if (m0 + m < M) {
          const T* xr = x + (size_t)(m0 + m) * ldx;
          if (VEC) {
            if (k < K) {
              const float4 v = *reinterpret_cast<const float4*>((const float*)xr + k);
              xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = k + i < K ? to_f32<T>(xr[k + i]) : 0.f;
          }
        }
#pragma unroll
        for (int f = 0; f < SK_FEAT; ++f)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[f][m] = fmaf(wv[f][i], xv[i], acc[f][m]);
      }
    }
#pragma unroll
    for (int f = 0; f < SK_FEAT; ++f)
#pragma unroll
      for (int m = 0; m < SK_TOK; ++m) {
        const float v = warp_sum(acc[f][m]);
        if (lane == 0) part[warp][f][m] = v;
      }
    __syncthreads();
    if (threadIdx.x < SK_FEAT * SK_TOK) {
      const int f = threadIdx.x % SK_FEAT, m = threadIdx.x / SK_FEAT;
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < SK_WARPS; ++wi) v += part[wi][f][m];
      if (n0 + f < N && m0 + m < M) epilogue_store<T>(out, (size_t)(m0 + m) * ldo + n0 + f, v, epi);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ stream kernel (float32, a few tokens)
constexpr int ST_FEAT = 8;       // features per CTA
constexpr int ST_TOK = 8;        // tokens at most
constexpr int ST_KT = 512;       // elements of K per stage
constexpr int ST_STAGES = 3;
constexpr int ST_THREADS = 256;
constexpr int ST_STAGE_FLOATS = (ST_FEAT + ST_TOK) * ST_KT;
constexpr int ST_SMEM_BYTES = ST_STAGES * ST_STAGE_FLOATS * 4;

__device__ __forceinline__ void st_cp_async16(void* smem, const void* gmem, int src_bytes) {   // src_bytes 0: sixteen zero bytes
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(ST_THREADS, 2)
gemm_stream_kernel(const float* __restrict__ x, const float* __restrict__ w, void* __restrict__ out, int M, int N, int K,
                   int ldx, int ldw, int ldo, int epi) {
  extern __shared__ __align__(16) float st_smem[];
  __shared__ float red[ST_THREADS / 32][32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * ST_FEAT;
  const int n_stages = (K + ST_KT - 1) / ST_KT;
  const int kq = tid & 127, tg = tid >> 7;   // this thread: elements kq * 4 .. + 3 of every stage, tokens tg * 4 .. + 3 of the pass
  static_assert(ST_FEAT == ST_TOK, "one loop brings a stage's weight rows and token rows");
  // More than 8 tokens go in passes of 8; the later passes find the CTA's weight rows in the L2.
  for (int m0 = 0; m0 < M; m0 += ST_TOK) {
    // stage s of K into its place in the ring: rows past N or M and elements past K arrive as zeros
    auto load_stage = [&](int s) {
      float* const ws = st_smem + (s % ST_STAGES) * ST_STAGE_FLOATS;
      float* const xs = ws + ST_FEAT * ST_KT;
      const int k0 = s * ST_KT;
#pragma unroll
      for (int i = tid; i < ST_FEAT * (ST_KT / 4); i += ST_THREADS) {
        const int r = i / (ST_KT / 4), c = (i % (ST_KT / 4)) * 4;
        const bool wt = n0 + r < N && k0 + c < K;
        st_cp_async16(&ws[r * ST_KT + c], w + (wt ? (size_t)(n0 + r) * ldw + k0 + c : 0), wt ? 16 : 0);
        const bool xt = m0 + r < M && k0 + c < K;
        st_cp_async16(&xs[r * ST_KT + c], x + (xt ? (size_t)(m0 + r) * ldx + k0 + c : 0), xt ? 16 : 0);
      }
    };
#pragma unroll
    for (int s = 0; s < ST_STAGES - 1; ++s) {
      if (s < n_stages) load_stage(s);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[ST_FEAT][4];
#pragma unroll
    for (int f = 0; f < ST_FEAT; ++f)
#pragma unroll
      for (int m = 0; m < 4; ++m) acc[f][m] = 0.f;
    for (int s = 0; s < n_stages; ++s) {
      // (the stage this load overwrites was read in the iteration before, which ended with a barrier)
      if (s + ST_STAGES - 1 < n_stages) load_stage(s + ST_STAGES - 1);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group %0;" ::"n"(ST_STAGES - 1) : "memory");   // all but the newest two groups: stage s is there
      __syncthreads();
      const float* const ws = st_smem + (s % ST_STAGES) * ST_STAGE_FLOATS;
      const float* const xs = ws + ST_FEAT * ST_KT;
      float4 xv[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) xv[m] = *reinterpret_cast<const float4*>(&xs[(tg * 4 + m) * ST_KT + kq * 4]);
#pragma unroll
      for (int f = 0; f < ST_FEAT; ++f) {
        const float4 wv = *reinterpret_cast<const float4*>(&ws[f * ST_KT + kq * 4]);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          acc[f][m] = fmaf(wv.x, xv[m].x, acc[f][m]);
          acc[f][m] = fmaf(wv.y, xv[m].y, acc[f][m]);
          acc[f][m] = fmaf(wv.z, xv[m].z, acc[f][m]);
          acc[f][m] = fmaf(wv.w, xv[m].w, acc[f][m]);
        }
      }
      __syncthreads();
    }
    // ---- the 32 lanes meet: at every step a lane keeps the half of its values that its partner
    // sends the other half of; after five steps lane i holds the warp's sum of value i = f * 4 + m
    float v[32];
#pragma unroll
    for (int f = 0; f < ST_FEAT; ++f)
#pragma unroll
      for (int m = 0; m < 4; ++m) v[f * 4 + m] = acc[f][m];
#pragma unroll
    for (int step = 0; step < 5; ++step) {
      const int off = 16 >> step, half = 16 >> step;     // values kept after this step
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float mine = upper ? v[i + half] : v[i];
        const float theirs = upper ? v[i] : v[i + half];
        v[i] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
      }
    }
    red[warp][lane] = v[0];
    __syncthreads();
    if (tid < 2 * 32) {
      const int g = tid >> 5, i = tid & 31;        // token group, value index
      float sum = 0.f;
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) sum += red[g * 4 + wi][i];
      const int m = m0 + g * 4 + (i & 3), n = n0 + (i >> 2);
      if (m < M && n < N) epilogue_store<float>(out, (size_t)m * ldo + n, sum, epi);
    }
    __syncthreads();     // `red` and the ring are free for the next pass
  }
}

template <typename T>
static int launch_generic(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                          int epilogue, cudaStream_t stream) {
  FERRUM_CHECK_ARG(epilogue >= EPI_STORE && epilogue <= EPI_RESIDUAL, "gemm: unknown epilogue %d", epilogue);
  const bool vec = sizeof(T) == 4 && K % 4 == 0 && ldx % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
  const T* xp = (const T*)x;
  const T* wp = (const T*)w;
  if constexpr (sizeof(T) == 4) {
    if (vec && M <= SK_MAX_TOKENS) {
      static bool configured = false;
      if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM_BYTES);
        FERRUM_CHECK_ARG(e == cudaSuccess, "gemm: cannot reserve %d bytes of shared memory: %s", ST_SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
      }
      gemm_stream_kernel<<<(N + ST_FEAT - 1) / ST_FEAT, ST_THREADS, ST_SMEM_BYTES, stream>>>((const float*)x, (const float*)w, out, M, N, K,
                                                                                           ldx, ldw, ldo, epilogue);
      FERRUM_CHECK_LAUNCH("gemm_generic");
      return 0;
    }
  }
  if (M <= SK_MAX_TOKENS) {
    const dim3 grid((N + SK_FEAT - 1) / SK_FEAT);
    if (vec) gemm_skinny_kernel<T, true><<<grid, SK_WARPS * 32, 0, stream>>>(xp, wp, out, M, N, K, ldx, ldw, ldo, epilogue);
    else gemm_skinny_kernel<T, false><<<grid, SK_WARPS * 32, 0, stream>>>(xp, wp, out, M, N, K, ldx, ldw, ldo, epilogue);
    FERRUM_CHECK_LAUNCH("gemm_generic");
    return 0;
  }
  const int bm = M <= 256 ? 64 : 128;     // (smaller tiles while the grid would not fill the GPU)
  const dim3 grid((N + TBN - 1) / TBN, (M + bm - 1) / bm);
  FERRUM_CHECK_ARG(grid.y <= 65535, "gemm: too many row tiles (%u)", grid.y);
#define TILED(BM_)                                                                                                        \
  do {                                                                                                                    \
    if (vec) gemm_tiled_kernel<T, BM_, true><<<grid, 256, 0, stream>>>(xp, wp, out, M, N, K, ldx, ldw, ldo, epilogue);   \
    else gemm_tiled_kernel<T, BM_, false><<<grid, 256, 0, stream>>>(xp, wp, out, M, N, K, ldx, ldw, ldo, epilogue);      \
  } while (0)
  if (bm == 64) TILED(64);
  else TILED(128);
#undef TILED
  FERRUM_CHECK_LAUNCH("gemm_generic");
  return 0;
}

FERRUM_API int ferrum_gemm_generic(const void* x, const void* w, void* out, int dtype, int M, int N, int K, int ldx,
                                   int ldw, int ldo, int epilogue, cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  FERRUM_CHECK_ARG(ldx >= K && ldw >= K && ldo >= N, "gemm: a row stride is shorter than its row");
  if (M == 0) return 0;
  FERRUM_DISPATCH_DTYPE(dtype, T, return launch_generic<T>(x, w, out, M, N, K, ldx, ldw, ldo, epilogue, stream));
  return 0;
}
