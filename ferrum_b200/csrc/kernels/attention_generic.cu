// Causal grouped-query attention over the paged cache, one warp per (token, query head).
//
// The same code runs a prompt portion and a decoded token: every query reads keys
// kv_lo..pos from the cache (the rotary kernel has already stored this step's keys), in
// chunks of 32 keys in ascending order, with an online softmax in float32.  A row's
// result therefore depends only on its own position and cache contents, never on the
// batch around it.  Formulas: query head h reads KV head h / (Hq/Hkv), score =
// q.k / sqrt(D), stable softmax, weighted sum of V (crates/model/src/llama.rs:220-247;
// crates/kernels/src/scalar.rs:125-141).  `window` > 0 keeps keys in (pos-window, pos].
//
// This is the float32 attention of the engine and the bfloat16 attention for head sizes
// the tensor-core kernels do not take.
#include "common.cuh"

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                         const int* __restrict__ positions, const int* __restrict__ req_of_token,
                         const int* __restrict__ block_table, int table_width, const T* __restrict__ kv_plane,
                         long long page_stride, int page_size, int Hq, int Hkv, int D, float scale, int window,
                         int* __restrict__ err) {
  __shared__ float qs[ATT_WARPS][ATT_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * ATT_WARPS + warp;
  if (h >= Hq) return;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)req_of_token[t] * table_width;
  const int kvh = h / (Hq / Hkv);
  const T* qrow = q + (size_t)t * ldq + (size_t)h * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_f32<T>(qrow[d]);
  __syncwarp();

  const size_t v_off = (size_t)Hkv * page_size * D;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] = 0.f;

  for (int base = lo; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    long long off = -1;  // element offset of this lane's K row
    float s = -INFINITY;
    if (valid) {
      const int lp = key / page_size;
      const int page = lp < table_width ? bt[lp] : -1;
      if (page < 0) {
        atomicExch(err, 5);
      } else {
        off = (long long)page * page_stride + ((long long)kvh * page_size + key % page_size) * D;
        const T* kr = kv_plane + off;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(qs[warp][d], to_f32<T>(kr[d]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // nothing finite yet: weights stay zero
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (off >= 0 && s > -INFINITY) ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAX_D / 32; ++i) acc[i] *= corr;
    const int n = min(32, pos - base + 1);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;
      const T* vr = kv_plane + oj + v_off;
#pragma unroll
      for (int i = 0; i < ATT_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pj, to_f32<T>(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* orow = out + (size_t)t * ldo + (size_t)h * D;
#pragma unroll
  for (int i = 0; i < ATT_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_f32<T>(acc[i] * inv);
  }
}

FERRUM_API int ferrum_attention_generic(const void* q, int ldq, void* out, int ldo, int dtype, int n_tokens,
                                        const int* positions, const int* req_of_token, const int* block_table,
                                        int table_width, const void* kv_plane, long long page_stride, int page_size,
                                        int Hq, int Hkv, int D, float scale, int window, int* err_flag,
                                        cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
  FERRUM_CHECK_ARG(D > 0 && D <= ATT_MAX_D, "attention: head size %d is outside (0, %d]", D, ATT_MAX_D);
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0, "attention: bad cache arguments");
  FERRUM_CHECK_ARG(ldq >= Hq * D && ldo >= Hq * D, "attention: a row stride is shorter than Hq*D");
  if (n_tokens == 0) return 0;
  dim3 grid(n_tokens, (Hq + ATT_WARPS - 1) / ATT_WARPS);
  FERRUM_CHECK_ARG(grid.y <= 65535, "attention: too many heads");
  FERRUM_DISPATCH_DTYPE(dtype, T, (attention_generic_kernel<T><<<grid, ATT_WARPS * 32, 0, stream>>>(
      (const T*)q, ldq, (T*)out, ldo, positions, req_of_token, block_table, table_width, (const T*)kv_plane, page_stride,
      page_size, Hq, Hkv, D, scale, window, err_flag)));
  FERRUM_CHECK_LAUNCH("attention_generic");
  return 0;
}
