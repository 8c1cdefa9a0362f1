// Memory-bound kernels of the step: embedding gather, RMSNorm, rotary encoding fused
// with the paged cache write, SwiGLU.  All arithmetic is float32; storage is float32,
// bfloat16 or float16.  Formulas follow the reference's scalar kernels
// (crates/kernels/src/scalar.rs:143-156 rms, :167-189 rope; crates/kernels/src/math.rs:8-10 silu).
#include "common.cuh"
#include "partials.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (the residual stream is float32 in every mode).
// An id outside [0, V) writes zeros and raises the error flag: never a wild read.
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int E, int V, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;
  if (!ok && threadIdx.x == 0) atomicExch(err, 1);
  const T* row = table + (size_t)(ok ? id : 0) * E;
  float* o = out + (size_t)t * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = ok ? to_f32<T>(row[i]) : 0.f;
}

FERRUM_API int ferrum_embedding(const void* table, int dtype, const int* ids, float* out, int n_tokens,
                                int E, int V, int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && E > 0 && V > 0, "embedding: bad sizes T=%d E=%d V=%d", n_tokens, E, V);
  if (n_tokens == 0) return 0;
  const int threads = E >= 1024 ? 256 : 128;
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(embedding_kernel<T>, n_tokens, threads, 0, stream, (const T*)table, ids, out, E, V, err_flag));
  FERRUM_CHECK_LAUNCH("embedding");
  return 0;
}

// ---------------------------------------------------------------- RMSNorm
// out[r, i] = x[src(r), i] * rsqrt(mean(x^2) + eps) * w[i]; src(r) = rows ? rows[r] : r.
// One block per row, the same reduction tree for every row.
template <typename TOut>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TOut* __restrict__ out, const int* __restrict__ rows, int E, float eps) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * E;
  float ss = 0.f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)E + eps);
  TOut* o = out + (size_t)r * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TOut>(xr[i] * inv * w[i]);
}

// Many rows of a width that is a multiple of 4: one block per row, float4 loads, the row kept
// in registers between the sum of squares and the scaling (read once, written once).
constexpr int NORM_VEC_MAX = 4;  // float4 per thread
// pack2 for an output type that may also be float (a branch the compiler removes for float)
template <typename TOut> __device__ __forceinline__ uint32_t pack2_out(float lo, float hi) { return pack2<TOut>(lo, hi); }
template <> __device__ __forceinline__ uint32_t pack2_out<float>(float, float) { return 0u; }
template <typename TOut>
__global__ void __launch_bounds__(512)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ out,
                   const int* __restrict__ rows, int E, float eps) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * E);
  const int n4 = E >> 2;
  float4 v[NORM_VEC_MAX];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_VEC_MAX; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)E + eps);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  TOut* o = out + (size_t)r * E;
#pragma unroll
  for (int k = 0; k < NORM_VEC_MAX; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i >= n4) continue;
    const float4 g = w4[i];
    const float a = v[k].x * inv * g.x, b = v[k].y * inv * g.y, c = v[k].z * inv * g.z, d = v[k].w * inv * g.w;
    if (sizeof(TOut) == 4) {
      reinterpret_cast<float4*>(o)[i] = make_float4(a, b, c, d);
    } else {
      uint2 pk;
      pk.x = pack2_out<TOut>(a, b);
      pk.y = pack2_out<TOut>(c, d);
      reinterpret_cast<uint2*>(o)[i] = pk;
    }
  }
}

// The norm of a few rows spread over a cluster of CTAs: with 8 rows and one CTA per row the
// kernel is a chain of memory latencies on 8 SMs.  Here NORM_CLUSTER CTAs share a row; each
// sums its slice (adding pending partials if any) and keeps it in registers, sends its sum of
// squares to every CTA of the cluster through distributed shared memory, and adds the eight
// sums in rank order, so the result is the same whichever CTA finishes first.
constexpr int NORM_CLUSTER = 8;
constexpr int NORM_KEEP = 4;  // elements a thread keeps between the two passes (more are read again)

__device__ __forceinline__ unsigned norm_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void norm_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void norm_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void norm_store_to_peer(float* local, unsigned rank, float v) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), peer;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer), "f"(v) : "memory");
}

template <typename TOut>
__global__ void __launch_bounds__(256)
rmsnorm_cluster_kernel(float* __restrict__ h, const float* __restrict__ w, TOut* __restrict__ out,
                       const int* __restrict__ rows, int E, float eps, const PartialLayout L) {
  __shared__ float red[32];
  __shared__ float slice_sums[NORM_CLUSTER];   // written by the CTAs of the cluster, one entry each
  __shared__ PartialTable tab;
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0, TRACE_NORM);
  // A CTA's shared memory may be written by a peer only once the CTA is known to run: every CTA
  // arrives here and waits for the others before it sends its sum (by then they have long arrived).
  norm_cluster_arrive();
  if (L.ws != nullptr) build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  const int r = blockIdx.x;
  const unsigned rank = norm_cluster_rank();
  const int src = rows ? rows[r] : r;
  const int per = (E + NORM_CLUSTER - 1) / NORM_CLUSTER;
  const int lo = rank * per, hi = min(E, lo + per);
  float* hr = h + (size_t)src * E;
  float keep[NORM_KEEP];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_KEEP; ++k) {
    const int i = lo + threadIdx.x + k * 256;
    float v = 0.f;
    if (i < hi) {
      v = hr[i];
      if (L.ws != nullptr) {
        v += partial_sum(L, tab, src, i);
        hr[i] = v;
      }
    }
    keep[k] = v;
    ss = fmaf(v, v, ss);
  }
  for (int i = lo + threadIdx.x + NORM_KEEP * 256; i < hi; i += 256) {  // rows wider than 8192
    float v = hr[i];
    if (L.ws != nullptr) {
      v += partial_sum(L, tab, src, i);
      hr[i] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  norm_cluster_wait();
  if (threadIdx.x < NORM_CLUSTER) norm_store_to_peer(&slice_sums[rank], threadIdx.x, ss);
  norm_cluster_arrive();
  norm_cluster_wait();
  float total = 0.f;
#pragma unroll
  for (int c = 0; c < NORM_CLUSTER; ++c) total += slice_sums[c];
  const float inv = 1.0f / sqrtf(total / (float)E + eps);
  TOut* o = out + (size_t)r * E;
#pragma unroll
  for (int k = 0; k < NORM_KEEP; ++k) {
    const int i = lo + threadIdx.x + k * 256;
    if (i < hi) o[i] = from_f32<TOut>(keep[k] * inv * w[i]);
  }
  for (int i = lo + threadIdx.x + NORM_KEEP * 256; i < hi; i += 256) o[i] = from_f32<TOut>(hr[i] * inv * w[i]);
  TRACE_MARK(TRACE_EXIT);
}

template <typename TOut>
static cudaError_t launch_norm_cluster(float* h, const float* w, TOut* out, const int* rows, int n_rows, int E, float eps,
                                       const PartialLayout& L, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_rows, NORM_CLUSTER);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = NORM_CLUSTER;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ferrum_dependent_launch_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, rmsnorm_cluster_kernel<TOut>, h, w, out, rows, E, eps, L);
}

// Rows at or below this count take the cluster kernel.
constexpr int NORM_CLUSTER_MAX_ROWS = 64;

FERRUM_API int ferrum_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows,
                              int n_rows, int E, float eps, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_rows >= 0 && E > 0, "rmsnorm: bad sizes rows=%d E=%d", n_rows, E);
  FERRUM_CHECK_ARG(eps > 0.f, "rmsnorm: eps must be positive");
  if (n_rows == 0) return 0;
  if (n_rows <= NORM_CLUSTER_MAX_ROWS && E >= 128) {
    const PartialLayout none{nullptr, 0, 0, 0, 0};
    cudaError_t e = cudaErrorInvalidValue;
    FERRUM_DISPATCH_DTYPE(out_dtype, T, e = launch_norm_cluster<T>(const_cast<float*>(x), w, (T*)out, rows, n_rows, E, eps, none, stream));
    FERRUM_CHECK_ARG(e == cudaSuccess, "rmsnorm: cluster launch failed: %s", cudaGetErrorString(e));
    return 0;
  }
  if (E % 4 == 0 && E >= 512 && E <= 4 * NORM_VEC_MAX * 512 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
      ((uintptr_t)out & 15) == 0) {
    const int n4 = E / 4;
    const int vthreads = n4 >= 2048 ? 512 : (n4 >= 512 ? 256 : 128);
    FERRUM_DISPATCH_DTYPE(out_dtype, T, launch_kernel(rmsnorm_vec_kernel<T>, n_rows, vthreads, 0, stream, x, w, (T*)out, rows, E, eps));
    FERRUM_CHECK_LAUNCH("rmsnorm");
    return 0;
  }
  const int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : 128);
  FERRUM_DISPATCH_DTYPE(out_dtype, T, launch_kernel(rmsnorm_kernel<T>, n_rows, threads, 0, stream, x, w, (T*)out, rows, E, eps));
  FERRUM_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// The same norm for a residual stream whose last product is still in partials: first
// h[r, :] += sum of the partials (the deferred residual sum, float32), then the norm.
template <typename TOut>
__global__ void rmsnorm_reduce_kernel(float* __restrict__ h, const float* __restrict__ w, TOut* __restrict__ out,
                                      const int* __restrict__ rows, int E, float eps, const PartialLayout L) {
  __shared__ float red[32];
  __shared__ PartialTable tab;
  build_partial_table(L, tab);   // shapes only: may run before the dependency wait
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* hr = h + (size_t)src * E;
  float ss = 0.f;
#pragma unroll 4
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    const float v = hr[i] + partial_sum(L, tab, src, i);
    hr[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);  // also orders the writes above before the reads below
  const float inv = 1.0f / sqrtf(ss / (float)E + eps);
  TOut* o = out + (size_t)r * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = from_f32<TOut>(hr[i] * inv * w[i]);
}

// h[r, :] += partials, nothing else (for a consumer that does not know about partials).
__global__ void residual_reduce_kernel(float* __restrict__ h, int E, const PartialLayout L) {
  __shared__ PartialTable tab;
  build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  float* hr = h + (size_t)blockIdx.x * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) hr[i] += partial_sum(L, tab, blockIdx.x, i);
}

static int make_layout(const float* ws, const int* layout, PartialLayout* L) {
  FERRUM_CHECK_ARG(ws && layout && layout[0] > 0 && layout[1] > 0 && layout[2] > 0 && layout[3] > 0, "partials: bad layout");
  FERRUM_CHECK_ARG(layout[1] <= PARTIAL_MAX_TILES && layout[2] < 65536, "partials: more than %d tiles", PARTIAL_MAX_TILES);
  {
    // a tile's contributors must fit the 32 slot bits: ranges are at least U/P units long
    const long long per = (long long)layout[0] * layout[1] / layout[2];
    FERRUM_CHECK_ARG(per > 0 && layout[0] / per + 2 <= PARTIAL_MAX_CONTRIB, "partials: too many CTAs share a tile");
  }
  L->ws = ws;
  L->nkb = layout[0];
  L->tiles = layout[1];
  L->n_ctas = layout[2];
  L->acc_cols = layout[3];
  return 0;
}

FERRUM_API int ferrum_rmsnorm_reduce(float* h, const float* w, void* out, int out_dtype, const int* rows, int n_rows,
                                     int E, float eps, const float* partials, const int* layout, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_rows >= 0 && E > 0 && eps > 0.f, "rmsnorm_reduce: bad arguments");
  if (n_rows == 0) return 0;
  PartialLayout L;
  if (int r = make_layout(partials, layout, &L)) return r;
  FERRUM_CHECK_ARG(E <= L.tiles * 128, "rmsnorm_reduce: the partials cover %d features, the rows have %d", L.tiles * 128, E);
  if (n_rows <= NORM_CLUSTER_MAX_ROWS && E >= 128) {
    cudaError_t e = cudaErrorInvalidValue;
    FERRUM_DISPATCH_DTYPE(out_dtype, T, e = launch_norm_cluster<T>(h, w, (T*)out, rows, n_rows, E, eps, L, stream));
    FERRUM_CHECK_ARG(e == cudaSuccess, "rmsnorm_reduce: cluster launch failed: %s", cudaGetErrorString(e));
    return 0;
  }
  const int threads = E >= 2048 ? 1024 : (E >= 512 ? 256 : 128);  // many loads per element: many threads
  FERRUM_DISPATCH_DTYPE(out_dtype, T, launch_kernel(rmsnorm_reduce_kernel<T>, n_rows, threads, 0, stream, h, w, (T*)out, rows, E, eps, L));
  FERRUM_CHECK_LAUNCH("rmsnorm_reduce");
  return 0;
}

FERRUM_API int ferrum_residual_reduce(float* h, int n_rows, int E, const float* partials, const int* layout,
                                      cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_rows >= 0 && E > 0, "residual_reduce: bad arguments");
  if (n_rows == 0) return 0;
  PartialLayout L;
  if (int r = make_layout(partials, layout, &L)) return r;
  FERRUM_CHECK_ARG(E <= L.tiles * 128 && n_rows <= L.acc_cols, "residual_reduce: the partials do not cover the rows");
  launch_kernel(residual_reduce_kernel, n_rows, 256, 0, stream, h, E, L);
  FERRUM_CHECK_LAUNCH("residual_reduce");
  return 0;
}

// ---------------------------------------------------------------- rotary + cache write
// qkv: [T, ld] rows of (q: Hq*D | k: Hkv*D | v: Hkv*D).  q is rotated in place; k is
// rotated and stored, v is stored, both at page block_table[req][pos / ps], row pos % ps.
// A page holds K[Hkv][ps][D] then V[Hkv][ps][D].  cos_sin: [n_pos, R/2, 2] float32.
// pairing 0: (2i, 2i+1); pairing 1: (i, i + R/2).  Dimensions R..D are copied unchanged.
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                                  const int* __restrict__ req_of_token, const int* __restrict__ block_table,
                                  int table_width, const float* __restrict__ cos_sin, int n_pos,
                                  T* __restrict__ kv_plane, long long page_stride, int page_size, int Hq,
                                  int Hkv, int D, int R, int pairing, int write_kv, int* __restrict__ err,
                                  const PartialLayout L) {
  __shared__ PartialTable tab;
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0, TRACE_ROPE);
  if (L.ws != nullptr) build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = R >> 1;
  T* row = qkv + (size_t)t * ld;
  // The row's head slots (Hq query heads, Hkv key heads, Hkv value heads) are shared out
  // between the gridDim.y blocks of this token.
  const int slots = Hq + 2 * Hkv;
  const int per_block = (slots + gridDim.y - 1) / gridDim.y;
  const int s_lo = blockIdx.y * per_block, s_hi = min(slots, s_lo + per_block);
  if (s_lo >= s_hi) return;
  if (L.ws != nullptr) {
    // the q, k, v product is still in partials: sum this block's part of the row first
    // (rounded to the storage type, as the product's own epilogue would have done)
    const int e_hi = min(s_hi, write_kv ? slots : Hq) * D;
#pragma unroll 2
    for (int i = s_lo * D + threadIdx.x; i < e_hi; i += blockDim.x) row[i] = from_f32<T>(partial_sum(L, tab, t, i));
    __syncthreads();
  }
  const bool pos_ok = pos >= 0 && (half == 0 || pos < n_pos);
  if (!pos_ok) {
    if (threadIdx.x == 0) atomicExch(err, 2);
    return;
  }
  const float* cs = cos_sin + (size_t)pos * half * 2;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_kv) {
    const int lp = pos / page_size;
    if (lp >= table_width) {
      if (threadIdx.x == 0) atomicExch(err, 3);
      return;
    }
    const int page = block_table[(size_t)req_of_token[t] * table_width + lp];
    if (page < 0) {
      if (threadIdx.x == 0) atomicExch(err, 4);
      return;
    }
    kdst = kv_plane + (size_t)page * page_stride + (size_t)(pos % page_size) * D;
    vdst = kdst + (size_t)Hkv * page_size * D;
  }
  const int hd2 = D >> 1;  // work items per head: D/2 "pairs" (rotated below `half`, copied above)
  // query and key heads of this block
  const int qk_hi = min(s_hi, Hq + Hkv);
  for (int w = s_lo * hd2 + threadIdx.x; w < qk_hi * hd2; w += blockDim.x) {
    const int h = w / hd2, i = w % hd2;
    T* src = row + (size_t)h * D;
    int ia, ib;
    float a, b;
    if (i < half) {
      ia = pairing == 0 ? 2 * i : i;
      ib = pairing == 0 ? 2 * i + 1 : i + half;
      const float x0 = to_f32<T>(src[ia]), x1 = to_f32<T>(src[ib]);
      const float c = cs[2 * i], s = cs[2 * i + 1];
      a = x0 * c - x1 * s;
      b = x0 * s + x1 * c;
    } else {  // the unrotated tail, two elements per item
      ia = R + 2 * (i - half);
      ib = ia + 1;
      a = to_f32<T>(src[ia]);
      b = to_f32<T>(src[ib]);
    }
    if (h < Hq) {
      if (i < half) {
        src[ia] = from_f32<T>(a);
        src[ib] = from_f32<T>(b);
      }
    } else if (write_kv) {
      T* dst = kdst + (size_t)(h - Hq) * page_size * D;
      dst[ia] = from_f32<T>(a);
      dst[ib] = from_f32<T>(b);
    }
  }
  // value heads of this block
  if (write_kv) {
    const int v_lo = max(s_lo, Hq + Hkv) - (Hq + Hkv), v_hi = s_hi - (Hq + Hkv);
    const T* v = row + (size_t)(Hq + Hkv) * D;
    for (int w = v_lo * D + threadIdx.x; w < v_hi * D; w += blockDim.x) {
      const int h = w / D, d = w % D;
      vdst[(size_t)h * page_size * D + d] = v[w];
    }
  }
  TRACE_MARK(TRACE_EXIT);
}

// Many tokens, a 16-bit type, the whole head rotated (R == D, D a multiple of 16): a thread rotates
// eight pairs with 16-byte loads and stores, or copies eight value elements.  Same formulas and
// the same error codes as the kernel above.
template <typename T>
__global__ void __launch_bounds__(128)
rope_cache_vec_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                      const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_width,
                      const float* __restrict__ cos_sin, int n_pos, T* __restrict__ kv_plane,
                      long long page_stride, int page_size, int Hq, int Hkv, int D, int pairing, int write_kv,
                      int n_tokens, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int chunks = D >> 4;                         // rotation items per head
  const int rot_items = (Hq + Hkv) * chunks;
  const int per_token = rot_items + (write_kv ? Hkv * (D >> 3) : 0);
  const int t = blockIdx.y, item = blockIdx.x * blockDim.x + threadIdx.x;   // the grid is (items, tokens)
  if (item >= per_token) return;
  const int pos = positions[t];
  const int half = D >> 1;
  if (pos < 0 || pos >= n_pos) {
    if (item == 0) atomicExch(err, 2);
    return;
  }
  T* row = qkv + (size_t)t * ld;
  T* kdst = nullptr;
  if (write_kv) {
    const int lp = pos / page_size;
    if (lp >= table_width) {
      if (item == 0) atomicExch(err, 3);
      return;
    }
    const int page = block_table[(size_t)req_of_token[t] * table_width + lp];
    if (page < 0) {
      if (item == 0) atomicExch(err, 4);
      return;
    }
    kdst = kv_plane + (size_t)page * page_stride + (size_t)(pos % page_size) * D;
  }
  if (item >= rot_items) {  // a value chunk
    const int w = item - rot_items, h = w / (D >> 3), c = w % (D >> 3);
    const uint4 v = *reinterpret_cast<const uint4*>(row + (size_t)(Hq + Hkv + h) * D + c * 8);
    *reinterpret_cast<uint4*>(kdst + (size_t)(Hkv + h) * page_size * D + c * 8) = v;
    return;
  }
  const int h = item / chunks, c = item % chunks;
  if (h >= Hq && !write_kv) return;
  T* src = row + (size_t)h * D;
  const int o0 = pairing == 0 ? c * 16 : c * 8, o1 = pairing == 0 ? c * 16 + 8 : half + c * 8;
  uint4 r0 = *reinterpret_cast<const uint4*>(src + o0), r1 = *reinterpret_cast<const uint4*>(src + o1);
  const T* e0 = reinterpret_cast<const T*>(&r0);
  const T* e1 = reinterpret_cast<const T*>(&r1);
  const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + ((size_t)pos * half + c * 8) * 2);
  uint4 w0, w1;
  T* f0 = reinterpret_cast<T*>(&w0);
  T* f1 = reinterpret_cast<T*>(&w1);
#pragma unroll
  for (int k = 0; k < 4; ++k) {  // pairs 2k and 2k+1 of this chunk
    const float4 cs = cs4[k];  // cos, sin, cos, sin
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int i = 2 * k + q;
      const float cv = q == 0 ? cs.x : cs.z, sv = q == 0 ? cs.y : cs.w;
      float x0, x1;
      if (pairing == 0) {  // elements 2i and 2i+1 of the 16 loaded
        x0 = to_f32<T>(i < 4 ? e0[2 * i] : e1[2 * i - 8]);
        x1 = to_f32<T>(i < 4 ? e0[2 * i + 1] : e1[2 * i - 7]);
      } else {
        x0 = to_f32<T>(e0[i]);
        x1 = to_f32<T>(e1[i]);
      }
      const T a = from_f32<T>(x0 * cv - x1 * sv), b = from_f32<T>(x0 * sv + x1 * cv);
      if (pairing == 0) {
        if (i < 4) {
          f0[2 * i] = a;
          f0[2 * i + 1] = b;
        } else {
          f1[2 * i - 8] = a;
          f1[2 * i - 7] = b;
        }
      } else {
        f0[i] = a;
        f1[i] = b;
      }
    }
  }
  T* dst = h < Hq ? src : kdst + (size_t)(h - Hq) * page_size * D;
  *reinterpret_cast<uint4*>(dst + o0) = w0;
  *reinterpret_cast<uint4*>(dst + o1) = w1;
}

FERRUM_API int ferrum_rope_cache_write(void* qkv, int dtype, int n_tokens, int ld, const int* positions,
                                       const int* req_of_token, const int* block_table, int table_width,
                                       const float* cos_sin, int n_pos, void* kv_plane, long long page_stride,
                                       int page_size, int Hq, int Hkv, int D, int R, int pairing, int write_kv,
                                       int* err_flag, const float* partials, const int* layout, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && Hq > 0 && Hkv > 0 && D > 0 && D % 2 == 0, "rope: bad sizes T=%d Hq=%d Hkv=%d D=%d",
                   n_tokens, Hq, Hkv, D);
  FERRUM_CHECK_ARG(R >= 0 && R % 2 == 0 && R <= D, "rope: rope_dim %d must be even and at most head_dim %d", R, D);
  FERRUM_CHECK_ARG(ld >= (Hq + 2 * Hkv) * D, "rope: row stride %d shorter than (Hq+2Hkv)*D", ld);
  FERRUM_CHECK_ARG(pairing == 0 || pairing == 1, "rope: pairing code %d", pairing);
  FERRUM_CHECK_ARG(!write_kv || (page_size > 0 && table_width > 0 && kv_plane), "rope: cache arguments missing");
  if (n_tokens == 0) return 0;
  PartialLayout L{nullptr, 0, 0, 0, 0};
  if (partials != nullptr) {
    if (int r = make_layout(partials, layout, &L)) return r;
    FERRUM_CHECK_ARG((write_kv ? Hq + 2 * Hkv : Hq) * D <= L.tiles * 128 && n_tokens <= L.acc_cols,
                     "rope: the partials do not cover the rows");
  }
  if (ferrum_is_16bit(dtype) && n_tokens > 64 && n_tokens <= 65535 && partials == nullptr && R == D && D % 16 == 0 && ld % 8 == 0 &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)cos_sin & 15) == 0 &&
      (!write_kv || (((uintptr_t)kv_plane & 15) == 0 && page_stride % 8 == 0))) {
    const int per_token = (Hq + Hkv) * (D / 16) + (write_kv ? Hkv * (D / 8) : 0);
    FERRUM_DISPATCH_16BIT(dtype, T, launch_kernel(rope_cache_vec_kernel<T>, dim3((per_token + 127) / 128, n_tokens), dim3(128), 0, stream,
                                                  (T*)qkv, ld, positions, req_of_token, block_table, table_width, cos_sin, n_pos,
                                                  (T*)kv_plane, page_stride, page_size, Hq, Hkv, D, pairing, write_kv, n_tokens, err_flag));
    FERRUM_CHECK_LAUNCH("rope_cache_write");
    return 0;
  }
  const int threads = 256;
  // few tokens, or a product still in partials (several loads per element): several blocks per
  // token, four head slots each, so that a row is read by many SMs at once
  const dim3 grid(n_tokens, (n_tokens <= 64 || partials != nullptr) ? (Hq + 2 * Hkv + 3) / 4 : 1);
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(rope_cache_kernel<T>, grid, threads, 0, stream, (T*)qkv, ld, positions, req_of_token,
                                                block_table, table_width, cos_sin, n_pos, (T*)kv_plane, page_stride, page_size, Hq,
                                                Hkv, D, R, pairing, write_kv, err_flag, L));
  FERRUM_CHECK_LAUNCH("rope_cache_write");
  return 0;
}

// ---------------------------------------------------------------- SwiGLU
// act[t, f] = silu(gu[t, f]) * gu[t, F + f], silu(g) = g / (1 + exp(-g)), in float32.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int F, int ld_in, int ld_out) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.y;
  const T* g = gu + (size_t)t * ld_in;
  const T* u = g + F;
  T* o = act + (size_t)t * ld_out;
  for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x) {
    const float gv = to_f32<T>(g[f]);
    o[f] = from_f32<T>(gv / (1.0f + expf(-gv)) * to_f32<T>(u[f]));
  }
}

// 16-bit rows of 16-byte multiples: 16-byte loads and stores, SWIGLU_VEC groups of eight features
// per thread with all their loads issued before the arithmetic.
constexpr int SWIGLU_VEC = 4;
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int F, int ld_in, int ld_out) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.y;
  const int groups = F >> 3;
  const int i0 = blockIdx.x * (blockDim.x * SWIGLU_VEC) + threadIdx.x;  // this thread's groups: i0 + k * blockDim.x
  const T* row = gu + (size_t)t * ld_in;
  uint4 g[SWIGLU_VEC], u[SWIGLU_VEC];
#pragma unroll
  for (int k = 0; k < SWIGLU_VEC; ++k) {
    const int i = i0 + k * blockDim.x;
    if (i < groups) {
      g[k] = *reinterpret_cast<const uint4*>(row + i * 8);
      u[k] = *reinterpret_cast<const uint4*>(row + F + i * 8);
    }
  }
#pragma unroll
  for (int k = 0; k < SWIGLU_VEC; ++k) {
    const int i = i0 + k * blockDim.x;
    if (i >= groups) continue;
    const T* ge = reinterpret_cast<const T*>(&g[k]);
    const T* ue = reinterpret_cast<const T*>(&u[k]);
    uint4 o;
    uint32_t* o2 = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gx = to_f32<T>(ge[2 * j]), gy = to_f32<T>(ge[2 * j + 1]), ux = to_f32<T>(ue[2 * j]), uy = to_f32<T>(ue[2 * j + 1]);
      // fast exponential and division, as in the products' own SwiGLU epilogues: the result is
      // rounded to 16 bits, and the arithmetic, not the memory, set this kernel's time
      o2[j] = pack2<T>(__fdividef(gx, 1.0f + __expf(-gx)) * ux, __fdividef(gy, 1.0f + __expf(-gy)) * uy);
    }
    *reinterpret_cast<uint4*>(act + (size_t)t * ld_out + i * 8) = o;
  }
}

// act[t, f] = silu(gate) * up where gate and up are still partials of a two-product launch
// (columns t and acc_cols / 2 + t of the partial tiles).
template <typename T>
__global__ void swiglu_reduce_kernel(T* __restrict__ act, int F, int ld_out, const PartialLayout L) {
  __shared__ PartialTable tab;
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0, TRACE_SWIGLU_REDUCE);
  build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  const int t = blockIdx.y;
  T* o = act + (size_t)t * ld_out;
  for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x) {
    const float g = partial_sum(L, tab, t, f), u = partial_sum(L, tab, L.acc_cols / 2 + t, f);
    o[f] = from_f32<T>(g / (1.0f + __expf(-g)) * u);
  }
  TRACE_MARK(TRACE_EXIT);
}

// The same for many tokens: a thread owns four neighbouring features (one 16-byte piece of a
// partial's column: they share a tile and so their contributors) and walks SWIGLU_REDUCE_TOKENS
// tokens with the slot addresses it worked out once.  One load and one table lookup per
// feature and token made this kernel, not memory, the limit at 64 tokens.
constexpr int SWIGLU_REDUCE_TOKENS = 2;
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_reduce_vec_kernel(T* __restrict__ act, int n_tokens, int F, int ld_out, const PartialLayout L) {
  __shared__ PartialTable tab;
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1, TRACE_SWIGLU_REDUCE);
  build_partial_table(L, tab);
  pdl_launch();
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  const int f = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (f >= F) return;
  const int tile = f >> 7, nl = f & 127;
  const int fc = tab.first_and_count[tile];
  const int c_first = fc & 0xFFFF, count = fc >> 16;
  const unsigned bits = tab.slot_bits[tile];
  const size_t slot_floats = (size_t)L.acc_cols * 128;
  const float* base[PARTIAL_MAX_CONTRIB];
#pragma unroll
  for (int s = 0; s < PARTIAL_MAX_CONTRIB; ++s)
    base[s] = L.ws + (size_t)((c_first + (s < count ? s : 0)) * 2 + ((bits >> (s < count ? s : 0)) & 1)) * slot_floats + nl;
  const int t0 = blockIdx.y * SWIGLU_REDUCE_TOKENS;
  const int up_col = L.acc_cols / 2;
#pragma unroll
  for (int t = t0; t < t0 + SWIGLU_REDUCE_TOKENS; ++t) {  // unrolled: the tokens' loads are in flight together
    if (t >= n_tokens) break;
    float4 g[PARTIAL_MAX_CONTRIB], u[PARTIAL_MAX_CONTRIB];
#pragma unroll
    for (int s = 0; s < PARTIAL_MAX_CONTRIB; ++s) {  // all loads first, then the sums in contributor (K) order
      const bool have = s < count;
      g[s] = have ? __ldcg(reinterpret_cast<const float4*>(base[s] + (size_t)t * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
      u[s] = have ? __ldcg(reinterpret_cast<const float4*>(base[s] + (size_t)(up_col + t) * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 gs = make_float4(0.f, 0.f, 0.f, 0.f), us = gs;
#pragma unroll
    for (int s = 0; s < PARTIAL_MAX_CONTRIB; ++s) {
      gs.x += g[s].x; gs.y += g[s].y; gs.z += g[s].z; gs.w += g[s].w;
      us.x += u[s].x; us.y += u[s].y; us.z += u[s].z; us.w += u[s].w;
    }
    uint2 pk;
    pk.x = pack2<T>(gs.x / (1.0f + __expf(-gs.x)) * us.x, gs.y / (1.0f + __expf(-gs.y)) * us.y);
    pk.y = pack2<T>(gs.z / (1.0f + __expf(-gs.z)) * us.z, gs.w / (1.0f + __expf(-gs.w)) * us.w);
    *reinterpret_cast<uint2*>(act + (size_t)t * ld_out + f) = pk;
  }
  TRACE_MARK(TRACE_EXIT);
}

FERRUM_API int ferrum_swiglu_reduce(void* act, int dtype, int n_tokens, int F, int ld_out, const float* partials, const int* layout,
                                    cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && F > 0 && ld_out >= F, "swiglu_reduce: bad sizes");
  if (n_tokens == 0) return 0;
  PartialLayout L;
  if (int r = make_layout(partials, layout, &L)) return r;
  FERRUM_CHECK_ARG(F <= L.tiles * 128 && n_tokens <= L.acc_cols / 2, "swiglu_reduce: the partials do not cover the rows");
  if (n_tokens > 16 && F % 4 == 0 && ld_out % 4 == 0 && ((uintptr_t)act & 7) == 0) {
    dim3 vgrid((F / 4 + 255) / 256, (n_tokens + SWIGLU_REDUCE_TOKENS - 1) / SWIGLU_REDUCE_TOKENS);
    FERRUM_DISPATCH_16BIT(dtype, T, launch_kernel(swiglu_reduce_vec_kernel<T>, vgrid, dim3(256), 0, stream, (T*)act, n_tokens, F, ld_out, L));
    FERRUM_CHECK_LAUNCH("swiglu_reduce");
    return 0;
  }
  dim3 grid((F + 255) / 256 > 32 ? 32 : (F + 255) / 256, n_tokens);
  FERRUM_DISPATCH_16BIT(dtype, T, launch_kernel(swiglu_reduce_kernel<T>, grid, dim3(256), 0, stream, (T*)act, F, ld_out, L));
  FERRUM_CHECK_LAUNCH("swiglu_reduce");
  return 0;
}

FERRUM_API int ferrum_swiglu(const void* gu, void* act, int dtype, int n_tokens, int F, int ld_in, int ld_out,
                             cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && F > 0 && ld_in >= 2 * F && ld_out >= F, "swiglu: bad sizes T=%d F=%d", n_tokens, F);
  if (n_tokens == 0) return 0;
  FERRUM_CHECK_ARG(n_tokens <= 65535, "swiglu: more than 65535 tokens in one call");
  if (ferrum_is_16bit(dtype) && F % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && ((uintptr_t)gu & 15) == 0 &&
      ((uintptr_t)act & 15) == 0) {
    dim3 vgrid((F / 8 + 256 * SWIGLU_VEC - 1) / (256 * SWIGLU_VEC), n_tokens);
    FERRUM_DISPATCH_16BIT(dtype, T, launch_kernel(swiglu_vec_kernel<T>, vgrid, dim3(256), 0, stream, (const T*)gu, (T*)act, F, ld_in, ld_out));
    FERRUM_CHECK_LAUNCH("swiglu");
    return 0;
  }
  dim3 grid((F + 255) / 256 > 64 ? 64 : (F + 255) / 256, n_tokens);
  FERRUM_DISPATCH_DTYPE(dtype, T, launch_kernel(swiglu_kernel<T>, grid, 256, 0, stream, (const T*)gu, (T*)act, F, ld_in, ld_out));
  FERRUM_CHECK_LAUNCH("swiglu");
  return 0;
}

FERRUM_TRACE_READER(ferrum_trace_elementwise)
