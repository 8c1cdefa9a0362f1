// Causal grouped-query attention over the paged cache on the CUDA cores, any head size up to
// 256, float32 arithmetic throughout: the float32 attention of the engine, and the 16-bit
// attention for head sizes the tensor-core kernels do not take.
//
// The same code runs a prompt portion and a decoded token: a row is one token and up to four
// query heads of one KV head, and reads keys lo..pos from the cache (the rotary kernel has
// already stored this step's keys).  A CTA of four warps handles a row, or one 128-key split of
// it.  A warp takes every fourth key of the CTA's range; its 32 lanes read one key row
// together (lane i reads elements i, i + 32, ... : whole 128-byte lines), so a K/V row read
// once serves the row's heads.  Per head the warp keeps an online softmax (max, sum and the
// weighted values) in float32 with expf; the four warps are then merged in warp order.
//
// Two ways to hand out the work, chosen by the number of rows alone.  Many rows (a prompt
// portion): one CTA per row walks its whole key range and writes the output.  Few rows
// (decoding): one CTA per row and 128-key split writes (max, sum, values) partials and a second
// kernel folds the splits in ascending order.  The split borders are multiples of 128 in
// absolute key positions: a function of the position alone, never of the batch.
// Formulas: query head h reads KV head h / (Hq/Hkv), score = q.k / sqrt(D), stable softmax,
// weighted sum of V (crates/model/src/llama.rs:220-247; crates/kernels/src/scalar.rs:125-141).
// `window` > 0 keeps keys in (pos-window, pos].
#include "common.cuh"

constexpr int AG_WARPS = 4;
constexpr int AG_HEADS = 4;      // query heads of one KV head that share a CTA's key reads
constexpr int AG_SPLIT = 128;    // keys per split (absolute positions s * 128 .. s * 128 + 127)
constexpr int AG_MAX_D = 256;
constexpr int AG_DI = AG_MAX_D / 32;
constexpr int AG_KEYS = 4;       // keys a warp fetches together

// (m, l, o) of b folded into a: the softmax of the union of two key sets.
__device__ __forceinline__ void ag_fold(float& m, float& l, float& o, float mb, float lb, float ob) {
  const float m_new = fmaxf(m, mb);
  const float fa = m == -INFINITY ? 0.f : expf(m - m_new);
  const float fb = mb == -INFINITY ? 0.f : expf(mb - m_new);
  l = l * fa + lb * fb;
  o = o * fa + ob * fb;
  m = m_new;
}

// part: null (the CTA covers the row's whole key range and writes `out`), or the partials
// [token][head][split slot][D + 2] of the split that blockIdx.y names.
template <typename T, int DI>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                         const int* __restrict__ positions, const int* __restrict__ req_of_token,
                         const int* __restrict__ block_table, int table_width, const T* __restrict__ kv_plane,
                         long long page_stride, int page_size, int Hq, int Hkv, int D, float scale, int window,
                         int* __restrict__ err, float* __restrict__ part, int split_slots) {
  __shared__ float sm_ml[AG_WARPS][AG_HEADS][2];
  __shared__ float sm_o[AG_WARPS][AG_HEADS][DI * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int chunks = (G + AG_HEADS - 1) / AG_HEADS;
  const int t = blockIdx.x / (Hkv * chunks);
  const int kvh = (blockIdx.x / chunks) % Hkv;
  const int chunk = blockIdx.x % chunks;
  const int h0 = kvh * G + chunk * AG_HEADS;
  const int nh = min(AG_HEADS, G - chunk * AG_HEADS);
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  int k_begin = lo, k_end = pos + 1;
  if (part != nullptr) {
    const int s = lo / AG_SPLIT + blockIdx.y;
    if (s * AG_SPLIT > pos) return;            // this row has fewer splits
    k_begin = max(lo, s * AG_SPLIT);
    k_end = min(pos + 1, (s + 1) * AG_SPLIT);
  }
  const int* bt = block_table + (size_t)req_of_token[t] * table_width;

  float qr[AG_HEADS][DI];
#pragma unroll
  for (int g = 0; g < AG_HEADS; ++g)
#pragma unroll
    for (int i = 0; i < DI; ++i) {
      const int d = lane + 32 * i;
      qr[g][i] = (g < nh && d < D) ? to_f32<T>(q[(size_t)t * ldq + (size_t)(h0 + g) * D + d]) : 0.f;
    }
  float m[AG_HEADS], l[AG_HEADS], acc[AG_HEADS][DI];
#pragma unroll
  for (int g = 0; g < AG_HEADS; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DI; ++i) acc[g][i] = 0.f;
  }
  const size_t v_off = (size_t)Hkv * page_size * D;
  // This warp's keys: every fourth key of the range, counted in absolute positions.  AG_KEYS keys
  // are fetched together (their loads are in flight at once: a warp that handled one key at a
  // time was a chain of memory latencies) and then folded into the softmax one after the other.
  int key0 = k_begin + ((warp - k_begin) & (AG_WARPS - 1));
  for (; key0 < k_end; key0 += AG_WARPS * AG_KEYS) {
    float kd[AG_KEYS][DI], vd[AG_KEYS][DI];
    bool have[AG_KEYS];
#pragma unroll
    for (int j = 0; j < AG_KEYS; ++j) {
      const int key = key0 + j * AG_WARPS;
      const int lp = key / page_size;
      const int page = (key < k_end && lp < table_width) ? bt[lp] : -1;
      have[j] = page >= 0;
      if (key < k_end && page < 0 && lane == 0) atomicExch(err, 5);
      const T* kr = kv_plane + (size_t)max(page, 0) * page_stride + ((size_t)kvh * page_size + key % page_size) * D;
      const T* vr = kr + v_off;
#pragma unroll
      for (int i = 0; i < DI; ++i) {
        const int d = lane + 32 * i;
        kd[j][i] = (have[j] && d < D) ? to_f32<T>(kr[d]) : 0.f;
        vd[j][i] = (have[j] && d < D) ? to_f32<T>(vr[d]) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < AG_KEYS; ++j) {
      if (!have[j]) continue;          // (uniform over the warp)
#pragma unroll
      for (int g = 0; g < AG_HEADS; ++g) {
        if (g >= nh) break;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < DI; ++i) dot = fmaf(qr[g][i], kd[j][i], dot);
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m[g], s);
        const float corr = m[g] == -INFINITY ? 0.f : expf(m[g] - m_new);
        const float p = expf(s - m_new);
        l[g] = l[g] * corr + p;
#pragma unroll
        for (int i = 0; i < DI; ++i) acc[g][i] = fmaf(p, vd[j][i], acc[g][i] * corr);
        m[g] = m_new;
      }
    }
  }
  // ---- the four warps meet in warp order
#pragma unroll
  for (int g = 0; g < AG_HEADS; ++g) {
    if (lane == 0) {
      sm_ml[warp][g][0] = m[g];
      sm_ml[warp][g][1] = l[g];
    }
#pragma unroll
    for (int i = 0; i < DI; ++i) sm_o[warp][g][lane + 32 * i] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nh * DI * 32; idx += AG_WARPS * 32) {
    const int g = idx / (DI * 32), d = idx % (DI * 32);
    if (d >= D) continue;
    float M = -INFINITY, L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < AG_WARPS; ++w) ag_fold(M, L, O, sm_ml[w][g][0], sm_ml[w][g][1], sm_o[w][g][d]);
    if (part == nullptr) {
      out[(size_t)t * ldo + (size_t)(h0 + g) * D + d] = from_f32<T>(L > 0.f ? O / L : 0.f);
    } else {
      float* p = part + (((size_t)t * Hq + h0 + g) * split_slots + blockIdx.y) * (D + 2);
      p[2 + d] = O;
      if (d == 0) {
        p[0] = M;
        p[1] = L;
      }
    }
  }
}

// Folds the splits of every (token, head) in ascending key order: one warp each.
template <typename T>
__global__ void __launch_bounds__(32)
attention_generic_combine_kernel(T* __restrict__ out, int ldo, const float* __restrict__ part, const int* __restrict__ positions,
                                 int Hq, int D, int window, int split_slots) {
  const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos / AG_SPLIT - lo / AG_SPLIT + 1;
  const float* base = part + ((size_t)t * Hq + h) * split_slots * (D + 2);
  float M = -INFINITY, L = 0.f, O[AG_DI];
#pragma unroll
  for (int i = 0; i < AG_DI; ++i) O[i] = 0.f;
  const int total = min(n, split_slots);
  for (int s0 = 0; s0 < total; s0 += 4) {     // four splits' loads in flight, folded one after the other
    float mb[4], lb[4], ob[4][AG_DI];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool have = s0 + j < total;
      const float* p = base + (size_t)(have ? s0 + j : 0) * (D + 2);
      mb[j] = have ? p[0] : -INFINITY;
      lb[j] = have ? p[1] : 0.f;
#pragma unroll
      for (int i = 0; i < AG_DI; ++i) {
        const int d = lane + 32 * i;
        ob[j][i] = (have && d < D) ? p[2 + d] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (s0 + j >= total) break;
      const float m_new = fmaxf(M, mb[j]);
      const float fa = M == -INFINITY ? 0.f : expf(M - m_new);
      const float fb = mb[j] == -INFINITY ? 0.f : expf(mb[j] - m_new);
      L = L * fa + lb[j] * fb;
#pragma unroll
      for (int i = 0; i < AG_DI; ++i) O[i] = O[i] * fa + ob[j][i] * fb;
      M = m_new;
    }
  }
#pragma unroll
  for (int i = 0; i < AG_DI; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out[(size_t)t * ldo + (size_t)h * D + d] = from_f32<T>(L > 0.f ? O[i] / L : 0.f);
  }
}

// Keys per split, for the caller that sizes the partials: `split_slots` splits per (token, head),
// D + 2 floats each.
FERRUM_API int ferrum_attention_generic_split() { return AG_SPLIT; }

// part == null: one CTA per row walks the row's whole key range (for batches of many tokens).
// Otherwise `part` holds n_tokens * Hq * split_slots * (D + 2) floats, every row's key range is
// cut at multiples of 128 keys among split_slots CTAs (split_slots must cover the longest row),
// and a second launch folds the partials into `out`.
FERRUM_API int ferrum_attention_generic(const void* q, int ldq, void* out, int ldo, int dtype, int n_tokens,
                                        const int* positions, const int* req_of_token, const int* block_table,
                                        int table_width, const void* kv_plane, long long page_stride, int page_size,
                                        int Hq, int Hkv, int D, float scale, int window, int* err_flag, float* part,
                                        int split_slots, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
  FERRUM_CHECK_ARG(D > 0 && D <= AG_MAX_D, "attention: head size %d is outside (0, %d]", D, AG_MAX_D);
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0, "attention: bad cache arguments");
  FERRUM_CHECK_ARG(ldq >= Hq * D && ldo >= Hq * D, "attention: a row stride is shorter than Hq*D");
  FERRUM_CHECK_ARG(part == nullptr || (split_slots > 0 && split_slots <= 65535), "attention: bad number of split slots %d", split_slots);
  if (n_tokens == 0) return 0;
  const int G = Hq / Hkv;
  const long long rows = (long long)n_tokens * Hkv * ((G + AG_HEADS - 1) / AG_HEADS);
  FERRUM_CHECK_ARG(rows < (1LL << 31), "attention: too many rows");
  const dim3 grid((unsigned)rows, part ? split_slots : 1);
#define AG_LAUNCH(DI_)                                                                                                  \
  FERRUM_DISPATCH_DTYPE(dtype, T, (attention_generic_kernel<T, DI_><<<grid, AG_WARPS * 32, 0, stream>>>(              \
      (const T*)q, ldq, (T*)out, ldo, positions, req_of_token, block_table, table_width, (const T*)kv_plane, page_stride, \
      page_size, Hq, Hkv, D, scale, window, err_flag, part, split_slots)))
  if (D <= 32) AG_LAUNCH(1);
  else if (D <= 64) AG_LAUNCH(2);
  else if (D <= 128) AG_LAUNCH(4);
  else AG_LAUNCH(8);
#undef AG_LAUNCH
  FERRUM_CHECK_LAUNCH("attention_generic");
  if (part != nullptr) {
    const dim3 cgrid(n_tokens, Hq);
    FERRUM_CHECK_ARG(cgrid.y <= 65535, "attention: too many heads");
    FERRUM_DISPATCH_DTYPE(dtype, T, (attention_generic_combine_kernel<T><<<cgrid, 32, 0, stream>>>(
        (T*)out, ldo, part, positions, Hq, D, window, split_slots)));
    FERRUM_CHECK_LAUNCH("attention_generic_combine");
  }
  return 0;
}
