// Causal grouped-query attention over the paged cache on the CUDA cores, any head size up to
// 256, float32 arithmetic throughout: the float32 attention of the engine, and the 16-bit
// attention for head sizes the tensor-core kernels do not take.
//
// The same code runs a prompt portion and a decoded token: a row is one token and up to four
// query heads of one KV head, and reads keys lo..pos from the cache (the rotary kernel has
// already stored this step's keys).  A CTA of four warps handles a row, or one 128-key split of
// it, in tiles of 32 keys (16 for head sizes above 128): the four warps bring the tile's key and
// value rows into shared memory together (16-byte loads where the rows allow, converted to
// float32), then warp g works for head g alone: lane j forms the score of key j from shared
// memory (no reduction across lanes: a lane walks the head size in order), the warp takes the
// tile's maximum and sum by shuffles, leaves the weights in shared memory, and lane i adds the
// weighted values of elements i, i + 32, ... in key order.  Max, sum and the weighted values stay
// in float32 registers with expf.  (Before, a warp read one key row together and reduced every
// score across its lanes: some 90 instructions per key and head against about 15 here.)
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
constexpr int AG_HEADS = 4;      // query heads of one KV head that share a CTA's key reads: one warp each
constexpr int AG_SPLIT = 128;    // keys per split (absolute positions s * 128 .. s * 128 + 127)
constexpr int AG_MAX_D = 256;
constexpr int AG_DI = AG_MAX_D / 32;
static_assert(AG_HEADS == AG_WARPS, "warp g works for head g");

// Shared memory of a CTA for head sizes up to 32 * DI, two tiles deep: keys [2][TK][32 DI + 4]
// (the 4 floats of padding make a quarter warp's 16-byte reads of one column of eight rows hit
// different banks), values [2][TK][32 DI], queries [4][32 DI], weights [4][TK], row offsets
// [2][TK]; keys, values and queries are zero past the head size.
template <int DI>
struct AgTile {
  static constexpr int TK = DI <= 4 ? 32 : 16;
  static constexpr int DP = 32 * DI;
  static constexpr int KS = DP + 4;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + 2 * TK * KS;
  static constexpr int OFF_Q = OFF_V + 2 * TK * DP;
  static constexpr int OFF_P = OFF_Q + AG_HEADS * DP;
  static constexpr int OFF_ROW = OFF_P + AG_HEADS * TK;       // (an even number of floats: the offsets are 8-byte aligned)
  static constexpr int SMEM_BYTES = (OFF_ROW + 2 * TK * 2) * 4;
};

__device__ __forceinline__ void ag_cp_async16(void* smem, const void* gmem, int src_bytes) {   // src_bytes 0: sixteen zero bytes
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ag_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ag_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Four consecutive elements of a cache or query row as float32: one 16-byte (float) or 8-byte
// (16-bit types) load where `vec` says the rows are aligned for it, else element by element
// with a bound.
template <typename T>
__device__ __forceinline__ float4 ag_load4(const T* row, int d, int D, bool vec) {
  float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) {
    if (d < D) {   // (D is a multiple of 4 here)
      if constexpr (sizeof(T) == 4) {
        r = *reinterpret_cast<const float4*>(row + d);
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(row + d);
        const T* e = reinterpret_cast<const T*>(&u);
        r = make_float4(to_f32<T>(e[0]), to_f32<T>(e[1]), to_f32<T>(e[2]), to_f32<T>(e[3]));
      }
    }
  } else {
    if (d < D) r.x = to_f32<T>(row[d]);
    if (d + 1 < D) r.y = to_f32<T>(row[d + 1]);
    if (d + 2 < D) r.z = to_f32<T>(row[d + 2]);
    if (d + 3 < D) r.w = to_f32<T>(row[d + 3]);
  }
  return r;
}

// part: null (the CTA covers the row's whole key range and writes `out`), or the partials
// [token][head][split slot][D + 2] of the split that blockIdx.y names.
// The tile after the one being worked on is on its way meanwhile: float32 rows that are 16-byte
// aligned go from the cache to shared memory by cp.async (nothing passes through registers,
// absent rows arrive as zeros); other rows are loaded and converted by the threads.
template <typename T, int DI>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                         const int* __restrict__ positions, const int* __restrict__ req_of_token,
                         const int* __restrict__ block_table, int table_width, const T* __restrict__ kv_plane,
                         long long page_stride, int page_size, int Hq, int Hkv, int D, float scale, int window,
                         int* __restrict__ err, float* __restrict__ part, int split_slots, int vec) {
  using Tile = AgTile<DI>;
  constexpr int TK = Tile::TK, DP = Tile::DP, KS = Tile::KS;
  extern __shared__ __align__(16) float ag_smem[];
  float* const sm_k = ag_smem + Tile::OFF_K;
  float* const sm_v = ag_smem + Tile::OFF_V;
  float* const sm_q = ag_smem + Tile::OFF_Q;
  float* const sm_p = ag_smem + Tile::OFF_P;
  long long* const sm_row = reinterpret_cast<long long*>(ag_smem + Tile::OFF_ROW);   // [2][TK]: element offset of a key's row; -1: no such key
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
  const size_t v_off = (size_t)Hkv * page_size * D;
  const bool vec_ok = vec != 0;
  const bool async_rows = vec_ok && sizeof(T) == 4;
  const int n_tiles = (k_end - k_begin + TK - 1) / TK;

  // where the rows of tile n lie (threads 0 .. TK-1)
  auto find_rows = [&](int n) {
    if (threadIdx.x < TK) {
      const int key = k_begin + n * TK + threadIdx.x;
      long long off = -1;
      if (key < k_end) {
        const int lp = key / page_size;
        const int page = lp < table_width ? bt[lp] : -1;
        if (page < 0) atomicExch(err, 5);      // a key of the row's range without a page: read as absent, and the step fails
        else off = (long long)page * page_stride + ((long long)kvh * page_size + key % page_size) * D;
      }
      sm_row[(n & 1) * TK + threadIdx.x] = off;
    }
  };
  // tile n on its way into its buffer (the caller commits the group)
  auto load_tile = [&](int n) {
    const int b = n & 1;
    float* const kb = sm_k + b * TK * KS;
    float* const vb = sm_v + b * TK * DP;
    for (int idx = threadIdx.x; idx < TK * (DP / 4); idx += AG_WARPS * 32) {
      const int j = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
      const long long off = sm_row[b * TK + j];
      if (async_rows) {
        const bool there = off >= 0 && d < D;
        const T* src = kv_plane + (there ? off + d : 0);
        ag_cp_async16(&kb[j * KS + d], src, there ? 16 : 0);
        ag_cp_async16(&vb[j * DP + d], src + (there ? v_off : 0), there ? 16 : 0);
      } else {
        float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
        if (off >= 0) {
          kk = ag_load4<T>(kv_plane + off, d, D, vec_ok);
          vv = ag_load4<T>(kv_plane + off + v_off, d, D, vec_ok);
        }
        *reinterpret_cast<float4*>(&kb[j * KS + d]) = kk;
        *reinterpret_cast<float4*>(&vb[j * DP + d]) = vv;
      }
    }
  };

  // the row's queries, zero past the head size and for heads the chunk does not have
  for (int idx = threadIdx.x; idx < AG_HEADS * (DP / 4); idx += AG_WARPS * 32) {
    const int g = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (g < nh) v = ag_load4<T>(q + (size_t)t * ldq + (size_t)(h0 + g) * D, d, D, vec_ok && ldq % 4 == 0);
    *reinterpret_cast<float4*>(&sm_q[g * DP + d]) = v;
  }
  find_rows(0);
  __syncthreads();
  load_tile(0);
  ag_cp_async_commit();

  float m = -INFINITY, l = 0.f, acc[DI];      // of head `warp` (the same in all its lanes; acc: elements lane + 32 i)
#pragma unroll
  for (int i = 0; i < DI; ++i) acc[i] = 0.f;

  for (int n = 0; n < n_tiles; ++n) {
    const int b = n & 1;
    const bool more = n + 1 < n_tiles;
    if (more) find_rows(n + 1);                // (its buffer was last read for tile n - 1, before the barrier that ended it)
    __syncthreads();
    if (more) load_tile(n + 1);
    ag_cp_async_commit();
    ag_cp_async_wait<1>();                     // everything but the newest group: tile n is there
    const bool have = lane < TK && sm_row[b * TK + lane] >= 0;
    __syncthreads();
    if (warp < nh) {
      const float* const kb = sm_k + b * TK * KS;
      const float* const vb = sm_v + b * TK * DP;
      // ---- lane j: the score of key j for this warp's head, the head size walked in order
      float s = -INFINITY;
      if (have) {
        const float4* kr = reinterpret_cast<const float4*>(&kb[lane * KS]);
        const float4* qr = reinterpret_cast<const float4*>(&sm_q[warp * DP]);
        float dot = 0.f;
#pragma unroll 8
        for (int c = 0; c < DP / 4; ++c) {
          const float4 a = qr[c], k4 = kr[c];
          dot = fmaf(a.x, k4.x, dot);
          dot = fmaf(a.y, k4.y, dot);
          dot = fmaf(a.z, k4.z, dot);
          dot = fmaf(a.w, k4.w, dot);
        }
        s = dot * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));
      float corr = 1.f, pj = 0.f;
      if (m_new != -INFINITY) {                 // (else no key of the tile exists: nothing changes)
        corr = m == -INFINITY ? 0.f : expf(m - m_new);
        pj = s == -INFINITY ? 0.f : expf(s - m_new);
      }
      l = l * corr + warp_sum(pj);
      m = m_new;
      __syncwarp();                             // the weights of the tile before have been read
      if (lane < TK) sm_p[warp * TK + lane] = pj;
      __syncwarp();
      // ---- lane i: elements i, i + 32, ... of the weighted values, keys in ascending order
      float a[DI];
#pragma unroll
      for (int i = 0; i < DI; ++i) a[i] = acc[i] * corr;
      const float4* pr = reinterpret_cast<const float4*>(&sm_p[warp * TK]);
#pragma unroll 2
      for (int j4 = 0; j4 < TK / 4; ++j4) {
        const float4 pw = pr[j4];
        const float* vr = &vb[(j4 * 4) * DP + lane];
#pragma unroll
        for (int i = 0; i < DI; ++i) {
          a[i] = fmaf(pw.x, vr[32 * i], a[i]);
          a[i] = fmaf(pw.y, vr[DP + 32 * i], a[i]);
          a[i] = fmaf(pw.z, vr[2 * DP + 32 * i], a[i]);
          a[i] = fmaf(pw.w, vr[3 * DP + 32 * i], a[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < DI; ++i) acc[i] = a[i];
    }
  }
  ag_cp_async_wait<0>();
  if (warp >= nh) return;
  const int h = h0 + warp;
  if (part == nullptr) {
#pragma unroll
    for (int i = 0; i < DI; ++i) {
      const int d = lane + 32 * i;
      if (d < D) out[(size_t)t * ldo + (size_t)h * D + d] = from_f32<T>(l > 0.f ? acc[i] / l : 0.f);
    }
  } else {
    float* p = part + (((size_t)t * Hq + h) * split_slots + blockIdx.y) * (D + 2);
    if (lane == 0) {
      p[0] = m;
      p[1] = l;
    }
#pragma unroll
    for (int i = 0; i < DI; ++i) {
      const int d = lane + 32 * i;
      if (d < D) p[2 + d] = acc[i];
    }
  }
}

// ------------------------------------------------------------------ prompt portions: tiles of tokens
// With many tokens the kernel above reads every key row once per token.  Here a CTA takes up to
// AG_TQ consecutive tokens of ONE request (and up to four heads of one KV head): the tile of keys
// and values in shared memory serves all of them, the score loop reads a key element once for the
// AG_TQ queries of a head, and the value loop reads a value element once for AG_TQ weighted sums.
// A warp still works for one head alone; it keeps max, sum and the weighted values of four of the
// chunk's tokens (eight warps: four heads x two halves of the tokens).  The arithmetic of a row is the same as above (tiles of 32 keys from the first key that
// any of the CTA's rows sees), so a row's result depends on its chunk's first key only through
// where the tile borders fall: rounding.
// A CTA finds its chunk from q_start (tokens of request r are q_start[r] .. q_start[r+1]-1, in
// ascending positions): chunk c of the grid is the c-th chunk of AG_TQ tokens counted request by
// request; the grid has an upper bound of chunks and the CTAs past the last chunk leave.
constexpr int AG_TQ = 8;
constexpr int AG_TWARPS = 8;                 // warp w: head w % 4, tokens (w / 4) * 4 .. + 3 of the chunk
constexpr int AG_TH = AG_TQ / (AG_TWARPS / AG_HEADS);

template <int DI>
struct AgTokenTile {
  using Tile = AgTile<DI>;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + 2 * Tile::TK * Tile::KS;
  static constexpr int OFF_Q = OFF_V + 2 * Tile::TK * Tile::DP;                 // [AG_TQ][4][DP]
  static constexpr int OFF_P = OFF_Q + AG_TQ * AG_HEADS * Tile::DP;             // [4][AG_TQ][TK]
  static constexpr int OFF_ROW = OFF_P + AG_HEADS * AG_TQ * Tile::TK;
  static constexpr int SMEM_BYTES = (OFF_ROW + 2 * Tile::TK * 2) * 4;
};

template <typename T, int DI>
__global__ void __launch_bounds__(AG_TWARPS * 32)
attention_generic_tokens_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                                const int* __restrict__ positions, const int* __restrict__ q_start, int n_reqs,
                                const int* __restrict__ block_table, int table_width, const T* __restrict__ kv_plane,
                                long long page_stride, int page_size, int Hq, int Hkv, int D, float scale, int window,
                                int* __restrict__ err, int vec) {
  using Tile = AgTile<DI>;
  using TT = AgTokenTile<DI>;
  constexpr int TK = Tile::TK, DP = Tile::DP, KS = Tile::KS;
  extern __shared__ __align__(16) float ag_smem[];
  float* const sm_k = ag_smem + TT::OFF_K;
  float* const sm_v = ag_smem + TT::OFF_V;
  float* const sm_q = ag_smem + TT::OFF_Q;
  float* const sm_p = ag_smem + TT::OFF_P;
  long long* const sm_row = reinterpret_cast<long long*>(ag_smem + TT::OFF_ROW);
  __shared__ int chunk_req, chunk_t0, chunk_nt;
  const int warp = (threadIdx.x >> 5) & (AG_HEADS - 1), lane = threadIdx.x & 31;   // the head this warp works for
  const int i0 = (threadIdx.x >> 7) * AG_TH;                                      // ... and the first of its AG_TH tokens
  const int G = Hq / Hkv;
  const int hchunks = (G + AG_HEADS - 1) / AG_HEADS;
  const int c = blockIdx.x / (Hkv * hchunks);
  const int kvh = (blockIdx.x / hchunks) % Hkv;
  const int hchunk = blockIdx.x % hchunks;
  if (threadIdx.x == 0) {
    int left = c, r = 0, t0 = 0, nt = 0;
    for (; r < n_reqs; ++r) {
      const int a = q_start[r], len = q_start[r + 1] - a;
      const int n = (len + AG_TQ - 1) / AG_TQ;
      if (left < n) {
        t0 = a + left * AG_TQ;
        nt = min(AG_TQ, a + len - t0);
        break;
      }
      left -= n;
    }
    chunk_req = r;
    chunk_t0 = t0;
    chunk_nt = nt;     // 0: past the last chunk
  }
  __syncthreads();
  const int req = chunk_req, t0 = chunk_t0, nt = chunk_nt;
  if (nt == 0) return;
  const int h0 = kvh * G + hchunk * AG_HEADS;
  const int nh = min(AG_HEADS, G - hchunk * AG_HEADS);
  // rows: token t0 + i at position pos[i], seeing keys lo[i] .. pos[i]
  int k_begin = 0x7fffffff, k_end = 0;     // the keys that any row of the chunk sees
#pragma unroll
  for (int i = 0; i < AG_TQ; ++i) {
    if (i < nt) {
      const int p = positions[t0 + i];
      k_begin = min(k_begin, window > 0 ? max(0, p - window + 1) : 0);
      k_end = max(k_end, p + 1);
    }
  }
  int pos[AG_TH], lo[AG_TH];               // of this warp's rows
#pragma unroll
  for (int i = 0; i < AG_TH; ++i) {
    pos[i] = i0 + i < nt ? positions[t0 + i0 + i] : -1;
    lo[i] = i0 + i < nt ? (window > 0 ? max(0, pos[i] - window + 1) : 0) : 0x7fffffff;
  }
  const int* bt = block_table + (size_t)req * table_width;
  const size_t v_off = (size_t)Hkv * page_size * D;
  const bool vec_ok = vec != 0;
  const bool async_rows = vec_ok && sizeof(T) == 4;
  const int n_tiles = (k_end - k_begin + TK - 1) / TK;

  auto find_rows = [&](int n) {
    if (threadIdx.x < TK) {
      const int key = k_begin + n * TK + threadIdx.x;
      long long off = -1;
      if (key < k_end) {
        const int lp = key / page_size;
        const int page = lp < table_width ? bt[lp] : -1;
        if (page < 0) atomicExch(err, 5);
        else off = (long long)page * page_stride + ((long long)kvh * page_size + key % page_size) * D;
      }
      sm_row[(n & 1) * TK + threadIdx.x] = off;
    }
  };
  auto load_tile = [&](int n) {
    const int b = n & 1;
    float* const kb = sm_k + b * TK * KS;
    float* const vb = sm_v + b * TK * DP;
    for (int idx = threadIdx.x; idx < TK * (DP / 4); idx += AG_TWARPS * 32) {
      const int j = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
      const long long off = sm_row[b * TK + j];
      if (async_rows) {
        const bool there = off >= 0 && d < D;
        const T* src = kv_plane + (there ? off + d : 0);
        ag_cp_async16(&kb[j * KS + d], src, there ? 16 : 0);
        ag_cp_async16(&vb[j * DP + d], src + (there ? v_off : 0), there ? 16 : 0);
      } else {
        float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
        if (off >= 0) {
          kk = ag_load4<T>(kv_plane + off, d, D, vec_ok);
          vv = ag_load4<T>(kv_plane + off + v_off, d, D, vec_ok);
        }
        *reinterpret_cast<float4*>(&kb[j * KS + d]) = kk;
        *reinterpret_cast<float4*>(&vb[j * DP + d]) = vv;
      }
    }
  };

  // the chunk's queries [token][head][DP], zero past the head size and for rows that do not exist
  for (int idx = threadIdx.x; idx < AG_TQ * AG_HEADS * (DP / 4); idx += AG_TWARPS * 32) {
    const int i = idx / (AG_HEADS * (DP / 4)), g = (idx / (DP / 4)) % AG_HEADS, d = (idx % (DP / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < nt && g < nh) v = ag_load4<T>(q + (size_t)(t0 + i) * ldq + (size_t)(h0 + g) * D, d, D, vec_ok && ldq % 4 == 0);
    *reinterpret_cast<float4*>(&sm_q[(i * AG_HEADS + g) * DP + d]) = v;
  }
  find_rows(0);
  __syncthreads();
  load_tile(0);
  ag_cp_async_commit();

  float m[AG_TH], l[AG_TH], acc[AG_TH][DI];     // of this warp's rows: tokens i0 .. i0 + AG_TH - 1 of the chunk
#pragma unroll
  for (int i = 0; i < AG_TH; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < DI; ++e) acc[i][e] = 0.f;
  }

  for (int n = 0; n < n_tiles; ++n) {
    const int b = n & 1;
    const bool more = n + 1 < n_tiles;
    if (more) find_rows(n + 1);
    __syncthreads();
    if (more) load_tile(n + 1);
    ag_cp_async_commit();
    ag_cp_async_wait<1>();
    const bool have = lane < TK && sm_row[b * TK + lane] >= 0;
    __syncthreads();
    if (warp < nh) {
      const float* const kb = sm_k + b * TK * KS;
      const float* const vb = sm_v + b * TK * DP;
      const int key = k_begin + n * TK + lane;
      // ---- lane j: the scores of key j for this warp's head and the chunk's tokens
      float sc[AG_TH];
#pragma unroll
      for (int i = 0; i < AG_TH; ++i) sc[i] = 0.f;
      {
        const float4* kr = reinterpret_cast<const float4*>(&kb[(lane < TK ? lane : 0) * KS]);
#pragma unroll 4
        for (int cc = 0; cc < DP / 4; ++cc) {
          const float4 k4 = kr[cc];
#pragma unroll
          for (int i = 0; i < AG_TH; ++i) {
            const float4 a = *reinterpret_cast<const float4*>(&sm_q[((i0 + i) * AG_HEADS + warp) * DP + cc * 4]);
            sc[i] = fmaf(a.x, k4.x, sc[i]);
            sc[i] = fmaf(a.y, k4.y, sc[i]);
            sc[i] = fmaf(a.z, k4.z, sc[i]);
            sc[i] = fmaf(a.w, k4.w, sc[i]);
          }
        }
      }
      float corr[AG_TH];
      __syncwarp();                             // the weights of the tile before have been read
#pragma unroll
      for (int i = 0; i < AG_TH; ++i) {
        const bool seen = have && key <= pos[i] && key >= lo[i];
        const float sv = seen ? sc[i] * scale : -INFINITY;
        const float m_new = fmaxf(m[i], warp_max(sv));
        float cr = 1.f, pj = 0.f;
        if (m_new != -INFINITY) {
          cr = m[i] == -INFINITY ? 0.f : expf(m[i] - m_new);
          pj = sv == -INFINITY ? 0.f : expf(sv - m_new);
        }
        l[i] = l[i] * cr + warp_sum(pj);
        m[i] = m_new;
        corr[i] = cr;
        if (lane < TK) sm_p[(warp * AG_TQ + i0 + i) * TK + lane] = pj;
      }
      __syncwarp();
      // ---- lane e: elements e, e + 32, ... of the weighted values of every row, keys in ascending order
#pragma unroll
      for (int i = 0; i < AG_TH; ++i)
#pragma unroll
        for (int e = 0; e < DI; ++e) acc[i][e] *= corr[i];
#pragma unroll 1
      for (int j4 = 0; j4 < TK / 4; ++j4) {
        float vv[4][DI];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int e = 0; e < DI; ++e) vv[jj][e] = vb[(j4 * 4 + jj) * DP + lane + 32 * e];
#pragma unroll
        for (int i = 0; i < AG_TH; ++i) {
          const float4 pw = *reinterpret_cast<const float4*>(&sm_p[(warp * AG_TQ + i0 + i) * TK + j4 * 4]);
#pragma unroll
          for (int e = 0; e < DI; ++e) {
            float a = acc[i][e];
            a = fmaf(pw.x, vv[0][e], a);
            a = fmaf(pw.y, vv[1][e], a);
            a = fmaf(pw.z, vv[2][e], a);
            a = fmaf(pw.w, vv[3][e], a);
            acc[i][e] = a;
          }
        }
      }
    }
  }
  ag_cp_async_wait<0>();
  if (warp >= nh) return;
  const int h = h0 + warp;
#pragma unroll
  for (int i = 0; i < AG_TH; ++i) {
    if (i0 + i >= nt) break;
#pragma unroll
    for (int e = 0; e < DI; ++e) {
      const int d = lane + 32 * e;
      if (d < D) out[(size_t)(t0 + i0 + i) * ldo + (size_t)h * D + d] = from_f32<T>(l[i] > 0.f ? acc[i][e] / l[i] : 0.f);
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
// q_start (n_reqs + 1 entries on the device; may be null): with it and without `part`, tokens of a
// request that follow each other in the batch share their key tiles (the kernel for prompt portions).
FERRUM_API int ferrum_attention_generic(const void* q, int ldq, void* out, int ldo, int dtype, int n_tokens,
                                        const int* positions, const int* req_of_token, const int* block_table,
                                        int table_width, const void* kv_plane, long long page_stride, int page_size,
                                        int Hq, int Hkv, int D, float scale, int window, int* err_flag, float* part,
                                        int split_slots, const int* q_start, int n_reqs, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_tokens >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
  FERRUM_CHECK_ARG(D > 0 && D <= AG_MAX_D, "attention: head size %d is outside (0, %d]", D, AG_MAX_D);
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0, "attention: bad cache arguments");
  FERRUM_CHECK_ARG(ldq >= Hq * D && ldo >= Hq * D, "attention: a row stride is shorter than Hq*D");
  FERRUM_CHECK_ARG(part == nullptr || (split_slots > 0 && split_slots <= 65535), "attention: bad number of split slots %d", split_slots);
  if (n_tokens == 0) return 0;
  const int G = Hq / Hkv;
  const long long rows = (long long)n_tokens * Hkv * ((G + AG_HEADS - 1) / AG_HEADS);
  FERRUM_CHECK_ARG(rows < (1LL << 31), "attention: too many rows");
  // rows of D elements start on 16-byte (float32) or 8-byte (16-bit) borders: vector loads
  const int vec = D % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kv_plane & 15) == 0 && page_stride % 4 == 0;
  if (part == nullptr && q_start != nullptr && n_reqs > 0) {
    // an upper bound of the chunks of AG_TQ tokens, request by request
    const long long chunks = (n_tokens + AG_TQ - 1) / AG_TQ + n_reqs;
    const long long ctas = chunks * Hkv * ((G + AG_HEADS - 1) / AG_HEADS);
    FERRUM_CHECK_ARG(ctas < (1LL << 31), "attention: too many rows");
#define AG_LAUNCH_TOKENS(DI_)                                                                                           \
  FERRUM_DISPATCH_DTYPE(dtype, T, {                                                                                     \
    static bool configured = false;                                                                                     \
    if (!configured) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(attention_generic_tokens_kernel<T, DI_>,                                     \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, AgTokenTile<DI_>::SMEM_BYTES);  \
      FERRUM_CHECK_ARG(e == cudaSuccess, "attention: cannot reserve %d bytes of shared memory: %s",                     \
                       AgTokenTile<DI_>::SMEM_BYTES, cudaGetErrorString(e));                                            \
      configured = true;                                                                                                \
    }                                                                                                                   \
    attention_generic_tokens_kernel<T, DI_><<<(unsigned)ctas, AG_TWARPS * 32, AgTokenTile<DI_>::SMEM_BYTES, stream>>>(   \
      (const T*)q, ldq, (T*)out, ldo, positions, q_start, n_reqs, block_table, table_width, (const T*)kv_plane,         \
      page_stride, page_size, Hq, Hkv, D, scale, window, err_flag, vec);                                                \
  })
    if (D <= 32) AG_LAUNCH_TOKENS(1);
    else if (D <= 64) AG_LAUNCH_TOKENS(2);
    else if (D <= 128) AG_LAUNCH_TOKENS(4);
    else AG_LAUNCH_TOKENS(8);
#undef AG_LAUNCH_TOKENS
    FERRUM_CHECK_LAUNCH("attention_generic_tokens");
    return 0;
  }
  const dim3 grid((unsigned)rows, part ? split_slots : 1);
#define AG_LAUNCH(DI_)                                                                                                  \
  FERRUM_DISPATCH_DTYPE(dtype, T, {                                                                                     \
    static bool configured = false;                                                                                     \
    if (!configured) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T, DI_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           AgTile<DI_>::SMEM_BYTES);                                                    \
      FERRUM_CHECK_ARG(e == cudaSuccess, "attention: cannot reserve %d bytes of shared memory: %s", AgTile<DI_>::SMEM_BYTES, \
                       cudaGetErrorString(e));                                                                          \
      configured = true;                                                                                                \
    }                                                                                                                   \
    attention_generic_kernel<T, DI_><<<grid, AG_WARPS * 32, AgTile<DI_>::SMEM_BYTES, stream>>>(                        \
      (const T*)q, ldq, (T*)out, ldo, positions, req_of_token, block_table, table_width, (const T*)kv_plane, page_stride, \
      page_size, Hq, Hkv, D, scale, window, err_flag, part, split_slots, vec);                                          \
  })
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
