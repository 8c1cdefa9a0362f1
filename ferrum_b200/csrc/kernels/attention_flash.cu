// Paged causal GQA attention on the tensor cores (bfloat16 or float16), for prompt portions and for
// decoded tokens, with an optional split of the key range across CTAs.
//
// One CTA handles one work item x one KV head.  A work item is a tile of BM "packed rows"
// of one request and a key range [kv_begin, kv_end).  Packed row r of a request stands for
// token r / G, query head (kv_head * G + r % G), G = Hq / Hkv: all query heads that share a
// KV head sit in the same tile, so a K/V tile loaded once serves G heads.  A decoded token
// is a tile of G rows (BM = 16, four warps split every 64-key tile between them); a prompt
// portion is a run of BM = 64 row tiles (four warps own 16 rows each).
//
// Per 64-key tile: K and V rows are gathered page by page with cp.async into swizzled
// shared memory (double buffered), S = Q K^T and O += P V run on mma.sync m16n8k16 with
// float32 accumulators, and the softmax is the online one in float32 (scores scaled by
// log2(e)/sqrt(D), exp2).  A work item that covers its rows' whole key range writes the
// output; otherwise it writes (m, l, O) partials and `attention_combine` merges the
// splits in a fixed order.
//
// Two ways to hand out work.  Grid (items, Hkv): one item per CTA and KV head (prompt
// portions).  Or a balanced list: the host cuts the line of all (request, KV head, 64-key
// tile) units into one equal share per CTA slot of the GPU; a share is a few items, each
// naming its KV head, and the CTA walks them (decoded tokens: the whole GPU reads the cache
// at the same rate whatever the mix of context lengths).  Same formulas as the float32 kernel (attention_generic.cu);
// the reference computes them one head and one position at a time
// (crates/model/src/llama.rs:220-247).
#include "common.cuh"

namespace {

typedef uint16_t elem16;   // a bfloat16 or float16 element: the kernels move them and the template says which they are

struct FlashParams {
  const elem16* q;
  elem16* out;
  const elem16* kv_plane;
  const int* block_table;
  const int* q_start;   // [R + 1] first token of each request in this batch
  const int* pos0;      // [R] cached positions before this step
  const int* work;      // [n_work][8]: req, row0, kv_begin, kv_end, n_splits, part_slot, kv_head, -
  const int* cta_items; // null: CTA (x, y) runs item x for KV head y; else CTA x runs items [cta_items[x], cta_items[x+1])
  float* part_o;        // [slot][BM][D]
  float* part_ml;       // [slot][BM][2]
  int* err;             // raised to 5 when a key's page is missing from the block table
  long long page_stride;
  int ldq, ldo, page_size, page_shift, table_width;
  int Hq, Hkv, G, window;
  int trigger_early;    // let the kernels that follow in the stream start (and wait) while this one runs
  float scale_log2;
};

constexpr int BN = 64;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
template <bool HALF>
__device__ __forceinline__ void mma16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  if (HALF)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool HALF>
__device__ __forceinline__ unsigned pack16(float lo, float hi) {
  return HALF ? pack2<__half>(lo, hi) : pack2<__nv_bfloat16>(lo, hi);
}

// element (row, col) of a [rows][D] 16-bit tile whose 16-byte chunks are XOR-swizzled by row
template <int D>
__device__ __forceinline__ elem16* tile_ptr(elem16* base, int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return base + row * D + (chunk << 3) + (col & 7);
}

template <int D, int WM, int WN, bool HALF>
__device__ __forceinline__ void flash_item(const FlashParams& p, const int* wk, int kvh, uint8_t* smem_raw) {
  constexpr int BM = 16 * WM;
  constexpr int NT = WM * WN * 32;
  constexpr int KW = BN / WN;   // keys of a tile that one warp handles
  constexpr int CH = D / 8;     // 16-byte chunks per row
  static_assert(KW % 16 == 0, "a warp needs at least 16 keys per tile");
  elem16* sQ = reinterpret_cast<elem16*>(smem_raw);  // [BM][D]
  elem16* sK = sQ + BM * D;                           // [2][BN][D]
  elem16* sV = sK + 2 * BN * D;                       // [2][BN][D]

  const int req = wk[0], row0 = wk[1], kv_begin = wk[2], kv_end = wk[3], n_splits = wk[4], part = wk[5];
  if (n_splits == 0) return;  // padding of a fixed-size work list
  const int G = p.G;
  const int qs = p.q_start[req];
  const int n_rows = (p.q_start[req + 1] - qs) * G;
  const int pos0 = p.pos0[req];
  const int* bt = p.block_table + (size_t)req * p.table_width;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp % WM, wn = warp / WM;
  const int gid = lane >> 2, tig = lane & 3;
  const int ps = p.page_size;
  const size_t v_off = (size_t)p.Hkv * ps * D;

  // ---- Q tile -> shared memory
  for (int idx = tid; idx < BM * CH; idx += NT) {
    const int r = idx / CH, c = idx % CH;
    const int pr = row0 + r;
    elem16* dst = sQ + r * D + ((c ^ (r & 7)) << 3);
    if (pr < n_rows) {
      const elem16* src = p.q + (size_t)(qs + pr / G) * p.ldq + (size_t)(kvh * G + pr % G) * D + c * 8;
      cp_async16(dst, src, 16);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  // Every thread copies the same 16-byte column c of rows r_base, r_base + RPP, ... of a tile;
  // the swizzle term (row & 7) is the same for all of them because RPP is a multiple of 8.
  constexpr int RPP = NT / CH;       // rows covered by one pass of the CTA
  constexpr int PASSES = BN / RPP;
  static_assert(NT % CH == 0 && RPP % 8 == 0 && BN % RPP == 0, "load pattern");
  const int ld_c = tid % CH, ld_r = tid / CH;
  const int ld_off = ld_r * D + ((ld_c ^ (ld_r & 7)) << 3);
  const elem16* kv_head = p.kv_plane + (size_t)kvh * ps * D + ld_c * 8;
  const int ps_shift = p.page_shift;  // log2(page_size), or -1 when it is no power of two
  bool page_missing = false;   // a key of the range had no page (checked without a branch in the copy loop)
  auto load_tile = [&](int buf, int key0) {
    elem16* dk = sK + buf * BN * D + ld_off;
    elem16* dv = sV + buf * BN * D + ld_off;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const int key = key0 + ld_r + i * RPP;
      const bool in_range = key < kv_end;
      const int lp = ps_shift >= 0 ? key >> ps_shift : key / ps;
      const int in_page = ps_shift >= 0 ? key & (ps - 1) : key - lp * ps;
      const int page = (in_range && lp < p.table_width) ? bt[lp] : -1;
      const bool valid = page >= 0;      // a key without a page: nothing is read, the rows arrive as zeros
      page_missing |= in_range && !valid;
      const elem16* src = kv_head + (size_t)max(page, 0) * p.page_stride + in_page * D;
      cp_async16(dk + i * RPP * D, src, valid ? 16 : 0);
      cp_async16(dv + i * RPP * D, src + v_off, valid ? 16 : 0);
    }
  };
  const int n_tiles = (kv_end - kv_begin + BN - 1) / BN;
  if (n_tiles > 0) load_tile(0, kv_begin);
  cp_async_commit();

  // per-thread row bookkeeping: this thread owns rows gid and gid + 8 of its warp's 16
  int row_pos[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int pr = row0 + wm * 16 + gid + h * 8;
    row_ok[h] = pr < n_rows;
    row_pos[h] = pos0 + pr / G;
    row_lo[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
  }
  // the earliest position and the latest window start among the warp's rows that exist
  const int warp_row0 = row0 + wm * 16;
  const int warp_last = min(warp_row0 + 15, n_rows - 1);
  const int warp_min_pos = pos0 + warp_row0 / G;
  const int warp_max_lo = p.window > 0 && warp_last >= warp_row0 ? max(0, pos0 + warp_last / G - p.window + 1) : 0;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  unsigned qf[D / 16][4];

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < n_tiles) load_tile(buf ^ 1, kv_begin + (it + 1) * BN);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int r = wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(qf[kk], tile_ptr<D>(sQ, r, kk * 16 + (lane >> 4) * 8));
      }
    }
    elem16* tK = sK + buf * BN * D;
    elem16* tV = sV + buf * BN * D;
    const int key0 = kv_begin + it * BN + wn * KW;

    // ---- S = Q K^T for this warp's 16 rows x KW keys
    float s[KW / 8][4];
#pragma unroll
    for (int j = 0; j < KW / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int nb = 0; nb < KW / 16; ++nb) {
        unsigned b[4];
        const int r = wn * KW + nb * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(b, tile_ptr<D>(tK, r, kk * 16 + ((lane >> 3) & 1) * 8));
        mma16<HALF>(s[2 * nb], qf[kk], b[0], b[1]);
        mma16<HALF>(s[2 * nb + 1], qf[kk], b[2], b[3]);
      }
    }
    // ---- mask, scale, online softmax.  A tile that every row of the warp sees in full
    // needs no mask (rows past the request's last row compute on zeros and are dropped).
    float mx[2] = {-INFINITY, -INFINITY};
    if (key0 + KW - 1 <= warp_min_pos && key0 >= warp_max_lo && key0 + KW <= kv_end) {
#pragma unroll
      for (int j = 0; j < KW / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] *= p.scale_log2;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < KW / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + tig * 2 + (e & 1);
          const int h = e >> 1;
          const bool keep = row_ok[h] && key <= row_pos[h] && key >= row_lo[h] && key < kv_end;
          s[j][e] = keep ? s[j][e] * p.scale_log2 : -INFINITY;
          mx[h] = fmaxf(mx[h], s[j][e]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      corr[h] = exp2f(m_run[h] - m_use[h]);   // 0 when nothing was seen before
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
#pragma unroll
    for (int j = 0; j < KW / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[j][e] - m_use[e >> 1]);
        s[j][e] = pv;
        l_run[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < KW / 16; ++ks) {
      unsigned a[4];
      a[0] = pack16<HALF>(s[2 * ks][0], s[2 * ks][1]);
      a[1] = pack16<HALF>(s[2 * ks][2], s[2 * ks][3]);
      a[2] = pack16<HALF>(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      a[3] = pack16<HALF>(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int db = 0; db < D / 16; ++db) {
        unsigned b[4];
        const int r = wn * KW + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(b, tile_ptr<D>(tV, r, db * 16 + (lane >> 4) * 8));
        mma16<HALF>(o[2 * db], a, b[0], b[1]);
        mma16<HALF>(o[2 * db + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // everyone is done with this buffer before the next load overwrites it
  }
  cp_async_wait<0>();
  __syncthreads();
  if (page_missing) atomicExch(p.err, 5);   // the step fails; what this item writes is discarded by the host

  // ---- each warp leaves (m, l, O) in shared memory; the WN partial results are merged
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* sO = reinterpret_cast<float*>(smem_raw);        // [WN][BM][D]
  float* sML = sO + WN * BM * D;                          // [WN][BM][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = wm * 16 + gid + h * 8;
    if (tig == 0) {
      sML[(wn * BM + r) * 2] = m_run[h];
      sML[(wn * BM + r) * 2 + 1] = l_run[h];
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      float2 v = make_float2(o[j][2 * h], o[j][2 * h + 1]);
      *reinterpret_cast<float2*>(sO + ((size_t)(wn * BM + r)) * D + j * 8 + tig * 2) = v;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < BM * (D / 4); idx += NT) {
    const int r = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const int pr = row0 + r;
    if (pr >= n_rows) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WN; ++w) M = fmaxf(M, sML[(w * BM + r) * 2]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WN; ++w) {
      const float mw = sML[(w * BM + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += sML[(w * BM + r) * 2 + 1] * f;
      const float4 v = *reinterpret_cast<const float4*>(sO + ((size_t)(w * BM + r)) * D + d);
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
    }
    if (n_splits == 1) {
      const float inv = L > 0.f ? 1.0f / L : 0.f;
      elem16* dst = p.out + (size_t)(qs + pr / G) * p.ldo + (size_t)(kvh * G + pr % G) * D + d;
      uint2 packed;
      packed.x = pack16<HALF>(acc.x * inv, acc.y * inv);
      packed.y = pack16<HALF>(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(dst) = packed;
    } else {
      const size_t slot = (size_t)part * BM + r;
      *reinterpret_cast<float4*>(p.part_o + slot * D + d) = acc;
      if (d == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = L;
      }
    }
  }
}

template <int D, int WM, int WN, bool HALF>
__global__ void __launch_bounds__(WM * WN * 32)
flash_kernel(const FlashParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // Blocks of the next kernels that sit on the SMs waiting for this one to finish slow a large
  // attention grid down by a third (measured at 64 requests), so the dependents are released
  // early only on request: with a few decoded tokens the merge kernel's blocks are tiny, and
  // the blocks of the product after it move in as this kernel's blocks leave and fetch their
  // first weight tiles while the slowest blocks here finish.
  if (p.trigger_early) pdl_launch();
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0, TRACE_FLASH);
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  if (p.cta_items == nullptr) {
    const int* wk = p.work + (size_t)blockIdx.x * 8;
    // with one item per (CTA, head) the item's partial slot is per head
    int item[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) item[i] = wk[i];
    item[5] = item[5] * p.Hkv + blockIdx.y;
    flash_item<D, WM, WN, HALF>(p, item, blockIdx.y, smem_raw);
    TRACE_MARK(TRACE_EXIT);
    return;
  }
  const int begin = p.cta_items[blockIdx.x], end = p.cta_items[blockIdx.x + 1];
  for (int w = begin; w < end; ++w) {
    const int* wk = p.work + (size_t)w * 8;
    flash_item<D, WM, WN, HALF>(p, wk, wk[6], smem_raw);
    __syncthreads();  // the next item's loads reuse the shared memory the merge just read
  }
  TRACE_MARK(TRACE_EXIT);
}


// Merges the splits of every (token, head) whose tile was split.  tile_info: per (tile, KV
// head) [first part slot, n_splits, slot stride, 0]; req_tile0[r]: index of request r's first
// tile; token_list: the tokens to visit (null: all n_tokens).  A block is one (token, head):
// 32 lanes x 4 features, times blockDim.x / 32 warps that share the splits among them (a
// single decoded request's keys are cut into dozens of splits: one warp would walk them in
// seven rounds of memory latency).
constexpr int COMBINE_MAX_WARPS = 8;
template <int D>
__global__ void __launch_bounds__(32 * COMBINE_MAX_WARPS)
combine_kernel(elem16* out, int ldo, const float* part_o, const float* part_ml, const int* q_start,
               const int* req_of_token, const int* req_tile0, const int* tile_info, const int* token_list, int G,
               int Hkv, int BM, int half) {
  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0, TRACE_COMBINE);
  pdl_launch();
  // The index arrays were copied to the device before the step's first kernel ran: they are
  // read before the wait for the attention kernel, whose partials come after it.
  const int t = token_list ? token_list[blockIdx.x] : blockIdx.x, head = blockIdx.y;
  const int req = req_of_token[t];
  const int kvh = head / G;
  const int pr = (t - q_start[req]) * G + head % G;
  const int* info = tile_info + 4 * ((size_t)(req_tile0[req] + pr / BM) * Hkv + kvh);
  const int first = info[0], n = info[1], stride = info[2];
  pdl_wait();
  TRACE_MARK(TRACE_WAITED);
  TRACE_MARK(TRACE_EXIT);
  if (n <= 1) return;
  const int r = pr % BM;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int d = lane * 4;
  const bool active = d < D;
  // Eight splits at a time, all their loads in flight together (the kernel is a chain of memory
  // latencies otherwise); the running maximum is carried from one group to the next.  Which
  // warp takes which splits and the order of the sums are fixed, so the result does not depend
  // on which block of the attention kernel finished first.
  constexpr int GROUP = 8;
  float M = -INFINITY, L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = warp * GROUP; s0 < n && active; s0 += n_warps * GROUP) {
    float ms[GROUP], ls[GROUP];
    float4 v[GROUP];
#pragma unroll
    for (int k = 0; k < GROUP; ++k) {
      const bool have = s0 + k < n;
      const size_t slot = (size_t)(first + (have ? s0 + k : 0) * stride) * BM + r;
      ms[k] = have ? __ldcg(part_ml + slot * 2) : -INFINITY;
      ls[k] = have ? __ldcg(part_ml + slot * 2 + 1) : 0.f;
      v[k] = have ? __ldcg(reinterpret_cast<const float4*>(part_o + slot * D + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m_new = M;
#pragma unroll
    for (int k = 0; k < GROUP; ++k) m_new = fmaxf(m_new, ms[k]);
    const float keep = M == -INFINITY ? 0.f : exp2f(M - m_new);
    L *= keep;
    acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
    for (int k = 0; k < GROUP; ++k) {
      const float f = ms[k] == -INFINITY ? 0.f : exp2f(ms[k] - m_new);
      L += ls[k] * f;
      acc.x += v[k].x * f; acc.y += v[k].y * f; acc.z += v[k].z * f; acc.w += v[k].w * f;
    }
    M = m_new;
  }
  if (n_warps > 1) {  // the warps' sums meet in warp order
    // (dynamic shared memory, none with one warp: the blocks of this kernel become resident
    // beside the attention kernel's, which leave little)
    extern __shared__ float4 combine_smem[];
    float4(*sm_acc)[32] = reinterpret_cast<float4(*)[32]>(combine_smem);
    float2(*sm_ml)[32] = reinterpret_cast<float2(*)[32]>(combine_smem + n_warps * 32);
    sm_ml[warp][lane] = make_float2(M, L);
    sm_acc[warp][lane] = acc;
    __syncthreads();
    if (warp != 0) return;
    M = -INFINITY;
    L = 0.f;
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int w = 0; w < n_warps; ++w) {
      const float2 ml = sm_ml[w][lane];
      const float4 v = sm_acc[w][lane];
      const float m_new = fmaxf(M, ml.x);
      const float keep = M == -INFINITY ? 0.f : exp2f(M - m_new);
      const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - m_new);
      L = L * keep + ml.y * f;
      acc.x = acc.x * keep + v.x * f; acc.y = acc.y * keep + v.y * f;
      acc.z = acc.z * keep + v.z * f; acc.w = acc.w * keep + v.w * f;
      M = m_new;
    }
  }
  if (!active) return;
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  uint2 packed;
  packed.x = pack2_bits(acc.x * inv, acc.y * inv, half != 0);
  packed.y = pack2_bits(acc.z * inv, acc.w * inv, half != 0);
  *reinterpret_cast<uint2*>(out + (size_t)t * ldo + (size_t)head * D + d) = packed;
}

template <int D, int WM, int WN, bool HALF>
int launch_flash(const FlashParams& p, int n_work, int n_ctas, cudaStream_t stream) {
  constexpr int BM = 16 * WM;
  constexpr int kv_bytes = 4 * BN * D * 2 + BM * D * 2;
  constexpr int merge_bytes = WN * BM * (D + 2) * 4;
  constexpr int smem = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_kernel<D, WM, WN, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    FERRUM_CHECK_ARG(e == cudaSuccess, "attention_flash: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid = p.cta_items ? dim3(n_ctas, 1) : dim3(n_work, p.Hkv);
  launch_kernel(flash_kernel<D, WM, WN, HALF>, grid, dim3(WM * WN * 32), smem, stream, p);
  FERRUM_CHECK_LAUNCH("attention_flash");
  return 0;
}

}  // namespace

FERRUM_TRACE_READER(ferrum_trace_flash)

FERRUM_API int ferrum_attention_flash_supported(int D, int bm) { return (D == 64 || D == 128) && (bm == 16 || bm == 64); }

// work: [n_work][8] int32 on the device (see FlashParams).  bm: 16 (a few rows per request,
// key range split between four warps) or 64.  cta_items (n_ctas + 1 ints) selects the
// balanced-list mode; null runs a grid of (n_work, Hkv).
FERRUM_API int ferrum_attention_flash(const void* q, int ldq, void* out, int ldo, int dtype, const void* kv_plane,
                                      long long page_stride, int page_size, const int* block_table, int table_width,
                                      const int* q_start, const int* pos0, const int* work, int n_work,
                                      const int* cta_items, int n_ctas, float* part_o, float* part_ml, int Hq, int Hkv,
                                      int D, float scale, int window, int bm, int trigger_early, int* err_flag,
                                      cudaStream_t stream) {
  FERRUM_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention_flash: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
  FERRUM_CHECK_ARG(ferrum_is_16bit(dtype), "attention_flash: dtype code %d is not a 16-bit type", dtype);
  FERRUM_CHECK_ARG(err_flag != nullptr, "attention_flash: the error flag is required");
  FERRUM_CHECK_ARG(ferrum_attention_flash_supported(D, bm), "attention_flash: head size %d with row tile %d is not built; "
                   "use the generic kernel", D, bm);
  FERRUM_CHECK_ARG(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                   ((uintptr_t)kv_plane & 15) == 0, "attention_flash: operands must be 16-byte aligned");
  FERRUM_CHECK_ARG(page_size > 0 && table_width > 0 && window >= 0 && n_work >= 0, "attention_flash: bad arguments");
  if (n_work == 0) return 0;
  FERRUM_CHECK_ARG(cta_items == nullptr || n_ctas > 0, "attention_flash: an item list needs a CTA count");
  FlashParams p;
  p.cta_items = cta_items;
  p.q = (const elem16*)q; p.out = (elem16*)out; p.kv_plane = (const elem16*)kv_plane;
  p.err = err_flag;
  p.block_table = block_table; p.q_start = q_start; p.pos0 = pos0; p.work = work;
  p.part_o = part_o; p.part_ml = part_ml; p.page_stride = page_stride;
  p.ldq = ldq; p.ldo = ldo; p.page_size = page_size; p.table_width = table_width;
  p.page_shift = -1;
  for (int b = 0; b < 30; ++b)
    if ((1 << b) == page_size) p.page_shift = b;
  p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.window = window;
  p.trigger_early = trigger_early;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (dtype == FERRUM_F16) {
    if (D == 64 && bm == 16) return launch_flash<64, 1, 4, true>(p, n_work, n_ctas, stream);
    if (D == 64 && bm == 64) return launch_flash<64, 4, 1, true>(p, n_work, n_ctas, stream);
    if (D == 128 && bm == 16) return launch_flash<128, 1, 4, true>(p, n_work, n_ctas, stream);
    return launch_flash<128, 4, 1, true>(p, n_work, n_ctas, stream);
  }
  if (D == 64 && bm == 16) return launch_flash<64, 1, 4, false>(p, n_work, n_ctas, stream);
  if (D == 64 && bm == 64) return launch_flash<64, 4, 1, false>(p, n_work, n_ctas, stream);
  if (D == 128 && bm == 16) return launch_flash<128, 1, 4, false>(p, n_work, n_ctas, stream);
  return launch_flash<128, 4, 1, false>(p, n_work, n_ctas, stream);
}

FERRUM_API int ferrum_attention_combine(void* out, int ldo, int dtype, const float* part_o, const float* part_ml,
                                        const int* q_start, const int* req_of_token, const int* req_tile0,
                                        const int* tile_info, const int* token_list, int n_tokens, int Hq, int Hkv,
                                        int D, int bm, int n_warps, cudaStream_t stream) {
  FERRUM_CHECK_ARG(D == 64 || D == 128, "attention_combine: head size %d is not built", D);
  FERRUM_CHECK_ARG(ferrum_is_16bit(dtype), "attention_combine: dtype code %d is not a 16-bit type", dtype);
  const int half = dtype == FERRUM_F16;
  FERRUM_CHECK_ARG(n_warps >= 1 && n_warps <= COMBINE_MAX_WARPS, "attention_combine: %d warps per block (1..%d)", n_warps,
                   COMBINE_MAX_WARPS);
  if (n_tokens == 0) return 0;
  dim3 grid(n_tokens, Hq);
  FERRUM_CHECK_ARG(grid.y <= 65535, "attention_combine: too many heads");
  const int smem = n_warps > 1 ? n_warps * 32 * (int)(sizeof(float4) + sizeof(float2)) : 0;
  if (D == 64)
    launch_kernel(combine_kernel<64>, grid, dim3(32 * n_warps), smem, stream, (elem16*)out, ldo, part_o, part_ml, q_start,
                  req_of_token, req_tile0, tile_info, token_list, Hq / Hkv, Hkv, bm, half);
  else
    launch_kernel(combine_kernel<128>, grid, dim3(32 * n_warps), smem, stream, (elem16*)out, ldo, part_o, part_ml, q_start,
                  req_of_token, req_tile0, tile_info, token_list, Hq / Hkv, Hkv, bm, half);
  FERRUM_CHECK_LAUNCH("attention_combine");
  return 0;
}
