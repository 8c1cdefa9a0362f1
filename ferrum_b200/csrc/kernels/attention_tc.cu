// Paged causal GQA attention for prompt portions on the tcgen05 matrix unit (bfloat16 or float16).
//
// One CTA handles one work item x one KV head.  An item is a pair of row tiles of one request
// and a key range [kv_begin, kv_end).  A row tile is `tok` consecutive tokens x the G query
// heads of the KV head (tok = 128 / G, so tok * G <= 128 rows: row r is token r / G, head
// r % G); a TMA box over (head size, heads, tokens) puts it in shared memory as the 128-row
// K-major operand of the instruction.  Keys and values come page by page with TMA into
// 64-key stages.  Per 64 keys and row tile:
//   S = Q K^T          tcgen05.mma 128 x 64 x D into tensor memory
//   P = exp2(S - m)    128 threads, one per row, read S from tensor memory, keep the running
//                      maximum and sum in float32 and write P (bfloat16) back over the first
//                      half of the same columns
//   O += P V           tcgen05.mma 128 x D x 64 with P as the tensor-memory operand and V as the
//                      MN-major operand straight from the page layout, O in tensor memory
// P never passes through shared memory: the matrix unit fetches its shared-memory operands at
// about 64 bytes a cycle, and with Q re-read for every 64 keys that fetch, not the arithmetic,
// is what a stage costs (16 x 6 KB for the scores, 8 x 4 KB for the values).
// S has two buffers per row tile, so the matrix unit computes the scores of the stage after next
// while the threads of a tile work on P: a tile's threads never wait for a product that
// depends on their own P, and the two tiles share the matrix unit.  The running maximum is only moved (and O rescaled, in tensor
// memory, by the row's own thread) when it grows by more than 2^8; until then P is computed
// against the older maximum, which changes nothing in the quotient O / l.
//
// What sets the pace (clocks taken per role on a 2,048-token prompt): a 64-key stage of both tiles
// takes about 2,300 cycles, and the chain that closes every two stages is softmax of stage j
// (1,800 cycles for its 64 exponentials at the special-function unit's rate with the other tile's
// warp on the same scheduler, the maximum, P) -> P V of stage j (its P lies over the scores'
// buffer) -> Q K^T of stage j + 2 into that buffer (eight dependent steps: 1,600 cycles from the
// first instruction to the scores being seen) -> softmax of stage j + 2.  A thread gets one
// tcgen05.mma, and a warp one TMA copy, off about every 120 cycles whatever the instruction's
// size (one, two and four issuing threads: 121, 60 and 30 + cycles an instruction overall), which
// is why the steps of a product cost what they do.  Built, verified and measured without a gain
// (47.7 to 49.4 us against 47.7 us; 553 to 581 against 556 us at 8,192 tokens), each removing one
// of the three 2,100-to-2,300-cycle limits and meeting the next: a producer warp each for keys and
// values (one warp's sixteen copies of a stage take 2,300 cycles); an issuing thread each for
// Q K^T and P V of a tile (one thread's twelve steps and six commits take 2,100); P in columns of
// its own with one score buffer, so that the next scores are issued as soon as the current ones
// have been read (their eight dependent steps then end about when the softmax does, 1,900
// cycles); and all three together.  One issuing thread for both tiles, step by step in turn, was
// slower (54 us).  At 2,048 tokens a third of the time is outside this loop: 256 items of 1 to 32
// stages on 148 CTAs, each with some 3.5 us of start and end (Q, first keys, output).
//
// Roles (352 threads): warp 0 = TMA producer, warps 1 and 2 = MMA issuers of tile 0 and 1 (one
// issuing thread each: while one does its waits and commits, the other's products run; warp 1
// also owns the tensor memory), warps 3..6 = rows of tile 0, warps 7..10 = rows of tile 1.  Every wait is bounded; on a
// timeout the kernel raises the error flag, lets copies in flight land, frees its tensor
// memory and returns.  An item whose key range is a split writes (m, l, O) partials in the
// layout of the mma.sync kernel (attention_flash.cu) and `attention_combine` merges them.
// Same formulas as the float32 kernel (attention_generic.cu; the reference computes them one
// head and one position at a time, crates/model/src/llama.rs:220-247).
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

namespace {

constexpr float TC_LAZY = 8.0f;  // the running maximum moves when it grows by more than this (log2 units)

struct AttnTcParams {
  uint16_t* out;        // bfloat16 or float16 elements, as the template says
  const int* block_table;
  const int* q_start;   // [R + 1] first token of each request in this batch
  const int* pos0;      // [R] cached positions before this step
  const int* work;      // [n_work][8]: req, row0, kv_begin, kv_end, n_splits, part_slot, -, -
  float* part_o;        // [slot][2 * tok * G][D]
  float* part_ml;       // [slot][2 * tok * G][2]
  int* err;
  int ldo, page_size, page_shift, table_width;
  int Hkv, G, tok, window;
  float scale_log2;
};

// NT row tiles per CTA, BN keys per stage, NS stages of keys and of values.
template <int D, int NT, int BN, int NS>
struct AttnTcConfig {
  static constexpr int HALVES = D / 64;                          // 64-column spans of a head
  static constexpr int Q_TILE_BYTES = HALVES * 128 * 128;       // 128 rows x 128 bytes per 64 columns
  static constexpr int KV_HALF_BYTES = BN * 128;
  static constexpr int KV_STAGE_BYTES = HALVES * KV_HALF_BYTES;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + NT * Q_TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NS * KV_STAGE_BYTES;
  static constexpr int OFF_BARS = OFF_V + NS * KV_STAGE_BYTES;
  static constexpr int N_BARS = 1 + 4 * NS + 6 * NT;
  static constexpr int SMEM_BYTES = OFF_BARS + N_BARS * 8 + 1024 /*alignment slack*/;
  static constexpr int S_COL = 0;                 // S of tile t, buffer b: columns (2 t + b) * BN ..
  static constexpr int O_COL = NT * 2 * BN;       // O of tile t: columns O_COL + t * D ..
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 32 * (1 + NT + 4 * NT);   // producer, one issuer and four softmax warps per tile
  static_assert(O_COL + NT * D <= TMEM_COLS, "accumulators do not fit tensor memory");
  static_assert(SMEM_BYTES <= 232448, "stages do not fit shared memory");
  static_assert(BN % 64 == 0 && BN <= 256, "a stage is one or more 64-key spans");
};

// MN-major shared-memory operand with the 128-byte swizzle: 64 elements along N (128 bytes)
// x 8 along K form a 1024-byte atom; atoms follow each other along K at `sbo` bytes and along
// N at `lbo` bytes.  This is the layout a TMA box of (64 columns, rows) leaves when the rows
// are the K index, which is how value pages lie in the cache.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// 32 lanes x 32 columns of 32-bit from tensor memory (thread i: lane base + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
      "[%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n\t"
      "tcgen05.wait::st.sync.aligned;" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
      "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
      "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
      "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}

__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n\t"
      "tcgen05.wait::st.sync.aligned;" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
      "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
      "r"(v[31])
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool HALF>
__device__ __forceinline__ uint32_t pack2_16(float lo, float hi) {
  return HALF ? pack2<__half>(lo, hi) : pack2<__nv_bfloat16>(lo, hi);
}

template <int D, int NT, int BN, int NS, bool HALF>
__global__ void __launch_bounds__(AttnTcConfig<D, NT, BN, NS>::THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const AttnTcParams p) {
  using Cfg = AttnTcConfig<D, NT, BN, NS>;
  constexpr int HALVES = Cfg::HALVES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest in the grid: the work list is sorted by length, and this way the longest
  // items of every head start first
  const int kvh = blockIdx.x;
  const int* wk = p.work + (size_t)blockIdx.y * 8;
  const int req = wk[0], row0 = wk[1], kv_begin = wk[2], kv_end = wk[3], n_splits = wk[4];
  if (n_splits == 0 || kv_end <= kv_begin) return;  // padding of a fixed-size work list (uniform for the CTA)
  const int part = wk[5] * p.Hkv + kvh;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::OFF_BARS;
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (1 + NS + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (1 + 2 * NS + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (1 + 3 * NS + s); };
  auto s_ready = [&](int t, int b) { return bar_base + 8u * (1 + 4 * NS + 2 * t + b); };
  auto p_ready = [&](int t, int b) { return bar_base + 8u * (1 + 4 * NS + 2 * NT + 2 * t + b); };
  auto pv_done = [&](int t) { return bar_base + 8u * (1 + 4 * NS + 4 * NT + t); };
  auto o_done = [&](int t) { return bar_base + 8u * (1 + 4 * NS + 5 * NT + t); };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_kv);
    mbar_init(q_full, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), NT);   // one commit per issuer
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), NT);
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(s_ready(t, 0), 1);
      mbar_init(s_ready(t, 1), 1);
      mbar_init(p_ready(t, 0), 128);
      mbar_init(p_ready(t, 1), 128);
      mbar_init(pv_done(t), 1);
      mbar_init(o_done(t), 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_p = &abort_flag;
  // a whole warp waits and decides together, so that the warp-wide instructions after the wait
  // (tensor-memory loads, votes) are never entered by a part of it
  auto wait_all = [&](uint32_t bar, uint32_t parity) {
    const bool got = mbar_wait(bar, parity, abort_p);
    return __all_sync(0xffffffffu, got) != 0;
  };
  pdl_wait();

  const int G = p.G, tok = p.tok;
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int pos0 = p.pos0[req];
  const int tok0 = row0 / G;                  // first token of the item within its request
  const int kv0 = kv_begin & ~(BN - 1);       // stages start on BN-key borders: whole pages
  const int n_j = (kv_end - kv0 + BN - 1) / BN;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Lane 0 waits and posts the byte counts; lane i fetches page i of a stage (its table entry
    // is read one stage ahead, so that the lookups of a stage overlap instead of queueing).  The
    // keys of stage j + 1 are requested before the values of stage j: the scores run ahead.
    if (lane == 0) {
      mbar_expect_tx(q_full, NT * HALVES * tok * G * 128);
      for (int t = 0; t < NT; ++t)
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(smem_base + Cfg::OFF_Q + t * Cfg::Q_TILE_BYTES + h * 128 * 128, &map_q, q_full, h * 64, kvh * G,
                      qs + tok0 + t * tok);
    }
    const int ps = p.page_size;
    const int pages_per_stage = BN / ps;
    const int* bt = p.block_table + (size_t)req * p.table_width;
    auto page_of = [&](int j) {  // this lane's page of stage j; a page past the key range reads as zeros (masked keys)
      const int lp = ((kv0 + j * BN) >> p.page_shift) + lane;
      if (!(lane < pages_per_stage && j >= 0 && j < n_j)) return -1;
      const int page = lp < p.table_width ? bt[lp] : -1;
      // a key of the item's range without a page: the keys arrive as zeros and the step fails
      if (page < 0 && lp * ps < kv_end && (lp + 1) * ps > kv_begin) atomicExch(p.err, 5);
      return page;
    };
    // one stage of keys (kv = 0) or values (kv = 1); false on a timeout
    auto load_stage = [&](int j, int kv, int page) {
      const int s = j % NS;
      const uint32_t parity = ((j / NS) & 1) ^ 1;
      const uint32_t full = kv ? v_full(s) : k_full(s);
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(kv ? v_empty(s) : k_empty(s), parity, abort_p);
        if (ok) mbar_expect_tx(full, Cfg::KV_STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      if (lane < pages_per_stage) {
        const int y = page < 0 ? -ps : ((page * 2 + kv) * p.Hkv + kvh) * ps;   // a negative row: the box reads as zeros
        const uint32_t dst = smem_base + (kv ? Cfg::OFF_V : Cfg::OFF_K) + s * Cfg::KV_STAGE_BYTES + lane * ps * 128;
        for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * Cfg::KV_HALF_BYTES, &map_kv, full, h * 64, y);
      }
      return true;
    };
    int page_v = -1, page_k = page_of(0);
    bool ok = true;
    for (int j = 0; ok && j <= n_j; ++j) {   // keys of stage j, then values of stage j - 1
      const int next_k = page_of(j + 1);
      if (j < n_j) ok = load_stage(j, 0, page_k);
      if (ok && j > 0) ok = load_stage(j - 1, 1, page_v);
      page_v = page_k;
      page_k = next_k;
    }
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.err, 20);
    }
  } else if (warp <= NT) {
    // ------------------------------------------------------------ MMA issuer of one row tile
    if (lane == 0) {
      const int t = warp - 1;
      const uint32_t idesc_qk = umma_idesc_16bit(128, BN, HALF);
      const uint32_t idesc_pv = umma_idesc_16bit(128, D, HALF) | (1u << 16);  // B (values) is MN-major
      const uint32_t q_addr = smem_base + Cfg::OFF_Q + t * Cfg::Q_TILE_BYTES;
      const uint32_t o_tmem = tmem_base + Cfg::O_COL + t * D;
      auto issue_qk = [&](int s, int buf) {
        const uint32_t k_addr = smem_base + Cfg::OFF_K + s * Cfg::KV_STAGE_BYTES;
        const uint32_t s_tmem = tmem_base + Cfg::S_COL + (2 * t + buf) * BN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int h = kk >> 2, in = kk & 3;
          umma_bf16(s_tmem, umma_desc_k_sw128(q_addr + h * 128 * 128) + (uint64_t)(in * 2),
                    umma_desc_k_sw128(k_addr + h * Cfg::KV_HALF_BYTES) + (uint64_t)(in * 2), idesc_qk, kk > 0);
        }
      };
      auto issue_pv = [&](int s, int buf, bool accumulate) {
        const uint32_t v_addr = smem_base + Cfg::OFF_V + s * Cfg::KV_STAGE_BYTES;
        const uint32_t p_tmem = tmem_base + Cfg::S_COL + (2 * t + buf) * BN;  // P lies over the scores it came from
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)  // 16 keys on: 8 columns of P, 16 rows of V
          umma_bf16_ts(o_tmem, p_tmem + kk * 8, umma_desc_mn_sw128(v_addr + kk * 16 * 128, Cfg::KV_HALF_BYTES, 1024), idesc_pv,
                       accumulate || kk > 0);
      };
      // the scores of stages 0 and 1 go ahead; in the loop the scores of stage j + 2 follow P V of stage j
      bool ok = mbar_wait(q_full, 0, abort_p);
      for (int jj = 0; ok && jj < 2 && jj < n_j; ++jj) {
        ok = mbar_wait(k_full(jj % NS), (jj / NS) & 1, abort_p);
        if (!ok) break;
        tc_fence_after();
        issue_qk(jj % NS, jj);
        umma_commit(s_ready(t, jj));
        umma_commit(k_empty(jj % NS));
      }
      if (!ok) {
        abort_flag = 1;
        atomicExch(p.err, 22);
      }
      for (int j = 0; ok && j < n_j; ++j) {
        const int s = j % NS;
        const int jn = j + 2;
        const bool more = jn < n_j;
        const int s2 = jn % NS;
        ok = mbar_wait(v_full(s), (j / NS) & 1, abort_p);
        if (!ok) {
          abort_flag = 1;
          atomicExch(p.err, 23);
          break;
        }
        ok = mbar_wait(p_ready(t, j & 1), (j >> 1) & 1, abort_p);
        if (!ok) {
          abort_flag = 1;
          atomicExch(p.err, 24);
          break;
        }
        tc_fence_after();
        issue_pv(s, j & 1, j > 0);
        umma_commit(pv_done(t));
        if (j + 1 == n_j) umma_commit(o_done(t));
        umma_commit(v_empty(s));
        if (more) {
          ok = mbar_wait(k_full(s2), (jn / NS) & 1, abort_p);
          if (!ok) {
            abort_flag = 1;
            atomicExch(p.err, 23);
            break;
          }
          tc_fence_after();
          issue_qk(s2, j & 1);
          umma_commit(s_ready(t, j & 1));
          umma_commit(k_empty(s2));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax and output: one thread per row
    const int t = (warp - 1 - NT) >> 2;       // row tile of this warp
    const int quarter = warp & 3;             // the tensor-memory lanes this warp may touch
    const int r = quarter * 32 + lane;        // row of the tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int tok_in_req = tok0 + t * tok + r / G;
    const bool row_valid = r < tok * G && tok_in_req < q_len;
    const int qpos = pos0 + tok_in_req;
    // the tile's rows see keys up to qpos_min without a mask, none beyond qpos_max
    const int tile_first = tok0 + t * tok;
    const int qpos_min = pos0 + tile_first;
    const int qpos_max = pos0 + min(q_len - 1, tile_first + tok - 1);
    const bool tile_full = tok * G == 128 && tile_first + tok <= q_len;  // every row of the tile exists
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_j; ++j) {
      const int buf = j & 1;
      ok = wait_all(s_ready(t, buf), (j >> 1) & 1);
      if (!ok) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 25);
        break;
      }
      tc_fence_after();
      float s[BN];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32(lane_addr + Cfg::S_COL + (2 * t + buf) * BN + c0, &s[c0]);
      const int key0 = kv0 + j * BN;
      const bool unmasked = tile_full && key0 + BN - 1 <= qpos_min && key0 >= kv_begin && key0 + BN <= kv_end &&
                            (p.window == 0 || key0 > qpos_max - p.window);
      if (!unmasked) {
        const int hi = row_valid ? min(qpos, kv_end - 1) : -1;                                  // last visible key
        const int lo = max(kv_begin, p.window > 0 ? qpos - p.window + 1 : 0);                   // first visible key
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const int key = key0 + c;
          if (key > hi || key < lo) s[c] = -INFINITY;
        }
      }
      float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
      for (int c = 4; c < BN; c += 4) {
        mx0 = fmaxf(mx0, s[c]);
        mx1 = fmaxf(mx1, s[c + 1]);
        mx2 = fmaxf(mx2, s[c + 2]);
        mx3 = fmaxf(mx3, s[c + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float cand = fmaxf(m_run, mx * p.scale_log2);
      const bool grow = cand > m_run + TC_LAZY;   // also true for the first finite maximum
      if (__any_sync(0xffffffffu, grow)) {
        const float f = m_run == -INFINITY ? 0.f : fast_exp2(m_run - cand);  // cand is finite where m_run is
        l_run *= f;
        if (j > 0) {
          // (the scores of stage j were issued after P V of stage j - 2 and its commit, so that
          // arrival is in: the barrier is in phase j - 1 or j, and the parity names the right one)
          ok = wait_all(pv_done(t), (j - 1) & 1);
          if (!ok) {
            abort_flag = 1;
            if (lane == 0) atomicExch(p.err, 27);
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            float o[32];
            tmem_ld32(lane_addr + Cfg::O_COL + t * D + c0, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= f;
            tmem_st32(lane_addr + Cfg::O_COL + t * D + c0, o);
          }
        }
        m_run = cand;
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      uint32_t pk[BN / 2];
#pragma unroll
      for (int c = 0; c < BN; c += 4) {
        const float e0 = fast_exp2(fmaf(s[c], p.scale_log2, -m_use)), e1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_use));
        const float e2 = fast_exp2(fmaf(s[c + 2], p.scale_log2, -m_use)), e3 = fast_exp2(fmaf(s[c + 3], p.scale_log2, -m_use));
        l0 += e0;
        l1 += e1;
        l2 += e2;
        l3 += e3;
        pk[c / 2] = pack2_16<HALF>(e0, e1);
        pk[c / 2 + 1] = pack2_16<HALF>(e2, e3);
      }
      l_run += (l0 + l1) + (l2 + l3);
      if (j + 1 == n_j && kv_end - key0 < BN) {
        // Rows of the last stage past the key range may never have been written (or hold another
        // request's values): a zero weight times a stray NaN would still be a NaN.  The tile's
        // threads clear them once the stage has landed, before they announce P (all tiles write
        // the same zeros).
        const int s_last = j % NS;
        ok = wait_all(v_full(s_last), (j / NS) & 1);
        if (!ok) {
          abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 28);
          break;
        }
        const int first_bad = kv_end - key0;
        uint8_t* v = smem + Cfg::OFF_V + s_last * Cfg::KV_STAGE_BYTES;
        const int n16 = (BN - first_bad) * 8;  // 16-byte pieces per 64-column half
        for (int h = 0; h < HALVES; ++h)
          for (int i = r; i < n16; i += 128)
            *reinterpret_cast<uint4*>(v + h * Cfg::KV_HALF_BYTES + first_bad * 128 + i * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();   // the matrix unit reads these rows
      }
      // P replaces the first half of the scores' columns (every score of the row is in registers
      // by now); the scores of stage j + 2 come to these columns only after P V of this stage.
      // (Storing it 32 keys at a time behind the exponentials, with one wait at the end, was
      // measured slower: the wait is not what a stage spends its time on.)
#pragma unroll
      for (int c0 = 0; c0 < BN / 2; c0 += 32) tmem_st32u(lane_addr + Cfg::S_COL + (2 * t + buf) * BN + c0, &pk[c0]);
      tc_fence_before();     // this thread's tensor-memory accesses precede the products that follow
      // A warp may be a stage ahead of the tile's other warps (the next scores do not wait for
      // this P), so odd and even stages announce P on barriers of their own: an arrival is never
      // counted for the stage that the others still work on, and a barrier is used again only
      // after the scores of two stages on, which follow the product that waited for it.
      mbar_arrive(p_ready(t, buf));
    }
    // (not pv_done: a thread that never had to rescale has not followed its phases, and the
    // product of the stage before the last may still be running)
    if (ok) ok = wait_all(o_done(t), 0);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.err, 26);
    } else {
      tc_fence_after();
      const bool whole = n_splits == 1;
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      uint16_t* orow = p.out + (size_t)(qs + tok_in_req) * p.ldo + (size_t)(kvh * G + r % G) * D;
      const size_t prow = (size_t)part * (NT * tok * G) + t * tok * G + r;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float o[32];
        tmem_ld32(lane_addr + Cfg::O_COL + t * D + c0, o);  // every lane takes part in the load
        if (!row_valid) continue;
        if (whole) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = pack2_16<HALF>(o[c] * inv, o[c + 1] * inv);
            v.y = pack2_16<HALF>(o[c + 2] * inv, o[c + 3] * inv);
            v.z = pack2_16<HALF>(o[c + 4] * inv, o[c + 5] * inv);
            v.w = pack2_16<HALF>(o[c + 6] * inv, o[c + 7] * inv);
            *reinterpret_cast<uint4*>(orow + c0 + c) = v;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(p.part_o + prow * D + c0 + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
        }
      }
      if (!whole && row_valid) {
        p.part_ml[prow * 2] = m_run;
        p.part_ml[prow * 2 + 1] = l_run;
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // let TMA copies that were already issued land before the CTA's shared memory goes away
    const long long t0c = clock64();
    while (clock64() - t0c < 2000000LL) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ the CTA-pair kernel (head size 128)
// Two CTAs of a cluster take the two row tiles of an item, one each, and every product is ONE
// tcgen05.mma.cta_group::2 over both (M = 256):
//   S = Q K^T   Q sits in tensor memory (each CTA's own 128 rows, written there once per item),
//               and the 128 keys of a stage are split between the CTAs' shared memories (64 each)
//   O += P V    P in tensor memory as before, V split by columns: each CTA stages all 128 keys
//               of its 64 of the 128 value columns
// so an instruction fetches 2 KB per CTA from shared memory for 512 KFLOP of that CTA's rows
// (6 KB for 262 KFLOP above), each CTA loads half of every stage's keys and values by TMA (no
// multicast: the halves are different data), and a stage is 128 keys.  Tensor memory per CTA:
// two score buffers of 128 columns, O in 128, Q in 64.  The leader issues all products and commits
// to both CTAs' barriers; the peers' threads announce P on the leader's barriers.
//
// Measured on a B200 (32 query heads on 8, 2,048 / 8,192 tokens of one request): 82 / 913 us
// against 45 / 520 us of the kernel above, so the launch below takes this kernel only on request
// (ferrum_set_attention_pair_kernel).  Per-thread clocks showed why: the matrix unit is idle for
// most of a stage in both kernels; a stage's time goes to its softmax (64 exponentials a thread at
// the special-function unit's rate, the row maximum, the P store and its wait), and here the two
// row tiles' softmax runs on two SMs in lock-step with one product stream instead of overlapping
// on one SM, while both SMs pay the per-item start (Q through registers into tensor memory).
// Halving the shared-memory operand traffic does not touch what binds.
template <int NS>
struct AttnPairConfig {
  static constexpr int D = 128, BN = 128;
  static constexpr int K_HALF_BYTES = (BN / 2) * 128;          // this CTA's 64 keys x 64 columns
  static constexpr int K_STAGE_BYTES = 2 * K_HALF_BYTES;      // ... x 128 columns
  static constexpr int V_STAGE_BYTES = BN * 128;               // all 128 keys x this CTA's 64 columns
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + NS * K_STAGE_BYTES;
  static constexpr int OFF_BARS = OFF_V + NS * V_STAGE_BYTES;
  static constexpr int N_BARS = 1 + 5 * NS + 6;
  static constexpr int SMEM_BYTES = OFF_BARS + N_BARS * 8 + 1024;
  static constexpr int S_COL = 0, O_COL = 2 * BN, Q_COL = 2 * BN + D;   // 256 + 128 + 64 columns
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 32 * 10;                      // producer, issuer, eight softmax warps (two threads per row)
  static_assert(SMEM_BYTES <= 232448, "stages do not fit shared memory");
};

template <int NS, bool HALF>
__global__ void __launch_bounds__(AttnPairConfig<NS>::THREADS, 1)
attention_tc_pair_kernel(const __grid_constant__ CUtensorMap map_kv, const uint16_t* __restrict__ q, int ldq,
                         const AttnTcParams p) {
  using Cfg = AttnPairConfig<NS>;
  constexpr int D = Cfg::D, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float row_max[2][2][128];          // [stage parity][key half][row]: what the two threads of a row tell each other
  __shared__ float row_sum[2][128];             // [key half][row]: their sums, at the end

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0: leader (row tile 0), 1: its peer (row tile 1)
  const int kvh = blockIdx.x >> 1;
  const int* wk = p.work + (size_t)blockIdx.y * 8;
  const int req = wk[0], row0 = wk[1], kv_begin = wk[2], kv_end = wk[3], n_splits = wk[4];
  if (n_splits == 0 || kv_end <= kv_begin) return;  // padding of a fixed-size work list (the same for both CTAs)
  const int part = wk[5] * p.Hkv + kvh;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::OFF_BARS;
  const uint32_t q_ready = bar_base;                                       // leader: every softmax thread of the pair has put its part of Q in place
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };            // leader: bytes of both CTAs
  auto k_empty = [&](int s) { return bar_base + 8u * (1 + NS + s); };      // every CTA: the leader's commit
  auto v_full = [&](int s) { return bar_base + 8u * (1 + 2 * NS + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (1 + 3 * NS + s); };
  auto v_landed = [&](int s) { return bar_base + 8u * (1 + 4 * NS + s); }; // every CTA: the last stage's values are there
  auto s_ready = [&](int b) { return bar_base + 8u * (1 + 5 * NS + b); };  // every CTA
  auto p_ready = [&](int b) { return bar_base + 8u * (1 + 5 * NS + 2 + b); };  // leader: every softmax thread of the pair
  const uint32_t pv_done = bar_base + 8u * (1 + 5 * NS + 4);               // every CTA
  const uint32_t o_done = bar_base + 8u * (1 + 5 * NS + 5);                // every CTA

  if (threadIdx.x == 0) {
    abort_flag = 0;
    prefetch_tensormap(&map_kv);
    mbar_init(q_ready, 16);       // one arrival per softmax warp of the pair (8 warps in each CTA)
    for (int s = 0; s < NS; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(v_landed(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_ready(b), 1);
      mbar_init(p_ready(b), 16);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_p = &abort_flag;
  auto wait_all = [&](uint32_t bar, uint32_t parity) {
    const bool got = mbar_wait(bar, parity, abort_p);
    return __all_sync(0xffffffffu, got) != 0;
  };
  pdl_wait();

  const int G = p.G, tok = p.tok;
  const int qs = p.q_start[req];
  const int q_len = p.q_start[req + 1] - qs;
  const int pos0 = p.pos0[req];
  const int tok0 = row0 / G;
  const int kv0 = kv_begin & ~(BN - 1);       // stages start on 128-key borders: whole pages
  const int n_j = (kv_end - kv0 + BN - 1) / BN;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    // Keys: this CTA's 64 of the stage's 128, all columns.  Values: all 128 keys, this CTA's 64
    // columns.  Lane i looks up page i of a stage's 128 keys one stage ahead (the lookups overlap the
    // waits instead of standing in front of every copy); the keys' pages are a part of the same list.
    const int ps = p.page_size;
    const int k_pages = (BN / 2) / ps, v_pages = BN / ps;
    const int* bt = p.block_table + (size_t)req * p.table_width;
    auto pages_of = [&](int j) {  // this lane's page of stage j; -1 (the box reads as zeros) where there is none
      if (lane >= v_pages || j >= n_j) return -1;
      const int lp = ((kv0 + j * BN) >> p.page_shift) + lane;
      const int page = lp < p.table_width ? bt[lp] : -1;
      if (page < 0 && lp * ps < kv_end && (lp + 1) * ps > kv_begin) atomicExch(p.err, 5);
      return page;
    };
    auto load_stage = [&](int j, int kv, int page) {   // page: this lane's page of the stage's values (lane < v_pages)
      const int s = j % NS;
      const uint32_t parity = ((j / NS) & 1) ^ 1;
      const uint32_t full = kv ? v_full(s) : k_full(s);
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(kv ? v_empty(s) : k_empty(s), parity, abort_p);
        if (ok && rank == 0) mbar_expect_tx(full, 2 * (kv ? Cfg::V_STAGE_BYTES : Cfg::K_STAGE_BYTES));
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      const uint32_t leader_full = map_to_cta(full, 0);
      if (kv) {
        if (lane < v_pages) {
          const int y = page < 0 ? -ps : ((page * 2 + 1) * p.Hkv + kvh) * ps;   // a negative row: the box reads as zeros
          tma_load_2d_pair(smem_base + Cfg::OFF_V + s * Cfg::V_STAGE_BYTES + lane * ps * 128, &map_kv, leader_full,
                           (int)rank * 64, y);
        }
      } else {
        const int mine = __shfl_sync(0xffffffffu, page, ((int)rank * k_pages + lane) & 31);   // the keys' pages: this CTA's half of the list
        if (lane < k_pages) {
          const int y = mine < 0 ? -ps : ((mine * 2) * p.Hkv + kvh) * ps;
          const uint32_t dst = smem_base + Cfg::OFF_K + s * Cfg::K_STAGE_BYTES + lane * ps * 128;
          tma_load_2d_pair(dst, &map_kv, leader_full, 0, y);
          tma_load_2d_pair(dst + Cfg::K_HALF_BYTES, &map_kv, leader_full, 64, y);
        }
      }
      return true;
    };
    bool ok = true;
    int page_prev = -1, page_cur = pages_of(0);
    for (int j = 0; ok && j <= n_j; ++j) {   // keys of stage j, then values of stage j - 1
      const int page_next = pages_of(j + 1);
      if (j < n_j) ok = load_stage(j, 0, page_cur);
      if (ok && j > 0) ok = load_stage(j - 1, 1, page_prev);
      page_prev = page_cur;
      page_cur = page_next;
    }
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.err, 30);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (the leader's, for both CTAs)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_qk = umma_idesc_16bit(256, BN, HALF);
      const uint32_t idesc_pv = umma_idesc_16bit(256, D, HALF) | (1u << 16);  // B (values) is MN-major
      const uint32_t q_tmem = tmem_base + Cfg::Q_COL, o_tmem = tmem_base + Cfg::O_COL;
      auto issue_qk = [&](int s, int buf) {
        const uint32_t k_addr = smem_base + Cfg::OFF_K + s * Cfg::K_STAGE_BYTES;
        const uint32_t s_tmem = tmem_base + Cfg::S_COL + buf * BN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {  // 16 elements of the head on: 8 columns of Q, 32 bytes of a key row
          const int h = kk >> 2, in = kk & 3;
          umma_16bit_pair_ts(s_tmem, q_tmem + kk * 8, umma_desc_k_sw128(k_addr + h * Cfg::K_HALF_BYTES) + (uint64_t)(in * 2),
                             idesc_qk, kk > 0);
        }
      };
      auto issue_pv = [&](int s, int buf, bool accumulate) {
        const uint32_t v_addr = smem_base + Cfg::OFF_V + s * Cfg::V_STAGE_BYTES;
        const uint32_t p_tmem = tmem_base + Cfg::S_COL + buf * BN;  // P lies over the scores it came from
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)  // 16 keys on: 8 columns of P, 16 rows of V
          umma_16bit_pair_ts(o_tmem, p_tmem + kk * 8, umma_desc_mn_sw128(v_addr + kk * 16 * 128, Cfg::V_STAGE_BYTES, 1024),
                             idesc_pv, accumulate || kk > 0);
      };
      bool ok = mbar_wait_cluster(q_ready, 0, abort_p);
      int code = 32;
      for (int jj = 0; ok && jj < 2 && jj < n_j; ++jj) {
        ok = mbar_wait(k_full(jj % NS), (jj / NS) & 1, abort_p);
        if (!ok) break;
        tc_fence_after();
        issue_qk(jj % NS, jj);
        umma_commit_pair(s_ready(jj), 3);
        umma_commit_pair(k_empty(jj % NS), 3);
      }
      for (int j = 0; ok && j < n_j; ++j) {
        const int s = j % NS;
        const int jn = j + 2;
        const bool more = jn < n_j;
        const int s2 = jn % NS;
        ok = mbar_wait(v_full(s), (j / NS) & 1, abort_p);
        if (!ok) {
          code = 33;
          break;
        }
        if (j + 1 == n_j) umma_commit_pair(v_landed(s), 3);   // the CTAs may clear the rows past the last key
        ok = mbar_wait_cluster(p_ready(j & 1), (j >> 1) & 1, abort_p);
        if (!ok) {
          code = 34;
          break;
        }
        tc_fence_after();
        issue_pv(s, j & 1, j > 0);
        umma_commit_pair(pv_done, 3);
        if (j + 1 == n_j) umma_commit_pair(o_done, 3);
        umma_commit_pair(v_empty(s), 3);
        if (more) {
          ok = mbar_wait(k_full(s2), (jn / NS) & 1, abort_p);
          if (!ok) {
            code = 33;
            break;
          }
          tc_fence_after();
          issue_qk(s2, j & 1);
          umma_commit_pair(s_ready(j & 1), 3);
          umma_commit_pair(k_empty(s2), 3);
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicExch(p.err, code);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax and output: two threads per row of this CTA's tile
    // Warps 2..5 take the first 64 keys of every stage, warps 6..9 the other 64 (a warp reaches the
    // 32 lanes of tensor memory that its number modulo 4 names, so warps w and w + 4 share rows).
    // The two threads of a row agree on the row's maximum through shared memory once per stage;
    // each keeps the sum of its own keys, and they split the columns of O between them.
    const int t = (int)rank;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;             // which 64 keys of a stage, which 64 columns of O
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int tok_in_req = tok0 + t * tok + r / G;
    const bool row_valid = r < tok * G && tok_in_req < q_len;
    const int qpos = pos0 + tok_in_req;
    const int tile_first = tok0 + t * tok;
    const int qpos_min = pos0 + tile_first;
    const int qpos_max = pos0 + min(q_len - 1, tile_first + tok - 1);
    const bool tile_full = tok * G == 128 && tile_first + tok <= q_len;
    const uint32_t leader_q_ready = map_to_cta(q_ready, 0);
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };  // the two warps of these rows
    constexpr int HB = BN / 2;                    // keys of a stage per thread
    // ---- this row of Q into tensor memory: this thread's 64 of the 128 elements = 32 columns of two
    {
      uint32_t qw[32];
      const uint4* src = reinterpret_cast<const uint4*>(q + (size_t)(qs + (row_valid ? tok_in_req : 0)) * ldq +
                                                        (size_t)(kvh * G + r % G) * D + half * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 v = row_valid ? src[i] : make_uint4(0, 0, 0, 0);
        qw[4 * i] = v.x; qw[4 * i + 1] = v.y; qw[4 * i + 2] = v.z; qw[4 * i + 3] = v.w;
      }
      tmem_st32u(lane_addr + Cfg::Q_COL + half * 32, qw);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_q_ready);   // (one arrival a warp: a peer's arrivals cross to the leader's SM)
    }
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_j; ++j) {
      const int buf = j & 1;
      ok = wait_all(s_ready(buf), (j >> 1) & 1);
      if (!ok) {
        abort_flag = 1;
        if (lane == 0) atomicExch(p.err, 35);
        break;
      }
      tc_fence_after();
      float s[HB];
#pragma unroll
      for (int c0 = 0; c0 < HB; c0 += 32) tmem_ld32(lane_addr + Cfg::S_COL + buf * BN + half * HB + c0, &s[c0]);
      const int key0 = kv0 + j * BN;
      const bool unmasked = tile_full && key0 + BN - 1 <= qpos_min && key0 >= kv_begin && key0 + BN <= kv_end &&
                            (p.window == 0 || key0 > qpos_max - p.window);
      if (!unmasked) {
        const int hi = row_valid ? min(qpos, kv_end - 1) : -1;
        const int lo = max(kv_begin, p.window > 0 ? qpos - p.window + 1 : 0);
#pragma unroll
        for (int c = 0; c < HB; ++c) {
          const int key = key0 + half * HB + c;
          if (key > hi || key < lo) s[c] = -INFINITY;
        }
      }
      float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
      for (int c = 4; c < HB; c += 4) {
        mx0 = fmaxf(mx0, s[c]);
        mx1 = fmaxf(mx1, s[c + 1]);
        mx2 = fmaxf(mx2, s[c + 2]);
        mx3 = fmaxf(mx3, s[c + 3]);
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      row_max[buf][half][r] = mx;
      pair_sync();
      mx = fmaxf(mx, row_max[buf][half ^ 1][r]);
      const float cand = fmaxf(m_run, mx * p.scale_log2);
      const bool grow = cand > m_run + TC_LAZY;     // the same in both threads of the row: they share mx and m_run
      if (__any_sync(0xffffffffu, grow)) {
        const float f = m_run == -INFINITY ? 0.f : fast_exp2(m_run - cand);
        l_run *= f;
        if (j > 0) {
          ok = wait_all(pv_done, (j - 1) & 1);
          if (!ok) {
            abort_flag = 1;
            if (lane == 0) atomicExch(p.err, 37);
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D / 2; c0 += 32) {
            float o[32];
            tmem_ld32(lane_addr + Cfg::O_COL + half * (D / 2) + c0, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= f;
            tmem_st32(lane_addr + Cfg::O_COL + half * (D / 2) + c0, o);
          }
        }
        m_run = cand;
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      uint32_t pk[HB / 2];
#pragma unroll
      for (int c = 0; c < HB; c += 4) {
        const float e0 = fast_exp2(fmaf(s[c], p.scale_log2, -m_use)), e1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_use));
        const float e2 = fast_exp2(fmaf(s[c + 2], p.scale_log2, -m_use)), e3 = fast_exp2(fmaf(s[c + 3], p.scale_log2, -m_use));
        l0 += e0;
        l1 += e1;
        l2 += e2;
        l3 += e3;
        pk[c / 2] = pack2_16<HALF>(e0, e1);
        pk[c / 2 + 1] = pack2_16<HALF>(e2, e3);
      }
      l_run += (l0 + l1) + (l2 + l3);
      if (j + 1 == n_j && kv_end - key0 < BN) {
        // rows of the last stage past the key range may hold anything: cleared in this CTA's half of
        // the values once the stage has landed (the leader says so), before P is announced
        const int s_last = j % NS;
        ok = wait_all(v_landed(s_last), 0);
        if (!ok) {
          abort_flag = 1;
          if (lane == 0) atomicExch(p.err, 38);
          break;
        }
        const int first_bad = kv_end - key0;
        uint8_t* v = smem + Cfg::OFF_V + s_last * Cfg::V_STAGE_BYTES;
        const int n16 = (BN - first_bad) * 8;
        for (int i = half * 128 + r; i < n16; i += 256) *reinterpret_cast<uint4*>(v + first_bad * 128 + i * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
      }
      // P (two values a column) over the first half of the stage's score columns: this thread's 32 of the 64
      tmem_st32u(lane_addr + Cfg::S_COL + buf * BN + half * (HB / 2), pk);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(p_ready(buf), 0));
    }
    if (ok) ok = wait_all(o_done, 0);
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicExch(p.err, 36);
    } else {
      tc_fence_after();
      // the row's sum is the two threads' sums
      row_sum[half][r] = l_run;
      pair_sync();
      const float l_row = l_run + row_sum[half ^ 1][r];
      const bool whole = n_splits == 1;
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      uint16_t* orow = p.out + (size_t)(qs + tok_in_req) * p.ldo + (size_t)(kvh * G + r % G) * D + half * (D / 2);
      const size_t prow = (size_t)part * (2 * tok * G) + t * tok * G + r;
#pragma unroll 1
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        float o[32];
        tmem_ld32(lane_addr + Cfg::O_COL + half * (D / 2) + c0, o);
        if (!row_valid) continue;
        if (whole) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v;
            v.x = pack2_16<HALF>(o[c] * inv, o[c + 1] * inv);
            v.y = pack2_16<HALF>(o[c + 2] * inv, o[c + 3] * inv);
            v.z = pack2_16<HALF>(o[c + 4] * inv, o[c + 5] * inv);
            v.w = pack2_16<HALF>(o[c + 6] * inv, o[c + 7] * inv);
            *reinterpret_cast<uint4*>(orow + c0 + c) = v;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(p.part_o + prow * D + half * (D / 2) + c0 + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
        }
      }
      if (!whole && row_valid && half == 0) {
        p.part_ml[prow * 2] = m_run;
        p.part_ml[prow * 2 + 1] = l_row;
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    const long long t0c = clock64();
    while (clock64() - t0c < 2000000LL) {
    }
  }
  // neither CTA may leave while the other can still signal its barriers or read its tensor memory
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

struct AttnMapKey {
  const void* ptr;
  long long a, b, c;
  int kind;
  bool operator==(const AttnMapKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c && kind == o.kind; }
};
struct AttnMapKeyHash {
  size_t operator()(const AttnMapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long long>()(k.a);
    h = h * 1000003u ^ std::hash<long long>()(k.b);
    h = h * 1000003u ^ std::hash<long long>()(k.c * 2 + k.kind);
    return h;
  }
};
std::mutex g_map_mu;
std::unordered_map<AttnMapKey, CUtensorMap, AttnMapKeyHash> g_maps;

bool lookup_map(const AttnMapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> g(g_map_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) return false;
  *out = it->second;
  return true;
}
void keep_map(const AttnMapKey& key, const CUtensorMap& m) {
  std::lock_guard<std::mutex> g(g_map_mu);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
}

// Queries [rows, ld] bfloat16 seen as (D, Hq, rows); a box is 64 columns x G heads x tok tokens.
int query_map(const void* q, long long rows, int ldq, int Hq, int D, int G, int tok, CUtensorMap* out) {
  AttnMapKey key{q, rows, (long long)ldq * 4096 + D, (long long)Hq * 65536 + G * 256 + tok, 0};
  if (lookup_map(key, out)) return 0;
  EncodeTiledFn fn = encode_fn();
  FERRUM_CHECK_ARG(fn != nullptr, "attention_tc: the driver does not export cuTensorMapEncodeTiled");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Hq, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)ldq * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)tok};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FERRUM_CHECK_ARG(r == CUDA_SUCCESS, "attention_tc: encoding the query map failed with code %d", (int)r);
  keep_map(key, *out);
  return 0;
}

// The cache plane [pages, 2, Hkv, page_size, D] seen as rows of D; a box is 64 columns x one page of one head.
int cache_map(const void* plane, long long n_pages, int Hkv, int page_size, int D, CUtensorMap* out) {
  AttnMapKey key{plane, n_pages, (long long)Hkv * 65536 + page_size, D, 1};
  if (lookup_map(key, out)) return 0;
  EncodeTiledFn fn = encode_fn();
  FERRUM_CHECK_ARG(fn != nullptr, "attention_tc: the driver does not export cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)(n_pages * 2 * Hkv * page_size)};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(plane), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FERRUM_CHECK_ARG(r == CUDA_SUCCESS, "attention_tc: encoding the cache map failed with code %d", (int)r);
  keep_map(key, *out);
  return 0;
}

template <int D, int NT, int BN, int NS, bool HALF>
int launch_attention_tc(const CUtensorMap& mq, const CUtensorMap& mkv, const AttnTcParams& p, int n_work, cudaStream_t stream) {
  using Cfg = AttnTcConfig<D, NT, BN, NS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<D, NT, BN, NS, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    FERRUM_CHECK_ARG(e == cudaSuccess, "attention_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  launch_kernel(attention_tc_kernel<D, NT, BN, NS, HALF>, dim3(p.Hkv, n_work), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, mq, mkv, p);
  FERRUM_CHECK_LAUNCH("attention_tc");
  return 0;
}

template <int NS, bool HALF>
int launch_attention_tc_pair(const CUtensorMap& mkv, const void* q, int ldq, const AttnTcParams& p, int n_work, cudaStream_t stream) {
  using Cfg = AttnPairConfig<NS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_pair_kernel<NS, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    FERRUM_CHECK_ARG(e == cudaSuccess, "attention_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * p.Hkv, n_work);      // the two CTAs of a pair are neighbours in x
  cfg.blockDim = dim3(Cfg::THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ferrum_dependent_launch_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attention_tc_pair_kernel<NS, HALF>, mkv, (const uint16_t*)q, ldq, p);
  FERRUM_CHECK_ARG(e == cudaSuccess, "attention_tc: pair kernel launch failed: %s", cudaGetErrorString(e));
  FERRUM_CHECK_LAUNCH("attention_tc_pair");
  return 0;
}

bool g_attention_pair = false;

// The shape in use: two row tiles per CTA that share three stages of 64 keys.  One tile with
// stages of 128 keys (half the waits and fences per key, no second tile to fill the matrix unit
// while the first computes P) was measured slower: 67.8 against 51.8 us for a 2048-token prompt.
constexpr int TC_TILES = 2, TC_BN = 64, TC_STAGES = 3;

}  // namespace

// Head size 128 runs on CTA pairs (one row tile per CTA, see attention_tc_pair_kernel) unless this is
// switched off; the single-CTA kernel takes the same work items.
FERRUM_API void ferrum_set_attention_pair_kernel(int on) { g_attention_pair = on != 0; }

// Tokens per work item for a group of G query heads per KV head (an item is TC_TILES tiles of
// 128 / G tokens), or 0 when this kernel does not take the shape: head sizes 64 and 128; pages
// of 8 to 64 keys, a power of two; at most 128 heads per group.
FERRUM_API int ferrum_attention_tc_tokens(int D, int G, int page_size) {
  if (D != 64 && D != 128) return 0;
  if (page_size < 8 || page_size > TC_BN || (page_size & (page_size - 1)) != 0) return 0;
  if (G < 1 || G > 128) return 0;
  return TC_TILES * (128 / G);
}

// Items of ferrum_attention_tc_tokens * G rows in the work-list format of ferrum_attention_flash;
// grid (Hkv, n_work).  q has q_rows rows of ldq elements (the buffer's capacity, of which the
// batch may use fewer); the plane has n_pages pages.
FERRUM_API int ferrum_attention_tc(const void* q, int ldq, long long q_rows, void* out, int ldo, int dtype, const void* kv_plane,
                                   long long page_stride, long long n_pages, int page_size, const int* block_table,
                                   int table_width, const int* q_start, const int* pos0, const int* work, int n_work,
                                   float* part_o, float* part_ml, int Hq, int Hkv, int D, float scale, int window,
                                   int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention_tc: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
  const int G = Hq / Hkv;
  const int tok = ferrum_attention_tc_tokens(D, G, page_size) / TC_TILES;
  FERRUM_CHECK_ARG(tok > 0, "attention_tc: head size %d, group %d, page size %d is not built; use attention_flash", D, G, page_size);
  FERRUM_CHECK_ARG(err_flag != nullptr, "attention_tc: the error flag is required");
  FERRUM_CHECK_ARG(ferrum_is_16bit(dtype), "attention_tc: dtype code %d is not a 16-bit type", dtype);
  FERRUM_CHECK_ARG(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                   ((uintptr_t)kv_plane & 15) == 0, "attention_tc: operands must be 16-byte aligned");
  FERRUM_CHECK_ARG(page_stride == 2LL * Hkv * page_size * D, "attention_tc: the plane's pages must be dense "
                   "(stride %lld, expected %lld)", page_stride, 2LL * Hkv * page_size * D);
  FERRUM_CHECK_ARG(n_pages > 0 && n_pages * 2 * Hkv * page_size < (1LL << 31), "attention_tc: %lld pages are more than the "
                   "row index of the cache map holds", n_pages);
  FERRUM_CHECK_ARG(table_width > 0 && window >= 0 && n_work >= 0 && q_rows > 0, "attention_tc: bad arguments");
  if (n_work == 0) return 0;
  FERRUM_CHECK_ARG(n_work <= 65535, "attention_tc: %d work items are more than one launch takes", n_work);
  AttnTcParams p;
  p.out = (uint16_t*)out; p.block_table = block_table; p.q_start = q_start; p.pos0 = pos0; p.work = work;
  p.part_o = part_o; p.part_ml = part_ml; p.err = err_flag;
  p.ldo = ldo; p.page_size = page_size; p.table_width = table_width;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.Hkv = Hkv; p.G = G; p.tok = tok; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap mq, mkv;
  if (int r = cache_map(kv_plane, n_pages, Hkv, page_size, D, &mkv)) return r;
  if (D == 128 && g_attention_pair) {
    if (dtype == FERRUM_F16) return launch_attention_tc_pair<3, true>(mkv, q, ldq, p, n_work, stream);
    return launch_attention_tc_pair<3, false>(mkv, q, ldq, p, n_work, stream);
  }
  if (int r = query_map(q, q_rows, ldq, Hq, D, G, tok, &mq)) return r;
  if (dtype == FERRUM_F16) {
    if (D == 64) return launch_attention_tc<64, TC_TILES, TC_BN, TC_STAGES, true>(mq, mkv, p, n_work, stream);
    return launch_attention_tc<128, TC_TILES, TC_BN, TC_STAGES, true>(mq, mkv, p, n_work, stream);
  }
  if (D == 64) return launch_attention_tc<64, TC_TILES, TC_BN, TC_STAGES, false>(mq, mkv, p, n_work, stream);
  return launch_attention_tc<128, TC_TILES, TC_BN, TC_STAGES, false>(mq, mkv, p, n_work, stream);
}
