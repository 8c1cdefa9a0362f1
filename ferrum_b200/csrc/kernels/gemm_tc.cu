// 16-bit (bfloat16 or float16) matrix product on the tcgen05 tensor cores: out[t, n] = sum_k x[t, k] * w[n, k],
// float32 accumulation.  The two types differ in the instruction descriptor's operand format and in
// how the epilogue rounds; everything else (tensor maps, tiles, schedules) moves 16-bit elements.
//
// Orientation: the weight rows are the M side of the instruction (128 rows of W per tile,
// one row per TMEM lane) and the tokens are the N side (BT columns, 16..256).  The same
// kernel therefore serves a 2048-token prompt (BT = 256) and a single decoded token
// (BT = 16): in decode the tensor cores idle and every CTA is a TMA streaming engine for
// its share of the weights.  Both operands are K-major tiles of 64 bfloat16 per row, brought
// in by TMA with the 128-byte swizzle into a ring of stages; one thread issues the MMAs, the
// accumulators live in tensor memory, four warps read them back for the epilogue.
//
// Persistent, stream-K: the work is the line of all (tile, k-block) units, tile-major.  The
// grid is one CTA per SM and CTA c owns the contiguous units [c*U/P, (c+1)*U/P), so every SM
// streams the same number of bytes whatever the shape.  A CTA's range is a sequence of
// segments, one per tile it touches.  A segment that covers the whole K of its tile ends in
// the epilogue proper; a partial one writes its float32 accumulator to the workspace and
// bumps the tile's counter, and the CTA that arrives last adds the partials in K order (so
// the sum does not depend on arrival order) and runs the epilogue.  Nobody waits for anybody.
// Counters are left at zero for the next launch.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA issuer, warps
// 2..5 = epilogue.  Two accumulators in tensor memory let segment i+1 be computed while
// segment i is read back.  DUAL computes two products per segment, from weight rows n and
// dual_offset + n against the same tokens; the SwiGLU epilogue combines them, so gate and up
// need no interleaving in memory.
//
// Every mbarrier wait is bounded; on a timeout the kernel raises the error flag, lets the
// copies in flight land, frees its tensor memory and returns.
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

enum TcEpilogue : int {
  TC_STORE_BF16 = 0,  // out 16-bit [M, ldo] = acc   (the operands' type)
  TC_STORE_F32 = 1,   // out f32  [M, ldo] = acc
  TC_RESIDUAL = 2,    // out f32  [M, ldo] += acc
  TC_SWIGLU = 3,      // out 16-bit [M, ldo] = silu(acc0) * acc1   (DUAL only)
};

struct TcParams {
  void* out;
  float* workspace;
  int* counters;
  int* err;
  int M, N, K, ldo;
  int epilogue;
  int dual_offset;   // row of the second weight tile relative to the first (DUAL)
  int defer;         // 1: leave every segment's float32 partial in the workspace; the next kernel sums them
  int out_tma;       // 1: the pair kernel writes `out` through its tensor map (staged in shared memory)
  int stream_weights;  // 1: every weight tile is read once in this launch: its L2 lines are the first to go
  int gated;           // 1 (pair kernel): weight rows come interleaved (gate i, up i, gate i + 1, ...), N counts these
                       // rows, and the epilogue writes silu(gate) * up for N / 2 features
  int half;            // 0: operands and 16-bit outputs are bfloat16; 1: float16
  long long wait_cycles;  // limit of every mbarrier wait (0: the default of about a second); tests shorten it
  int drop_loads;      // test hook: the producer requests no tile at all, so that the waits for them run out
};

constexpr int TILE_N = 128;  // weight rows per tile (the instruction's M)
constexpr int TILE_K = 64;   // bfloat16 per row of a stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_BYTES = TILE_N * TILE_K * 2;

template <int BT, bool DUAL>
struct TcConfig {
  static constexpr int B_BYTES = BT * TILE_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  // few tokens: the CTA is a streaming engine and half the shared memory leaves room for a
  // second CTA on the SM (the next launch's, see the dependent-launch prologue)
  static constexpr int BUDGET = 196 * 1024;
  static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 10 ? 10 : (BUDGET / STAGE_BYTES);
  static constexpr int ACC_COLS = BT * (DUAL ? 2 : 1);
  static constexpr int ALL_COLS = 2 * ACC_COLS;  // two accumulators
  static constexpr int TMEM_COLS = ALL_COLS <= 32 ? 32 : (ALL_COLS <= 64 ? 64 : (ALL_COLS <= 128 ? 128 : (ALL_COLS <= 256 ? 256 : 512)));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(STAGES >= 2, "tile too large for the shared memory budget");
  static_assert(ALL_COLS <= 512, "accumulators do not fit tensor memory");
};

// Epilogue of 16 token columns t_base..t_base+15 of feature n.  Loads come first and
// stores last, so that the 16 read-modify-writes of the residual overlap instead of
// queueing behind each other.
__device__ __forceinline__ void tc_apply16(const TcParams& p, int t_base, int n, const float (&a0)[16], const float (&a1)[16]) {
  const int valid = p.M - t_base;  // columns j < valid exist
  if (valid <= 0) return;
  const size_t o = (size_t)t_base * p.ldo + n;
  const size_t ld = (size_t)p.ldo;
  switch (p.epilogue) {
    case TC_STORE_BF16: {
      uint16_t* out = (uint16_t*)p.out + o;
      const bool half = p.half != 0;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < valid) out[j * ld] = bits16(a0[j], half);
      break;
    }
    case TC_STORE_F32: {
      float* out = (float*)p.out + o;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < valid) out[j * ld] = a0[j];
      break;
    }
    case TC_RESIDUAL: {
      float* out = (float*)p.out + o;
      float r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = j < valid ? out[j * ld] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < valid) out[j * ld] = r[j] + a0[j];
      break;
    }
    case TC_SWIGLU: {
      uint16_t* out = (uint16_t*)p.out + o;
      const bool half = p.half != 0;
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < valid) out[j * ld] = bits16(a0[j] / (1.0f + __expf(-a0[j])) * a1[j], half);
      break;
    }
  }
}

// The CTA that owns unit u when CTA c owns [c*U/P, (c+1)*U/P).
__host__ __device__ __forceinline__ int unit_owner(long long u, long long U, int P) {
  return (int)(((u + 1) * P + U - 1) / U) - 1;
}

template <int BT, bool DUAL>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const TcParams p) {
  using Cfg = TcConfig<BT, DUAL>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::STAGE_BYTES);  // full[S], empty[S], acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = gridDim.x, cta = blockIdx.x;
  const int nkb = (p.K + TILE_K - 1) / TILE_K;
  const int tiles_n = (p.N + TILE_N - 1) / TILE_N;
  const int tiles_t = (p.M + BT - 1) / BT;
  const long long U = (long long)tiles_n * tiles_t * nkb;
  const long long u_begin = U * cta / P, u_end = U * (cta + 1) / P;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };

  TRACE_BEGIN(threadIdx.x == 0 && blockIdx.x == 0, TRACE_GEMM + (p.N / 64) * 16 + (DUAL ? 8 : 0));
  if (threadIdx.x == 0) {
    abort_flag = 0;
    is_last = 0;
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);  // one arrival per epilogue warp
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
  const long long wait_limit = p.wait_cycles > 0 ? p.wait_cycles : WAIT_LIMIT_CYCLES;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && p.drop_loads) {
      // (test hook) nothing is requested, nothing will be in flight: the other roles' waits run out
      pdl_wait();
      pdl_launch();
    } else if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      long long tile = u_begin / nkb;
      int kb = (int)(u_begin % nkb);
      const bool stream_w = p.stream_weights != 0;
      auto load_w = [&](uint32_t dst, uint32_t bar, int x, int y) {
        if (stream_w) tma_load_2d_hint(dst, &tmap_w, bar, x, y, L2_EVICT_FIRST);
        else tma_load_2d(dst, &tmap_w, bar, x, y);
      };
      // The weights never change, so the first ring of weight tiles is requested before the
      // kernel ahead of this one in the stream has finished; the activations it writes are
      // requested after the dependency wait.
      const int pre = (int)min((long long)STAGES, u_end - u_begin);
      {
        long long tl = tile;
        int k = kb;
        for (int i = 0; i < pre; ++i) {
          const uint32_t a = smem_base + i * Cfg::STAGE_BYTES;
          mbar_expect_tx(full_bar(i), Cfg::STAGE_BYTES);
          load_w(a, full_bar(i), k * TILE_K, (int)(tl % tiles_n) * TILE_N);
          if (DUAL) load_w(a + A_BYTES, full_bar(i), k * TILE_K, p.dual_offset + (int)(tl % tiles_n) * TILE_N);
          if (++k == nkb) {
            k = 0;
            ++tl;
          }
        }
      }
      pdl_wait();
      TRACE_MARK(TRACE_WAITED);
      pdl_launch();
      for (int i = 0; i < pre; ++i) {
        const uint32_t a = smem_base + i * Cfg::STAGE_BYTES;
        tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), &tmap_x, full_bar(i), kb * TILE_K, (int)(tile / tiles_n) * BT);
        if (++kb == nkb) {
          kb = 0;
          ++tile;
        }
      }
      s = pre % STAGES;
      phase = pre == STAGES ? 1 : 0;
      for (long long u = u_begin + pre; u < u_end; ++u) {
        if (!mbar_wait(empty_bar(s), phase ^ 1, abort_p, wait_limit)) {
          abort_flag = 1;
          atomicExch(p.err, 10);
          break;
        }
        const int n0 = (int)(tile % tiles_n) * TILE_N, t0 = (int)(tile / tiles_n) * BT;
        const uint32_t a = smem_base + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
        load_w(a, full_bar(s), kb * TILE_K, n0);
        if (DUAL) load_w(a + A_BYTES, full_bar(s), kb * TILE_K, p.dual_offset + n0);
        tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), &tmap_x, full_bar(s), kb * TILE_K, t0);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
        if (++kb == nkb) {
          kb = 0;
          ++tile;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_16bit(TILE_N, BT, p.half != 0);
      int s = 0;
      uint32_t phase = 0;
      int seg = 0;
      long long u = u_begin;
      bool ok = true;
      while (ok && u < u_end) {
        const long long tile = u / nkb;
        const long long seg_end = min(u_end, (tile + 1) * (long long)nkb);
        const int buf = seg & 1, use = seg >> 1;
        if (!mbar_wait(acc_empty_bar(buf), (use & 1) ^ 1, abort_p, wait_limit)) {
          abort_flag = 1;
          atomicExch(p.err, 13);
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * Cfg::ACC_COLS;
        bool first = true;
        for (; u < seg_end; ++u) {
          if (!mbar_wait(full_bar(s), phase, abort_p, wait_limit)) {
            abort_flag = 1;
            atomicExch(p.err, 11);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_base + s * Cfg::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a);
          const uint64_t a2_desc = umma_desc_k_sw128(a + A_BYTES);
          const uint64_t b_desc = umma_desc_k_sw128(a + A_BYTES * (DUAL ? 2 : 1));
#pragma unroll
          for (int kk = 0; kk < TILE_K / UMMA_K; ++kk) {
            const bool acc = !first || kk > 0;
            const uint64_t adv = (uint64_t)(kk * UMMA_K * 2 >> 4);  // 32 bytes per step, in 16-byte units
            umma_bf16(d0, a_desc + adv, b_desc + adv, idesc, acc);
            if (DUAL) umma_bf16(d0 + BT, a2_desc + adv, b_desc + adv, idesc, acc);
          }
          first = false;
          umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(acc_full_bar(buf));
        ++seg;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32*quarter .. +31
    const int n_local = quarter * 32 + lane;
    const int ep_tid = threadIdx.x - 64;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t tile_floats = (size_t)Cfg::ACC_COLS * TILE_N;
    int seg = 0;
    long long u = u_begin;
    pdl_wait();  // the epilogue reads and writes what earlier kernels of the stream wrote
    while (u < u_end) {
      const long long tile = u / nkb;
      const int kb0 = (int)(u % nkb);
      const long long seg_end = min(u_end, (tile + 1) * (long long)nkb);
      const bool whole = kb0 == 0 && seg_end == (tile + 1) * (long long)nkb;
      const int buf = seg & 1, use = seg >> 1;
      bool ok = mbar_wait(acc_full_bar(buf), use & 1, abort_p, wait_limit);
      if (!ok) abort_flag = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four warps agree on going on
      if (abort_flag) {
        if (ep_tid == 0) atomicExch(p.err, 12);
        break;
      }
      tc_fence_after();
      const int n0 = (int)(tile % tiles_n) * TILE_N, t0 = (int)(tile / tiles_n) * BT;
      const int n = n0 + n_local;
      const uint32_t acc_addr = lane_addr + buf * Cfg::ACC_COLS;
      if (whole && !p.defer) {
#pragma unroll 1
        for (int c0 = 0; c0 < BT; c0 += 16) {
          float v0[16], v1[16];
          tmem_ld16(acc_addr + c0, v0);
          if (DUAL) tmem_ld16(acc_addr + BT + c0, v1);
          if (n < p.N) tc_apply16(p, t0 + c0, n, v0, DUAL ? v1 : v0);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(buf));
      } else {
        // partial tile -> workspace [cta][slot][column][lane]; a CTA has at most two partial
        // segments: slot 0 if the segment lies in the tile where its range begins, else slot 1
        const int c_first = unit_owner(tile * nkb, U, P), c_last = unit_owner(tile * nkb + nkb - 1, U, P);
        const int n_contrib = c_last - c_first + 1;
        float* ws = p.workspace + ((size_t)cta * 2 + (u_begin / nkb == tile ? 0 : 1)) * tile_floats;
#pragma unroll 1
        for (int c0 = 0; c0 < Cfg::ACC_COLS; c0 += 16) {
          float v[16];
          tmem_ld16(acc_addr + c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) ws[(size_t)(c0 + j) * TILE_N + n_local] = v[j];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        if (p.defer) {  // the kernel that reads this product adds the partials itself
          u = seg_end;
          ++seg;
          continue;
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) {
          const int old = atomicAdd(p.counters + tile, 1);
          is_last = old == n_contrib - 1;
          if (is_last) p.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (is_last) {
          __threadfence();
          if (n < p.N) {
#pragma unroll 1
            for (int c0 = 0; c0 < BT && t0 + c0 < p.M; c0 += 16) {
              float a0[16], a1[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) a0[j] = a1[j] = 0.f;
              for (int cc = c_first; cc <= c_last; ++cc) {  // K order; 16 (or 32) loads in flight per thread
                const float* wsp = p.workspace + ((size_t)cc * 2 + ((U * cc / P) / nkb == tile ? 0 : 1)) * tile_floats +
                                   (size_t)c0 * TILE_N + n_local;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  a0[j] += __ldcg(wsp + (size_t)j * TILE_N);
                  if (DUAL) a1[j] += __ldcg(wsp + (size_t)(BT + j) * TILE_N);
                }
              }
              tc_apply16(p, t0 + c0, n, a0, a1);
            }
          }
        }
      }
      u = seg_end;
      ++seg;
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
  TRACE_MARK(TRACE_EXIT);
}

// ------------------------------------------------------------------ the CTA-pair kernel
// For many tokens the single-CTA tile (128 weight rows x 256 tokens) asks the L2 for 48 KB
// per 4.2 MFLOP and the tensor cores wait for operands half of the time.  Here two CTAs of a
// cluster compute a 256 x 256 tile with one tcgen05.mma.cta_group::2 per K step: each CTA
// loads its own 128 weight rows and its own 128 tokens (32 KB per stage instead of 48 KB for
// the same flops), the leader issues the MMAs, and each CTA's tensor memory receives its 128
// rows of the product, which its own epilogue warps read back.  Partial tiles are handled as
// in the single-CTA kernel with the cluster in the role of the CTA and the 128-row half tile
// in the role of the tile.  No multicast loads are used.
// Which parts of which tiles a cluster computes.  Whole waves first: in wave w cluster c takes
// tile w * P + c with all its k-blocks and writes it out itself, so neighbouring clusters work
// on neighbouring tiles at the same k-block and share their operands in the L2.  For the R
// tiles that are left (fewer than P) there are two ways.  As a rule R clusters take one more
// whole tile each and the others are done.  Only where that idles much (long tiles, few of
// them: (P - R) / P of a tile is PAIR_STREAMK_MIN_KB k-blocks or more) the left-over tiles are cut
// stream-K fashion: their units (tile, k-block) form a line that is divided evenly among the
// first Pr clusters, and a tile that several clusters share is summed from float32 partials
// by the cluster that holds its first k-blocks.  That costs some 20 us at the end of the
// kernel (partials out, a wait, partials in), which is why short tiles are not cut: measured
// on 2048 x [4096, 14336], cutting 54 left-over tiles of 224 k-blocks (60 k-blocks saved)
// gains nothing, on 512 x [4096, 14336] (127 saved) it takes 74 us to 60.  Tiles are numbered through groups of
// PAIR_GROUP_T token tiles, token tile fastest: a wave then reads about P / 8 weight tiles and
// 8 token tiles instead of P weight tiles and one token tile, and with many tokens the
// weights stream from memory once per group instead of once per token tile.
constexpr int PAIR_GROUP_T = 8;
constexpr int PAIR_STREAMK_MIN_KB = 80;
constexpr int PAIR_FINISHER_POLLS = 200;  // of about a microsecond each: how long a tile's finisher waits for the other partials
struct PairSchedule {
  int nkb, tiles_n, tiles_t, P, cluster, waves, Pr, whole_extra;
  long long full_tiles, Ur, r_begin, r_end;
  __host__ __device__ PairSchedule(int tiles_n_, int tiles_t_, int nkb_, int P_, int cluster_)
      : nkb(nkb_), tiles_n(tiles_n_), tiles_t(tiles_t_), P(P_), cluster(cluster_) {
    const long long tiles = (long long)tiles_n * tiles_t;
    const int R = (int)(tiles % P);
    waves = (int)(tiles / P);
    whole_extra = 0;
    Ur = 0;
    Pr = 0;
    r_begin = r_end = 0;
    if (R > 0 && (long long)(P - R) * nkb < (long long)PAIR_STREAMK_MIN_KB * P) {
      whole_extra = R;
    } else if (R > 0) {
      // few tiles left over would each be cut among many clusters: cut the last whole wave with them
      if (waves > 0 && 2 * R < P) --waves;
      Ur = (tiles - (long long)waves * P) * nkb;
      Pr = (int)(Ur < P ? Ur : P);   // every sharing cluster owns at least one unit
      r_begin = cluster < Pr ? Ur * cluster / Pr : 0;
      r_end = cluster < Pr ? Ur * (cluster + 1) / Pr : 0;
    }
    full_tiles = (long long)waves * P;
  }
  // this cluster's s-th segment: its tile and k-blocks [kb0, kb1); false when there is none
  __host__ __device__ bool segment(int s, long long& tile, int& kb0, int& kb1) const {
    if (s < waves) {
      tile = (long long)s * P + cluster;
      kb0 = 0;
      kb1 = nkb;
      return true;
    }
    if (whole_extra > 0) {
      if (s > waves || cluster >= whole_extra) return false;
      tile = full_tiles + cluster;
      kb0 = 0;
      kb1 = nkb;
      return true;
    }
    const int r = s - waves;
    const long long rt = r_begin / nkb + r;  // tile of the remainder
    if (rt * nkb >= r_end) return false;
    tile = full_tiles + rt;
    kb0 = r == 0 ? (int)(r_begin % nkb) : 0;
    kb1 = (int)(r_end - rt * nkb < nkb ? r_end - rt * nkb : nkb);
    return true;
  }
  __host__ __device__ void coords(long long tile, int& n_idx, int& t_idx) const {
    const long long per_group = (long long)PAIR_GROUP_T * tiles_n;
    const int g = (int)(tile / per_group);
    const int t_first = g * PAIR_GROUP_T;
    const int gt = tiles_t - t_first < PAIR_GROUP_T ? tiles_t - t_first : PAIR_GROUP_T;
    const int r = (int)(tile - g * per_group);
    t_idx = t_first + r % gt;
    n_idx = r / gt;
  }
  // the clusters that share a tile of the remainder, and the slot (0: the tile in which the
  // cluster's range begins, 1: the other) in which cluster cc leaves its partial of it
  __host__ __device__ int first_owner(long long tile) const { return unit_owner((tile - full_tiles) * nkb, Ur, Pr); }
  __host__ __device__ int last_owner(long long tile) const { return unit_owner((tile - full_tiles) * nkb + nkb - 1, Ur, Pr); }
  __host__ __device__ int slot_of(int cc, long long tile) const { return (Ur * cc / Pr) / nkb == tile - full_tiles ? 0 : 1; }
};

constexpr int PAIR_BT = 256;                              // tokens per tile pair
constexpr int PAIR_B_BYTES = (PAIR_BT / 2) * TILE_K * 2;  // each CTA stages half of the tokens
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_STAGES = 6;
// The epilogue's staging: two buffers of 32 tokens x 128 features (float32 at most).  A thread
// owns one feature of 32 tokens at a time; written to `out` directly that is 32 scattered
// read-modify-writes per thread and the epilogue, not the tensor cores, sets the pace of short
// products.  Staged, the tile leaves as one bulk store (or float32 add) per 32 tokens.
constexpr int PAIR_OUT_ROWS = 32;
constexpr int PAIR_OUT_BYTES = PAIR_OUT_ROWS * TILE_N * 4;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + 2 * PAIR_OUT_BYTES;

__global__ void __launch_bounds__(192, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_ws,
                    const TcParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr int ACC_COLS = PAIR_BT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * PAIR_STAGE_BYTES);  // full[S], empty[S], acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader of the pair
  const int P = gridDim.x / 2, cluster = blockIdx.x / 2;
  const int nkb = (p.K + TILE_K - 1) / TILE_K;
  const int tiles_n = (p.N + 2 * TILE_N - 1) / (2 * TILE_N);  // 256-row tiles
  const int tiles_t = (p.M + PAIR_BT - 1) / PAIR_BT;
  const PairSchedule sched(tiles_n, tiles_t, nkb, P, cluster);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t fetch_bar = bar_base + 8u * (2 * STAGES + 4);  // partials of other clusters copied into the idle stages

  if (threadIdx.x == 0) {
    abort_flag = 0;
    is_last = 0;
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
    if (p.out_tma) {
      prefetch_tensormap(&tmap_out);
      prefetch_tensormap(&tmap_ws);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // the leader's: its producer's expect_tx; bytes arrive from both CTAs
      mbar_init(empty_bar(s), 1);  // one multicast commit of the leader's MMA thread
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 8);  // the leader's: four epilogue warps of each CTA
    }
    mbar_init(fetch_bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_slot), 2 * ACC_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_p = &abort_flag;
  const long long wait_limit = p.wait_cycles > 0 ? p.wait_cycles : WAIT_LIMIT_CYCLES;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      pdl_wait();
      pdl_launch();
      long long tile;
      int kb0, kb1;
      bool ok = true;
      for (int seg = 0; ok && sched.segment(seg, tile, kb0, kb1); ++seg) {
        int n_idx, t_idx;
        sched.coords(tile, n_idx, t_idx);
        const int n0 = n_idx * 2 * TILE_N + (int)rank * TILE_N;
        const int t0 = t_idx * PAIR_BT + (int)rank * (PAIR_BT / 2);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(s), phase ^ 1, abort_p, wait_limit)) {
            abort_flag = 1;
            atomicExch(p.err, 10);
            ok = false;
            break;
          }
          const uint32_t a = smem_base + s * PAIR_STAGE_BYTES;
          const uint32_t leader_full = map_to_cta(full_bar(s), 0);  // (measured: this loop is not the limit; the copies are)
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * PAIR_STAGE_BYTES);
          if (p.gated) tma_load_3d_pair(a, &tmap_w, leader_full, kb * TILE_K, 0, n0 >> 1);  // (k, gate | up, feature)
          else tma_load_2d_pair(a, &tmap_w, leader_full, kb * TILE_K, n0);
          tma_load_2d_pair(a + A_BYTES, &tmap_x, leader_full, kb * TILE_K, t0);
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_16bit(2 * TILE_N, PAIR_BT, p.half != 0);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long tile;
      int kb0, kb1;
      for (int seg = 0; ok && sched.segment(seg, tile, kb0, kb1); ++seg) {
        const int buf = seg & 1, use = seg >> 1;
        if (!mbar_wait(acc_empty_bar(buf), (use & 1) ^ 1, abort_p, wait_limit)) {
          abort_flag = 1;
          atomicExch(p.err, 13);
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * ACC_COLS;
        bool first = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(s), phase, abort_p, wait_limit)) {
            abort_flag = 1;
            atomicExch(p.err, 11);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_base + s * PAIR_STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a);
          const uint64_t b_desc = umma_desc_k_sw128(a + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < TILE_K / UMMA_K; ++kk) {
            const uint64_t adv = (uint64_t)(kk * UMMA_K * 2 >> 4);
            umma_bf16_pair(d0, a_desc + adv, b_desc + adv, idesc, !first || kk > 0);
          }
          first = false;
          umma_commit_pair(empty_bar(s), 3);  // both CTAs may refill the stage
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_pair(acc_full_bar(buf), 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    const int n_local = quarter * 32 + lane;
    const int ep_tid = threadIdx.x - 64;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t tile_floats = (size_t)ACC_COLS * TILE_N;
    uint8_t* out_stage = smem + STAGES * PAIR_STAGE_BYTES + 256;
    const bool staged = p.out_tma != 0;
    int emitted = 0;  // staged stores issued so far; buffer = emitted & 1
    pdl_wait();
    // A staging buffer, once the bulk store that last used it has read it; and its way out:
    // through a tensor map (which clips at the tensor's edges), as a store or a float32 add.
    auto stage_acquire = [&]() {
      const int b = emitted & 1;
      if (ep_tid == 0) bulk_wait_read<1>();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      return out_stage + b * PAIR_OUT_BYTES;
    };
    auto stage_send = [&](uint8_t* st, const CUtensorMap* map, bool add, int x, int y) {
      fence_proxy_async();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ep_tid == 0) {
        if (add) tma_reduce_add_2d(map, smem_u32(st), x, y);
        else tma_store_2d(map, smem_u32(st), x, y);
        bulk_commit();
      }
      ++emitted;
    };
    // 32 token columns c0.. of this thread's feature go to `out`: staged and sent through the
    // tensor map (which clips at M and N), or written by the thread itself.
    auto emit32 = [&](int t0, int c0, int n0_cta, const float (&v)[32]) {
      if (staged) {
        uint8_t* stage = stage_acquire();
        if (p.epilogue == TC_RESIDUAL) {
          float* st = (float*)stage;
#pragma unroll
          for (int j = 0; j < 32; ++j) st[j * TILE_N + n_local] = v[j];
        } else {
          uint16_t* st = (uint16_t*)stage;
          const bool half = p.half != 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) st[j * TILE_N + n_local] = bits16(v[j], half);
        }
        stage_send(stage, &tmap_out, p.epilogue == TC_RESIDUAL, n0_cta, t0 + c0);
      } else if (n0_cta + n_local < p.N) {
        float lo[16], hi[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          lo[j] = v[j];
          hi[j] = v[16 + j];
        }
        tc_apply16(p, t0 + c0, n0_cta + n_local, lo, lo);
        tc_apply16(p, t0 + c0 + 16, n0_cta + n_local, hi, hi);
      }
    };
    // The same for interleaved gate and up rows: even lanes hold a feature's gate, odd lanes its
    // up product.  The two exchange halves of their 32 tokens, so that each ends with both
    // values of 16 tokens, and the tile leaves as 32 tokens x 64 features of bfloat16.
    auto emit32_gated = [&](int t0, int c0, int n0_cta, const float (&v)[32]) {
      const int odd = lane & 1;
      uint8_t* stage = stage_acquire();
      uint16_t* st = (uint16_t*)stage + (odd * 16) * (TILE_N / 2) + (n_local >> 1);
      const bool half = p.half != 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float theirs = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[16 + j], 1);
        const float g = odd ? theirs : v[j], up = odd ? v[16 + j] : theirs;
        st[j * (TILE_N / 2)] = bits16(g / (1.0f + __expf(-g)) * up, half);
      }
      stage_send(stage, &tmap_out, false, n0_cta >> 1, t0 + c0);
    };
    uint32_t fetch_phase = 0;
    long long tile;
    int kb0, kb1;
    for (int seg = 0; sched.segment(seg, tile, kb0, kb1); ++seg) {
      const bool whole = kb0 == 0 && kb1 == nkb;
      const int buf = seg & 1, use = seg >> 1;
      bool ok = mbar_wait(acc_full_bar(buf), use & 1, abort_p, wait_limit);
      if (!ok) abort_flag = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (abort_flag) {
        if (ep_tid == 0) atomicExch(p.err, 12);
        break;
      }
      tc_fence_after();
      int n_idx, t_idx;
      sched.coords(tile, n_idx, t_idx);
      const int n0 = n_idx * 2 * TILE_N + (int)rank * TILE_N, t0 = t_idx * PAIR_BT;
      const int n = n0 + n_local;
      const uint32_t acc_addr = lane_addr + buf * ACC_COLS;
      const uint32_t leader_acc_empty = map_to_cta(acc_empty_bar(buf), 0);
      if (whole && p.epilogue == TC_RESIDUAL && !staged) {
        // 32 columns at a time: the residual loads are issued before the accumulator is read,
        // so that each batch costs one memory latency, not two
        float* out = (float*)p.out + (size_t)t0 * p.ldo + n;
        const size_t ld = (size_t)p.ldo;
#pragma unroll 1
        for (int c0 = 0; c0 < PAIR_BT; c0 += 32) {
          const int valid = n < p.N ? p.M - t0 - c0 : 0;
          float r[32], v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = j < valid ? out[(c0 + j) * ld] : 0.f;
          tmem_ld16(acc_addr + c0, &v[0]);
          tmem_ld16(acc_addr + c0 + 16, &v[16]);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) out[(c0 + j) * ld] = r[j] + v[j];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
      } else if (whole && p.gated) {
#pragma unroll 1
        for (int c0 = 0; c0 < PAIR_BT && t0 + c0 < p.M; c0 += 32) {
          float v[32];
          tmem_ld16(acc_addr + c0, &v[0]);
          tmem_ld16(acc_addr + c0 + 16, &v[16]);
          emit32_gated(t0, c0, n0, v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
      } else if (whole) {
#pragma unroll 1
        for (int c0 = 0; c0 < PAIR_BT && t0 + c0 < p.M; c0 += 32) {
          float v[32];
          tmem_ld16(acc_addr + c0, &v[0]);
          tmem_ld16(acc_addr + c0 + 16, &v[16]);
          emit32(t0, c0, n0, v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
      } else {
        // half-tile partial -> workspace [cluster][end][rank][column][lane]
        const int c_first = sched.first_owner(tile), c_last = sched.last_owner(tile);
        const int n_contrib = c_last - c_first + 1;
        const size_t my_slot = ((size_t)cluster * 2 + sched.slot_of(cluster, tile)) * 2 + rank;
        float* ws = p.workspace + my_slot * tile_floats;
        int* const counter = p.counters + tile * 2 + rank;
        // The cluster that holds a tile's first k-blocks reaches it at the end of its range: it is
        // the tile's finisher.  It writes no partial of its own.  It waits (a bounded time) until
        // the others have left theirs, copies them into the idle stages with bulk copies, as many
        // columns at a time as fit, and adds them to its accumulator from tensor memory in K
        // order: the same sum, bit for bit, as the general case below, which remains for a finisher
        // whose wait ran out (the others never wait, so nothing can block).
        {
          long long t2;
          int a2, b2;
          const int others = n_contrib - 1;
          // columns per pass: what the stages hold of `others` partials (512 bytes per column)
          const int pass_cols = min(PAIR_BT, (int)((STAGES * PAIR_STAGE_BYTES) / (others * TILE_N * 4)) & ~31);
          const bool finisher = staged && cluster == c_first && pass_cols >= 32 && !sched.segment(seg + 1, t2, a2, b2);
          if (finisher) {
            if (ep_tid == 0) {
              int polls = 0;
              while (ld_acquire_gpu(counter) != others && ++polls < PAIR_FINISHER_POLLS && !*abort_p) __nanosleep(100);
              is_last = polls < PAIR_FINISHER_POLLS && !*abort_p;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
          const bool fast = finisher && is_last;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (fast) {
            const float* fetched = (const float*)smem;  // [contributor][column][128 rows]
            bool fine = true;
            for (int cb = 0; cb < PAIR_BT && t0 + cb < p.M && fine; cb += pass_cols) {
              const int ncols = min(pass_cols, PAIR_BT - cb);
              if (ep_tid == 0) {
                fence_proxy_async();  // the threads' reads of the pass before precede these copies
                mbar_expect_tx(fetch_bar, (uint32_t)(others * ncols * TILE_N * 4));
                for (int i = 0; i < others; ++i) {
                  const int cc = c_first + 1 + i;
                  const float* src = p.workspace + (((size_t)cc * 2 + sched.slot_of(cc, tile)) * 2 + rank) * tile_floats + (size_t)cb * TILE_N;
                  const uint32_t dst = smem_base + (uint32_t)(i * pass_cols * TILE_N * 4);
                  for (int c = 0; c < ncols; c += 32)  // 16 KB a copy
                    bulk_load(dst + c * TILE_N * 4, src + (size_t)c * TILE_N, 32 * TILE_N * 4, fetch_bar);
                }
              }
              fine = mbar_wait(fetch_bar, fetch_phase, abort_p, wait_limit);
              fetch_phase ^= 1;
              if (!fine) abort_flag = 1;
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (abort_flag) {
                if (ep_tid == 0) atomicExch(p.err, 14);
                fine = false;
                break;
              }
#pragma unroll 1
              for (int c0 = cb; c0 < cb + ncols && t0 + c0 < p.M; c0 += 32) {
                float v[32];
                tmem_ld16(acc_addr + c0, &v[0]);
                tmem_ld16(acc_addr + c0 + 16, &v[16]);
                for (int i = 0; i < others; ++i) {
                  const float* f = fetched + (size_t)i * pass_cols * TILE_N + (size_t)(c0 - cb) * TILE_N + n_local;
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += f[j * TILE_N];
                }
                if (p.gated) emit32_gated(t0, c0, n0, v);
                else emit32(t0, c0, n0, v);
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");  // all have read the stages before the next copies land
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
            if (ep_tid == 0 && fine) *counter = 0;
            continue;
          }
        }
        if (staged) {
          // the partial leaves like the output: 32 columns at a time through shared memory, as bulk
          // stores into the workspace seen as rows of 128 floats
#pragma unroll 1
          for (int c0 = 0; c0 < ACC_COLS; c0 += 32) {
            float v[32];
            tmem_ld16(acc_addr + c0, &v[0]);
            tmem_ld16(acc_addr + c0 + 16, &v[16]);
            float* st = (float*)stage_acquire();
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * TILE_N + n_local] = v[j];
            stage_send((uint8_t*)st, &tmap_ws, false, 0, (int)(my_slot * ACC_COLS) + c0);
          }
          if (ep_tid == 0) bulk_wait_all();  // the partial is written before it is announced
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < ACC_COLS; c0 += 16) {
            float v[16];
            tmem_ld16(acc_addr + c0, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) ws[(size_t)(c0 + j) * TILE_N + n_local] = v[j];
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ep_tid == 0) {
          const int old = atomicAdd(counter, 1);
          is_last = old == n_contrib - 1;
          if (is_last) *counter = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (is_last && staged) {
          // The last arriver adds the partials in K order.  A thread takes four neighbouring
          // features of eight columns, two contributors at a time: 16-byte loads, 16 of them in
          // flight per thread (with one load of 4 bytes per feature and column this reduction,
          // not the products, set the time of a product of a few hundred tokens).
          __threadfence();
          const int q4 = (ep_tid & 31) * 4, cg = (ep_tid >> 5) * 8;
          auto slot_of = [&](int cc) { return ((size_t)cc * 2 + sched.slot_of(cc, tile)) * 2 + rank; };
#pragma unroll 1
          for (int c0 = 0; c0 < PAIR_BT && t0 + c0 < p.M; c0 += 32) {
            float4 acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int cc = c_first; cc <= c_last; cc += 2) {
              const bool two = cc + 1 <= c_last;
              const float4* a = reinterpret_cast<const float4*>(p.workspace + slot_of(cc) * tile_floats + (size_t)(c0 + cg) * TILE_N + q4);
              const float4* b = reinterpret_cast<const float4*>(p.workspace + slot_of(two ? cc + 1 : cc) * tile_floats +
                                                                (size_t)(c0 + cg) * TILE_N + q4);
              float4 va[8], vb[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                va[k] = __ldcg(a + k * (TILE_N / 4));
                vb[k] = two ? __ldcg(b + k * (TILE_N / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int k = 0; k < 8; ++k) {  // first cc, then cc + 1: K order
                acc[k].x += va[k].x; acc[k].y += va[k].y; acc[k].z += va[k].z; acc[k].w += va[k].w;
                acc[k].x += vb[k].x; acc[k].y += vb[k].y; acc[k].z += vb[k].z; acc[k].w += vb[k].w;
              }
            }
            uint8_t* stage = stage_acquire();
            if (p.gated) {  // four neighbouring rows are two (gate, up) pairs
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t o2 = pack2_bits(acc[k].x / (1.0f + __expf(-acc[k].x)) * acc[k].y,
                                               acc[k].z / (1.0f + __expf(-acc[k].z)) * acc[k].w, p.half != 0);
                *reinterpret_cast<uint32_t*>((uint16_t*)stage + (cg + k) * (TILE_N / 2) + (q4 >> 1)) = o2;
              }
              stage_send(stage, &tmap_out, false, n0 >> 1, t0 + c0);
              continue;
            }
            if (p.epilogue == TC_RESIDUAL) {
#pragma unroll
              for (int k = 0; k < 8; ++k) *reinterpret_cast<float4*>((float*)stage + (cg + k) * TILE_N + q4) = acc[k];
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                uint2 pk;
                pk.x = pack2_bits(acc[k].x, acc[k].y, p.half != 0);
                pk.y = pack2_bits(acc[k].z, acc[k].w, p.half != 0);
                *reinterpret_cast<uint2*>((uint16_t*)stage + (cg + k) * TILE_N + q4) = pk;
              }
            }
            stage_send(stage, &tmap_out, p.epilogue == TC_RESIDUAL, n0, t0 + c0);
          }
        } else if (is_last) {  // the same for the four warps: they go through emit32 together
          __threadfence();
#pragma unroll 1
          for (int c0 = 0; c0 < PAIR_BT && t0 + c0 < p.M; c0 += 32) {
            float a0[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) a0[j] = 0.f;
            for (int cc = c_first; cc <= c_last; ++cc) {  // K order
              const float* wsp = p.workspace + (((size_t)cc * 2 + sched.slot_of(cc, tile)) * 2 + rank) * tile_floats +
                                 (size_t)c0 * TILE_N + n_local;
#pragma unroll
              for (int j = 0; j < 32; ++j) a0[j] += __ldcg(wsp + (size_t)j * TILE_N);
            }
            emit32(t0, c0, n0, a0);
          }
        }
      }
    }
    if (staged && ep_tid == 0) bulk_wait_all();  // shared memory and `out` are settled before the CTA leaves
    tc_fence_before();
  }

  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    const long long t0c = clock64();
    while (clock64() - t0c < 2000000LL) {
    }
  }
  // neither CTA may leave while the other can still read its shared memory or signal its barriers
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * ACC_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  int kind;  // 0: bfloat16 operand, 64-column boxes, 128-byte swizzle; 1 / 2: float32 / bfloat16 output, 128-column boxes;
             // 3: bfloat16 output, 64-column boxes; 4: gate and up rows of a weight interleaved (box_rows = rows between them)
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long long>()(k.rows);
    h = h * 1000003u ^ std::hash<long long>()(k.cols);
    h = h * 1000003u ^ std::hash<long long>()(k.ld);
    h = h * 1000003u ^ std::hash<long long>()((long long)k.box_rows * 8 + k.kind);
    return h;
  }
};

// A tensor map of a row-major bfloat16 matrix [rows, cols] with row stride ld, read in
// boxes of box_rows x 64 with the 128-byte swizzle; out-of-range elements read as zero.
// Maps are pure functions of their key and are kept for reuse.
static int get_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out,
                          int kind = 0) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows, kind};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  FERRUM_CHECK_ARG(fn != nullptr, "gemm_tc: the driver does not export cuTensorMapEncodeTiled");
  CUresult r;
  if (kind == 4) {
    // [rows] features of a gate block and of an up block `box_rows` rows further on, seen as
    // (k, gate | up, feature): a box of 64 x 2 x 64 lands as 128 rows gate 0, up 0, gate 1, ...
    cuuint64_t dims[3] = {(cuuint64_t)cols, 2, (cuuint64_t)rows};
    cuuint64_t strides[2] = {(cuuint64_t)box_rows * (cuuint64_t)ld * 2, (cuuint64_t)ld * 2};
    cuuint32_t box[3] = {(cuuint32_t)TILE_K, 2, (cuuint32_t)(TILE_N / 2)};
    cuuint32_t estr[3] = {1, 1, 1};
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (kind == 1 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)(kind == 0 ? TILE_K : (kind == 3 ? TILE_N / 2 : TILE_N)), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    r = fn(out, kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
           kind == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  FERRUM_CHECK_ARG(r == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%lld ld=%lld kind=%d)",
                   (int)r, rows, cols, ld, kind);
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

template <int BT, bool DUAL>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, int n_ctas, cudaStream_t stream) {
  using Cfg = TcConfig<BT, DUAL>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  launch_kernel(gemm_tc_kernel<BT, DUAL>, dim3(n_ctas), dim3(192), Cfg::SMEM_BYTES, stream, mw, mx, p);
  FERRUM_CHECK_LAUNCH("gemm_tc");
  return 0;
}

// Test hooks (see ferrum_gemm_tc_test_hooks): a shorter limit for every wait of the kernels, and a
// producer that requests nothing.
static long long g_wait_cycles = 0;
static int g_drop_loads = 0;
// wait_cycles > 0 shortens every bounded wait of the tensor-core product kernels to that many
// clock cycles (0: the default, about a second).  drop_loads = 1 makes the single-CTA kernel's
// producer request no tile, so that the waits for them run out: the kernel then raises an error
// code (10 to 13), frees its tensor memory and returns, and the context stays usable.  For
// tests of that path only; both settings stay until they are set back.
FERRUM_API void ferrum_gemm_tc_test_hooks(long long wait_cycles, int drop_loads) {
  g_wait_cycles = wait_cycles > 0 ? wait_cycles : 0;
  g_drop_loads = drop_loads != 0;
}

static bool g_pair_kernel = true;
// The CTA-pair kernel can be switched off (every shape then runs on the single-CTA kernel).
FERRUM_API void ferrum_set_gemm_pair_kernel(int on) { g_pair_kernel = on != 0; }

static int launch_tc_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const CUtensorMap& ms,
                          const TcParams& p, int n_ctas, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
    FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", PAIR_SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ctas);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, mw, mx, mo, ms, p);
  FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc: pair kernel launch failed: %s", cudaGetErrorString(e));
  FERRUM_CHECK_LAUNCH("gemm_tc_pair");
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&prop, dev) == cudaSuccess) n = prop.multiProcessorCount;
    if (n <= 0) n = 148;
  }
  return n;
}

// The token-tile width the kernel uses for M tokens.
FERRUM_API int ferrum_gemm_tc_token_tile(int M, int dual) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128 || dual) return 128;
  return 256;
}

// The grid the kernel runs with when the caller passes n_ctas = 0: one CTA per SM.
FERRUM_API int ferrum_gemm_tc_default_ctas() { return sm_count(); }

// Workspace floats and tile counters a launch needs.  Partial tiles arise where a CTA's
// range of units begins or ends inside a tile, so every CTA has two partial slots.
FERRUM_API long long ferrum_gemm_tc_workspace(int M, int N, int K, int dual, int n_ctas, int* n_tiles) {
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  if (n_ctas <= 0) n_ctas = sm_count();
  // counters: one per 128-row tile; the pair kernel numbers them by 256-row tile and half
  long long tiles = 2LL * ((N + 2 * TILE_N - 1) / (2 * TILE_N)) * ((M + bt - 1) / bt);
  if (dual && M > TILE_N)  // may run on the pair kernel as one product of 2 N interleaved rows
    tiles = std::max(tiles, 2LL * ((2LL * N + 2 * TILE_N - 1) / (2 * TILE_N)) * ((M + PAIR_BT - 1) / PAIR_BT));
  if (n_tiles) *n_tiles = (int)tiles;
  return 2LL * n_ctas * (long long)(bt * (dual ? 2 : 1)) * TILE_N;
}

// x [M, K] (row stride ldx) and w [w_rows, K] (row stride ldw) of the 16-bit type `dtype`
// (FERRUM_BF16 or FERRUM_F16), N output features.
// dual_offset > 0 selects the two-product kernel with the SwiGLU epilogue: the second weight
// tile starts at row dual_offset + n.  n_ctas = 0 means one CTA per SM.
FERRUM_API int ferrum_gemm_tc(const void* x, const void* w, void* out, int dtype, int M, int N, int K, int ldx, int ldw, int ldo,
                              int w_rows, int epilogue, int dual_offset, int n_ctas, float* workspace,
                              long long workspace_floats, int* counters, int n_counters, int* err_flag,
                              cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  FERRUM_CHECK_ARG(ferrum_is_16bit(dtype), "gemm_tc: dtype code %d is not a 16-bit type", dtype);
  FERRUM_CHECK_ARG(err_flag != nullptr, "gemm_tc: the error flag is required");
  if (M == 0) return 0;
  FERRUM_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_tc: K=%d and the row strides (%d, %d) must be multiples of 8 "
                   "(16-byte rows for TMA); use the generic kernel", K, ldx, ldw);
  FERRUM_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
  FERRUM_CHECK_ARG(ldx >= K && ldw >= K && ldo >= N, "gemm_tc: a row stride is shorter than its row");
  const bool dual = dual_offset > 0;
  FERRUM_CHECK_ARG(dual == (epilogue == TC_SWIGLU), "gemm_tc: the SwiGLU epilogue needs dual_offset, and only it does");
  FERRUM_CHECK_ARG(epilogue >= 0 && epilogue <= 3, "gemm_tc: unknown epilogue %d", epilogue);
  FERRUM_CHECK_ARG(w_rows >= N + dual_offset, "gemm_tc: w has %d rows, needs %d", w_rows, N + dual_offset);
  if (n_ctas <= 0) n_ctas = sm_count();
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  int tiles = 0;
  const long long need = ferrum_gemm_tc_workspace(M, N, K, dual, n_ctas, &tiles);
  FERRUM_CHECK_ARG(workspace && workspace_floats >= need, "gemm_tc: needs %lld workspace floats, got %lld", need, workspace_floats);
  FERRUM_CHECK_ARG(counters && n_counters >= tiles, "gemm_tc: needs %d tile counters, got %d", tiles, n_counters);
  {
    // every CTA must own at least one unit, or the CTAs that share a tile are not consecutive
    const long long units = (long long)((N + TILE_N - 1) / TILE_N) * ((M + bt - 1) / bt) * ((K + TILE_K - 1) / TILE_K);
    if (n_ctas > units) n_ctas = (int)units;
  }
  TcParams p{out, workspace, counters, err_flag, M, N, K, ldo, epilogue, dual_offset, 0};
  p.half = dtype == FERRUM_F16;
  p.wait_cycles = g_wait_cycles;
  p.drop_loads = g_drop_loads;
  p.stream_weights = (M + bt - 1) / bt == 1;  // one token tile: no weight tile is read twice
  CUtensorMap mw, mx;
  if (dual && M > TILE_N && g_pair_kernel && n_ctas >= 2 && ((uintptr_t)out & 15) == 0 && ldo % 8 == 0) {
    // Two products of many tokens: the pair kernel computes them as one product whose weight
    // rows alternate between gate and up (a three-dimensional tensor map interleaves them on
    // the way into shared memory), and its epilogue applies the activation.
    p.N = 2 * N;
    p.gated = 1;
    p.stream_weights = 0;
    const long long units = (long long)((p.N + 2 * TILE_N - 1) / (2 * TILE_N)) * ((M + PAIR_BT - 1) / PAIR_BT) * ((K + TILE_K - 1) / TILE_K);
    int pairs = n_ctas / 2;
    if (pairs > units) pairs = (int)units;
    CUtensorMap mo, ms;
    if (int r = get_tensor_map(w, N, K, ldw, dual_offset, &mw, 4)) return r;
    if (int r = get_tensor_map(x, M, K, ldx, PAIR_BT / 2, &mx)) return r;
    if (int r = get_tensor_map(out, M, N, ldo, PAIR_OUT_ROWS, &mo, 3)) return r;
    FERRUM_CHECK_ARG(((uintptr_t)workspace & 15) == 0, "gemm_tc: the workspace must be 16-byte aligned");
    if (int r = get_tensor_map(workspace, workspace_floats / TILE_N, TILE_N, TILE_N, PAIR_OUT_ROWS, &ms, 1)) return r;
    p.out_tma = 1;
    return launch_tc_pair(mw, mx, mo, ms, p, 2 * pairs, stream);
  }
  if (int r = get_tensor_map(w, w_rows, K, ldw, TILE_N, &mw)) return r;
  if (bt == PAIR_BT && !dual && g_pair_kernel && n_ctas >= 2) {
    // many tokens: pairs of CTAs on 256 x 256 tiles; each CTA stages 128 tokens
    const long long units = (long long)((N + 2 * TILE_N - 1) / (2 * TILE_N)) * ((M + PAIR_BT - 1) / PAIR_BT) * ((K + TILE_K - 1) / TILE_K);
    int pairs = n_ctas / 2;
    if (pairs > units) pairs = (int)units;
    if (int r = get_tensor_map(x, M, K, ldx, PAIR_BT / 2, &mx)) return r;
    // the output through a tensor map where its rows are 16-byte multiples; else by the threads
    CUtensorMap mo = mw;
    const int esize = epilogue == TC_RESIDUAL ? 4 : 2;
    if ((epilogue == TC_RESIDUAL || epilogue == TC_STORE_BF16) && ((uintptr_t)out & 15) == 0 && ((long long)ldo * esize) % 16 == 0) {
      if (int r = get_tensor_map(out, M, N, ldo, PAIR_OUT_ROWS, &mo, epilogue == TC_RESIDUAL ? 1 : 2)) return r;
      p.out_tma = 1;
    }
    // the workspace as rows of 128 floats (one row per column of a partial half tile)
    CUtensorMap ms = mw;
    if (p.out_tma) {
      FERRUM_CHECK_ARG(((uintptr_t)workspace & 15) == 0, "gemm_tc: the workspace must be 16-byte aligned");
      if (int r = get_tensor_map(workspace, workspace_floats / TILE_N, TILE_N, TILE_N, PAIR_OUT_ROWS, &ms, 1)) return r;
    }
    return launch_tc_pair(mw, mx, mo, ms, p, 2 * pairs, stream);
  }
  if (int r = get_tensor_map(x, M, K, ldx, bt, &mx)) return r;
#define TC_CASE(BT_)                                                         \
  case BT_:                                                                  \
    return dual ? launch_tc<BT_, true>(mw, mx, p, n_ctas, stream) : launch_tc<BT_, false>(mw, mx, p, n_ctas, stream);
  switch (bt) {
    TC_CASE(16)
    TC_CASE(32)
    TC_CASE(64)
    TC_CASE(128)
    case 256:
      return launch_tc<256, false>(mw, mx, p, n_ctas, stream);
  }
#undef TC_CASE
  FERRUM_CHECK_ARG(false, "gemm_tc: no kernel for token tile %d", bt);
}

// For tests of the schedule on the host: pair `cluster`'s s-th segment when `pairs` pairs
// compute M tokens x `rows` weight rows (for gate and up as one product: both) over K.
// out[0..7] = tile, first k-block, one past the last, weight tile index, token tile index, and
// for a tile that pairs share its first and last contributor and the slot (0 or 1) of this
// pair's partial (-1 each for a whole tile).  Returns 0 when the pair has no such segment.
FERRUM_API int ferrum_gemm_pair_schedule(int M, long long rows, int K, int pairs, int cluster, int s, long long* out) {
  const int nkb = (K + TILE_K - 1) / TILE_K;
  const int tiles_n = (int)((rows + 2 * TILE_N - 1) / (2 * TILE_N)), tiles_t = (M + PAIR_BT - 1) / PAIR_BT;
  const PairSchedule sched(tiles_n, tiles_t, nkb, pairs, cluster);
  long long tile;
  int kb0, kb1, n_idx, t_idx;
  if (!sched.segment(s, tile, kb0, kb1)) return 0;
  sched.coords(tile, n_idx, t_idx);
  const bool whole = kb0 == 0 && kb1 == nkb;
  out[0] = tile;
  out[1] = kb0;
  out[2] = kb1;
  out[3] = n_idx;
  out[4] = t_idx;
  out[5] = whole ? -1 : sched.first_owner(tile);
  out[6] = whole ? -1 : sched.last_owner(tile);
  out[7] = whole ? -1 : sched.slot_of(cluster, tile);
  return 1;
}

// ------------------------------------------------------------------ deferred reduction
// With few tokens every output tile is shared by several CTAs and the in-kernel reduction
// (fence, counter, reload) is a serial tail of several microseconds per launch.  In deferred
// mode the kernel stops after writing its float32 partials; the kernel that consumes the
// product (RMSNorm, the rotary kernel, ...) adds them while it reads, in K order, with
// partial_sum() of partials.cuh.  Requirements: one token tile (M <= 256, or 128 for two
// products) and at most one output tile per CTA, so that a CTA writes at most two partials.
// With 65 to 256 tokens the in-kernel reduction is worse still: the last arriver of a tile
// reads several 64 to 128 KB partials and read-modify-writes the output on its own.
FERRUM_API int ferrum_gemm_tc_can_defer(int M, int N, int K, int dual, int n_ctas) {
  if (n_ctas <= 0) n_ctas = sm_count();
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  const long long tiles = (N + TILE_N - 1) / TILE_N;
  const long long units = tiles * ((K + TILE_K - 1) / TILE_K);
  if (n_ctas > units) n_ctas = (int)units;
  // at most 8 CTAs may share a tile (the consumers keep that many loads in flight per element)
  const long long per = units / n_ctas;
  return M > 0 && M <= bt && tiles <= n_ctas && per > 0 && ((K + TILE_K - 1) / TILE_K) / per + 2 <= 8;
}

// layout[0..3] = k-blocks per tile, tiles, CTAs, columns per partial: what partial_sum() needs.
FERRUM_API int ferrum_gemm_tc_deferred(const void* x, const void* w, int dtype, int M, int N, int K, int ldx, int ldw, int w_rows,
                                       int dual_offset, int n_ctas, float* workspace, long long workspace_floats,
                                       int* layout, int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(M > 0 && N > 0 && K > 0 && err_flag && layout, "gemm_tc_deferred: bad arguments");
  FERRUM_CHECK_ARG(ferrum_is_16bit(dtype), "gemm_tc_deferred: dtype code %d is not a 16-bit type", dtype);
  FERRUM_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0,
                   "gemm_tc_deferred: operands must have 16-byte rows and alignment");
  FERRUM_CHECK_ARG(ldx >= K && ldw >= K, "gemm_tc_deferred: a row stride is shorter than its row");
  const bool dual = dual_offset > 0;
  FERRUM_CHECK_ARG(w_rows >= N + dual_offset, "gemm_tc_deferred: w has %d rows, needs %d", w_rows, N + dual_offset);
  FERRUM_CHECK_ARG(ferrum_gemm_tc_can_defer(M, N, K, dual, n_ctas), "gemm_tc_deferred: shape M=%d N=%d K=%d cannot defer its "
                   "reduction (more than one token tile, or more output tiles than CTAs)", M, N, K);
  if (n_ctas <= 0) n_ctas = sm_count();
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  const int nkb = (K + TILE_K - 1) / TILE_K, tiles = (N + TILE_N - 1) / TILE_N;
  if (n_ctas > (long long)tiles * nkb) n_ctas = tiles * nkb;
  const int acc_cols = bt * (dual ? 2 : 1);
  const long long need = 2LL * n_ctas * acc_cols * TILE_N;
  FERRUM_CHECK_ARG(workspace && workspace_floats >= need, "gemm_tc_deferred: needs %lld workspace floats, got %lld", need,
                   workspace_floats);
  layout[0] = nkb;
  layout[1] = tiles;
  layout[2] = n_ctas;
  layout[3] = acc_cols;
  CUtensorMap mw, mx;
  if (int r = get_tensor_map(w, w_rows, K, ldw, TILE_N, &mw)) return r;
  if (int r = get_tensor_map(x, M, K, ldx, bt, &mx)) return r;
  TcParams p{nullptr, workspace, nullptr, err_flag, M, N, K, 0, dual ? TC_SWIGLU : TC_STORE_F32, dual_offset, 1};
  p.half = dtype == FERRUM_F16;
  p.wait_cycles = g_wait_cycles;
  p.stream_weights = 1;  // deferred mode has one token tile: no weight tile is read twice
  switch (bt) {
    case 16: return dual ? launch_tc<16, true>(mw, mx, p, n_ctas, stream) : launch_tc<16, false>(mw, mx, p, n_ctas, stream);
    case 32: return dual ? launch_tc<32, true>(mw, mx, p, n_ctas, stream) : launch_tc<32, false>(mw, mx, p, n_ctas, stream);
    case 64: return dual ? launch_tc<64, true>(mw, mx, p, n_ctas, stream) : launch_tc<64, false>(mw, mx, p, n_ctas, stream);
    case 128: return dual ? launch_tc<128, true>(mw, mx, p, n_ctas, stream) : launch_tc<128, false>(mw, mx, p, n_ctas, stream);
    case 256:
      if (!dual) return launch_tc<256, false>(mw, mx, p, n_ctas, stream);
  }
  FERRUM_CHECK_ARG(false, "gemm_tc_deferred: no kernel for token tile %d", bt);
}

// ------------------------------------------------------------------ no-allocation entry point
// See ferrum_noalloc.h for who needs this and for the rules of use.
#include "ferrum_noalloc.h"

// Scratch of ferrum_gemm_tc_noalloc: float32 partial tiles, then the tile counters.  It is
// part of the library's device image: every GPU that loads the library holds it until exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FERRUM_NOALLOC_SCRATCH_BYTES + FERRUM_NOALLOC_MAX_TILES * sizeof(int)];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel
// can use; the device address is looked up once per device, with that device current.
static int noalloc_scratch_address(unsigned char** out) {
  constexpr int kMaxDevices = 64;
  static unsigned char* addr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
  FERRUM_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "gemm_tc_noalloc: device ordinal %d is not supported", dev);
  std::lock_guard<std::mutex> g(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    FERRUM_CHECK_ARG(e == cudaSuccess && p != nullptr, "gemm_tc_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = addr[dev];
  return 0;
}

// A tensor map built on the stack (the cached variant keeps maps in a host container).
static int encode_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  EncodeTiledFn fn = get_encode_fn();
  FERRUM_CHECK_ARG(fn != nullptr, "gemm_tc_noalloc: the driver does not export cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FERRUM_CHECK_ARG(r == CUDA_SUCCESS, "gemm_tc_noalloc: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

FERRUM_API int ferrum_gemm_tc_noalloc(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw,
                                      int ldo, int w_rows, int epilogue, int dual_offset, int* err_flag,
                                      cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_tc_noalloc: bad sizes M=%d N=%d K=%d", M, N, K);
  FERRUM_CHECK_ARG(err_flag != nullptr, "gemm_tc_noalloc: the error flag is required");
  if (M == 0) return 0;
  FERRUM_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_tc_noalloc: K=%d and the row strides (%d, %d) must be "
                   "multiples of 8 (16-byte rows for TMA)", K, ldx, ldw);
  FERRUM_CHECK_ARG(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc_noalloc: operands must be 16-byte aligned");
  FERRUM_CHECK_ARG(ldx >= K && ldw >= K && ldo >= N, "gemm_tc_noalloc: a row stride is shorter than its row");
  const bool dual = dual_offset > 0;
  FERRUM_CHECK_ARG(epilogue >= 0 && epilogue <= 3, "gemm_tc_noalloc: unknown epilogue %d", epilogue);
  FERRUM_CHECK_ARG(dual == (epilogue == TC_SWIGLU), "gemm_tc_noalloc: the SwiGLU epilogue needs dual_offset, and only it does");
  FERRUM_CHECK_ARG(w_rows >= N + dual_offset, "gemm_tc_noalloc: w has %d rows, needs %d", w_rows, N + dual_offset);
  int n_ctas = sm_count();
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  int tiles = 0;
  const long long need_floats = ferrum_gemm_tc_workspace(M, N, K, dual, n_ctas, &tiles);
  FERRUM_CHECK_ARG(need_floats * (long long)sizeof(float) <= (long long)FERRUM_NOALLOC_SCRATCH_BYTES,
                   "gemm_tc_noalloc: %d tokens%s need %lld bytes of scratch, the built-in array holds %u; use ferrum_gemm_tc "
                   "with a caller-provided workspace", M, dual ? " with the SwiGLU epilogue" : "",
                   need_floats * (long long)sizeof(float), FERRUM_NOALLOC_SCRATCH_BYTES);
  FERRUM_CHECK_ARG(tiles <= FERRUM_NOALLOC_MAX_TILES, "gemm_tc_noalloc: %d output tiles exceed the built-in %d counters", tiles,
                   FERRUM_NOALLOC_MAX_TILES);
  unsigned char* scratch = nullptr;
  if (int r = noalloc_scratch_address(&scratch)) return r;
  float* workspace = reinterpret_cast<float*>(scratch);
  int* counters = reinterpret_cast<int*>(scratch + FERRUM_NOALLOC_SCRATCH_BYTES);
  // the counters are the only part of the shared array that must start at zero
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)tiles * sizeof(int), stream);
  FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
  {
    const long long units = (long long)((N + TILE_N - 1) / TILE_N) * ((M + bt - 1) / bt) * ((K + TILE_K - 1) / TILE_K);
    if (n_ctas > units) n_ctas = (int)units;
  }
  CUtensorMap mw, mx;
  if (int r = encode_tensor_map(w, w_rows, K, ldw, TILE_N, &mw)) return r;
  if (int r = encode_tensor_map(x, M, K, ldx, bt, &mx)) return r;
  TcParams p{out, workspace, counters, err_flag, M, N, K, ldo, epilogue, dual_offset, 0};
  switch (bt) {
    case 16: return dual ? launch_tc<16, true>(mw, mx, p, n_ctas, stream) : launch_tc<16, false>(mw, mx, p, n_ctas, stream);
    case 32: return dual ? launch_tc<32, true>(mw, mx, p, n_ctas, stream) : launch_tc<32, false>(mw, mx, p, n_ctas, stream);
    case 64: return dual ? launch_tc<64, true>(mw, mx, p, n_ctas, stream) : launch_tc<64, false>(mw, mx, p, n_ctas, stream);
    case 128: return dual ? launch_tc<128, true>(mw, mx, p, n_ctas, stream) : launch_tc<128, false>(mw, mx, p, n_ctas, stream);
    case 256: return launch_tc<256, false>(mw, mx, p, n_ctas, stream);
  }
  FERRUM_CHECK_ARG(false, "gemm_tc_noalloc: no kernel for token tile %d", bt);
}

FERRUM_TRACE_READER(ferrum_trace_gemm)
