// bfloat16 matrix product on the tcgen05 tensor cores: out[t, n] = sum_k x[t, k] * w[n, k].
//
// Orientation: the weight rows are the M side of the instruction (128 rows of W per CTA,
// one row per TMEM lane) and the tokens are the N side (BT columns, 16..256).  The same
// kernel therefore serves a 2048-token prompt (BT = 256) and a single decoded token
// (BT = 16): in decode the tensor cores idle and the CTA is a TMA streaming engine for its
// slice of the weights.  Both operands are K-major tiles of 64 bfloat16 per row, brought in
// by TMA with the 128-byte swizzle into a ring of stages; one thread issues the MMAs, the
// accumulator lives in tensor memory, four warps read it back for the epilogue.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA issuer,
// warps 2..5 = epilogue.  DUAL computes two accumulators from two weight tiles (rows n and
// dual_offset + n) against the same tokens; the SwiGLU epilogue combines them, so gate and
// up need no interleaving in memory.
//
// Split-K: grid.z CTAs share a tile's K range.  Each writes its float32 partial tile to the
// workspace; the CTA that arrives last at the tile's counter adds the partials in split
// order (so the sum does not depend on arrival order) and runs the epilogue.  Nobody waits
// for anybody.  The counter is left at zero for the next launch.
//
// Every mbarrier wait is bounded; on a timeout the kernel raises the error flag, lets the
// copies in flight land, frees its tensor memory and returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

enum TcEpilogue : int {
  TC_STORE_BF16 = 0,  // out bf16 [M, ldo] = acc
  TC_STORE_F32 = 1,   // out f32  [M, ldo] = acc
  TC_RESIDUAL = 2,    // out f32  [M, ldo] += acc
  TC_SWIGLU = 3,      // out bf16 [M, ldo] = silu(acc0) * acc1   (DUAL only)
};

struct TcParams {
  void* out;
  float* workspace;
  int* counters;
  int* err;
  int M, N, K, ldo;
  int epilogue;
  int dual_offset;  // row of the second weight tile relative to the first (DUAL)
};

constexpr int TILE_N = 128;  // weight rows per CTA (the instruction's M)
constexpr int TILE_K = 64;   // bfloat16 per row of a stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_BYTES = TILE_N * TILE_K * 2;

template <int BT, bool DUAL>
struct TcConfig {
  static constexpr int B_BYTES = BT * TILE_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  static constexpr int BUDGET = 196 * 1024;
  static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 8 ? 8 : (BUDGET / STAGE_BYTES);
  static constexpr int ACC_COLS = BT * (DUAL ? 2 : 1);
  static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(STAGES >= 2, "tile too large for the shared memory budget");
};

__device__ __forceinline__ void tc_apply(const TcParams& p, int t, int n, float a0, float a1) {
  const size_t o = (size_t)t * p.ldo + n;
  switch (p.epilogue) {
    case TC_STORE_BF16: ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(a0); break;
    case TC_STORE_F32: ((float*)p.out)[o] = a0; break;
    case TC_RESIDUAL: ((float*)p.out)[o] += a0; break;
    case TC_SWIGLU: ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(a0 / (1.0f + __expf(-a0)) * a1); break;
  }
}

template <int BT, bool DUAL>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const TcParams p) {
  using Cfg = TcConfig<BT, DUAL>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::STAGE_BYTES);  // full[S], empty[S], acc_full
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TILE_N, t0 = blockIdx.y * BT;
  const int splits = gridDim.z, split = blockIdx.z;
  const int nkb = (p.K + TILE_K - 1) / TILE_K;
  const int kb_begin = (int)((long long)nkb * split / splits), kb_end = (int)((long long)nkb * (split + 1) / splits);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t acc_bar = bar_base + 8u * (2 * STAGES);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    is_last = 0;
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(empty_bar(s), phase ^ 1, abort_p)) {
          abort_flag = 1;
          atomicExch(p.err, 10);
          break;
        }
        const uint32_t a = smem_base + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
        tma_load_2d(a, &tmap_w, full_bar(s), kb * TILE_K, n0);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmap_w, full_bar(s), kb * TILE_K, p.dual_offset + n0);
        tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), &tmap_x, full_bar(s), kb * TILE_K, t0);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(TILE_N, BT);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(full_bar(s), phase, abort_p)) {
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
          const bool acc = (kb > kb_begin) || (kk > 0);
          const uint64_t adv = (uint64_t)(kk * UMMA_K * 2 >> 4);  // 32 bytes per step, in 16-byte units
          umma_bf16(tmem_base, a_desc + adv, b_desc + adv, idesc, acc);
          if (DUAL) umma_bf16(tmem_base + BT, a2_desc + adv, b_desc + adv, idesc, acc);
        }
        umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(acc_bar);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32*quarter .. +31
    const int n_local = quarter * 32 + lane;
    const int n = n0 + n_local;
    const int ep_tid = threadIdx.x - 64;
    bool ok = mbar_wait(acc_bar, 0, abort_p);
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
    if (!ok && lane == 0) {
      abort_flag = 1;
      atomicExch(p.err, 12);
    }
    tc_fence_after();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (ok && splits == 1) {
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 16) {
        float v0[16], v1[16];
        tmem_ld16(lane_addr + c0, v0);
        if (DUAL) tmem_ld16(lane_addr + BT + c0, v1);
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t < p.M) tc_apply(p, t, n, v0[j], DUAL ? v1[j] : 0.f);
          }
        }
      }
    } else if (ok) {
      // partial tile -> workspace [tile][split][column][lane]
      const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
      float* ws = p.workspace + (tile * splits + split) * (size_t)(Cfg::ACC_COLS * TILE_N);
#pragma unroll 1
      for (int c0 = 0; c0 < Cfg::ACC_COLS; c0 += 16) {
        float v[16];
        tmem_ld16(lane_addr + c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) ws[(size_t)(c0 + j) * TILE_N + n_local] = v[j];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ep_tid == 0) {
        const int old = atomicAdd(p.counters + tile, 1);
        if (old == splits - 1) {
          is_last = 1;
          p.counters[tile] = 0;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (is_last) {
        __threadfence();
        const float* base = p.workspace + tile * splits * (size_t)(Cfg::ACC_COLS * TILE_N);
        if (n < p.N) {
#pragma unroll 1
          for (int c = 0; c < BT; ++c) {
            const int t = t0 + c;
            if (t >= p.M) break;
            float a0 = 0.f, a1 = 0.f;
            for (int s = 0; s < splits; ++s) {
              const float* wsp = base + (size_t)s * (Cfg::ACC_COLS * TILE_N);
              a0 += __ldcg(wsp + (size_t)c * TILE_N + n_local);
              if (DUAL) a1 += __ldcg(wsp + (size_t)(BT + c) * TILE_N + n_local);
            }
            tc_apply(p, t, n, a0, a1);
          }
        }
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
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long long>()(k.rows);
    h = h * 1000003u ^ std::hash<long long>()(k.cols);
    h = h * 1000003u ^ std::hash<long long>()(k.ld);
    h = h * 1000003u ^ std::hash<int>()(k.box_rows);
    return h;
  }
};

// A tensor map of a row-major bfloat16 matrix [rows, cols] with row stride ld, read in
// boxes of box_rows x 64 with the 128-byte swizzle; out-of-range elements read as zero.
// Maps are pure functions of their key and are kept for reuse.
static int get_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows};
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
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FERRUM_CHECK_ARG(r == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%lld ld=%lld)",
                   (int)r, rows, cols, ld);
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

template <int BT, bool DUAL>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, int splits, cudaStream_t stream) {
  using Cfg = TcConfig<BT, DUAL>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    FERRUM_CHECK_ARG(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((p.N + TILE_N - 1) / TILE_N, (p.M + BT - 1) / BT, splits);
  FERRUM_CHECK_ARG(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
  gemm_tc_kernel<BT, DUAL><<<grid, 192, Cfg::SMEM_BYTES, stream>>>(mw, mx, p);
  FERRUM_CHECK_LAUNCH("gemm_tc");
  return 0;
}

// Workspace floats one launch needs (0 without split-K); also the number of tile counters.
FERRUM_API long long ferrum_gemm_tc_workspace(int M, int N, int bt, int dual, int splits, int* n_tiles) {
  const long long tiles = (long long)((N + TILE_N - 1) / TILE_N) * ((M + bt - 1) / bt);
  if (n_tiles) *n_tiles = (int)tiles;
  if (splits <= 1) return 0;
  return tiles * splits * (long long)(bt * (dual ? 2 : 1)) * TILE_N;
}

// The token-tile width the kernel uses for M tokens.
FERRUM_API int ferrum_gemm_tc_token_tile(int M, int dual) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128 || dual) return 128;
  return 256;
}

// x [M, K] bf16 (row stride ldx), w [N (+dual_offset) rows, K] bf16 (row stride ldw).
// dual_offset > 0 selects the two-accumulator kernel with the SwiGLU epilogue: the second
// weight tile starts at row dual_offset + n.  w_rows is the number of rows of w in memory.
FERRUM_API int ferrum_gemm_tc(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                              int w_rows, int epilogue, int dual_offset, int splits, float* workspace,
                              long long workspace_floats, int* counters, int n_counters, int* err_flag,
                              cudaStream_t stream) {
  FERRUM_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
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
  const int nkb = (K + TILE_K - 1) / TILE_K;
  FERRUM_CHECK_ARG(splits >= 1 && splits <= nkb, "gemm_tc: splits=%d must be in [1, %d]", splits, nkb);
  const int bt = ferrum_gemm_tc_token_tile(M, dual);
  int tiles = 0;
  const long long need = ferrum_gemm_tc_workspace(M, N, bt, dual, splits, &tiles);
  if (splits > 1) {
    FERRUM_CHECK_ARG(workspace && workspace_floats >= need, "gemm_tc: split-K needs %lld workspace floats, got %lld", need,
                     workspace_floats);
    FERRUM_CHECK_ARG(counters && n_counters >= tiles, "gemm_tc: split-K needs %d tile counters, got %d", tiles, n_counters);
  }
  CUtensorMap mw, mx;
  if (int r = get_tensor_map(w, w_rows, K, ldw, TILE_N, &mw)) return r;
  if (int r = get_tensor_map(x, M, K, ldx, bt, &mx)) return r;
  TcParams p{out, workspace, counters, err_flag, M, N, K, ldo, epilogue, dual_offset};
#define TC_CASE(BT_)                                                         \
  case BT_:                                                                  \
    return dual ? launch_tc<BT_, true>(mw, mx, p, splits, stream) : launch_tc<BT_, false>(mw, mx, p, splits, stream);
  switch (bt) {
    TC_CASE(16)
    TC_CASE(32)
    TC_CASE(64)
    TC_CASE(128)
    case 256:
      return launch_tc<256, false>(mw, mx, p, splits, stream);
  }
#undef TC_CASE
  FERRUM_CHECK_ARG(false, "gemm_tc: no kernel for token tile %d", bt);
}
