// Next-token choice on the GPU: argmax, or the Gumbel-max draw from softmax(logits / T).
//
// Greedy follows the reference's argmax (crates/core-types/src/model.rs:44-62): the lowest
// index wins ties, NaN entries are skipped, a row of NaN only is an error (id -1 and the
// error flag).  With a temperature the kernel returns argmax_i(logit_i / T + g_i) where
// g_i = -log(-log(u_i)) and u_i is a pure function of (seed, counter, i), so a request's
// draw does not depend on the batch it is in.  The reference samples greedily only.
#include "common.cuh"

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // an index of -1 marks "nothing seen"
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// A large vocabulary is shared out between the SAMPLE_CLUSTER CTAs of a cluster (gridDim.y of
// them per row; 1 for a small vocabulary): a handful of rows would otherwise be read by a
// handful of SMs.  The slices' winners meet in the first CTA's shared memory; `better` does not
// depend on the order in which it sees them.
constexpr int SAMPLE_CLUSTER = 8;

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ inv_temperature,
              const unsigned long long* __restrict__ seeds, const int* __restrict__ counters,
              int* __restrict__ out_ids, int* __restrict__ also_to, int* __restrict__ err) {
  __shared__ Best red[32];
  __shared__ Best slice_best[SAMPLE_CLUSTER];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int n_slices = gridDim.y, slice = blockIdx.y;
  // a CTA's shared memory may be written by a peer only once the CTA is known to run: arrive
  // now, wait before the hand-over below
  if (n_slices > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const int per = (V + n_slices - 1) / n_slices;
  const int v_lo = slice * per, v_hi = min(V, v_lo + per);
  const float* row = logits + (size_t)r * ld;
  const float inv_t = inv_temperature ? inv_temperature[r] : 0.f;
  uint32_t key = 0;
  if (inv_t != 0.f) {
    const unsigned long long seed = seeds[r];
    key = mix32((uint32_t)seed ^ mix32((uint32_t)(seed >> 32) ^ mix32((uint32_t)counters[r])));
  }
  Best best{0.f, -1};
  for (int i = v_lo + threadIdx.x; i < v_hi; i += blockDim.x) {
    float z = row[i];
    if (z != z) continue;
    if (inv_t != 0.f) {
      const uint32_t bits = mix32(key ^ mix32((uint32_t)i)) >> 9;
      const float u = __fmul_rn(__fadd_rn((float)bits, 0.5f), 1.0f / 8388608.0f);
      const float g = -logf(-logf(u));
      z = __fadd_rn(__fmul_rn(z, inv_t), g);
    }
    best = better(best, Best{z, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (n_slices > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? red[lane] : Best{0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (lane == 0 && n_slices > 1) {
      // hand the slice's winner to the first CTA of the cluster
      unsigned local = (unsigned)__cvta_generic_to_shared(&slice_best[slice]), remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
      asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(remote), "r"(__float_as_uint(best.v)), "r"(best.i) : "memory");
    }
  }
  if (n_slices > 1) {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (slice != 0 || threadIdx.x != 0) return;
    best = slice_best[0];
    for (int c = 1; c < n_slices; ++c) best = better(best, slice_best[c]);
  } else if (threadIdx.x != 0) {
    return;
  }
  out_ids[r] = best.i;
  if (also_to != nullptr) also_to[r] = best.i;
  if (best.i < 0) atomicExch(err, 6);
}

// inv_temperature[r] == 0 (or a null array) means greedy for row r.  also_to (may be null) receives
// the ids as well: the token buffer of a step that is queued behind this one.
FERRUM_API int ferrum_sample(const float* logits, int ld, int n_rows, int V, const float* inv_temperature,
                             const unsigned long long* seeds, const int* counters, int* out_ids, int* also_to,
                             int* err_flag, cudaStream_t stream) {
  FERRUM_CHECK_ARG(n_rows >= 0 && V > 0 && ld >= V, "sample: bad sizes rows=%d V=%d ld=%d", n_rows, V, ld);
  FERRUM_CHECK_ARG(!inv_temperature || (seeds && counters), "sample: temperature given without seeds and counters");
  if (n_rows == 0) return 0;
  const int slices = V >= 16384 ? SAMPLE_CLUSTER : 1;
  const int threads = V >= 8192 * slices ? 1024 : 256;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_rows, slices);
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = slices;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ferrum_dependent_launch_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, inv_temperature, seeds, counters, out_ids, also_to, err_flag);
  FERRUM_CHECK_ARG(e == cudaSuccess, "sample: launch failed: %s", cudaGetErrorString(e));
  FERRUM_CHECK_LAUNCH("sample");
  return 0;
}
