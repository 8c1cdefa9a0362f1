// Reading a product that the tensor-core kernel left as float32 partials (deferred mode).
//
// The kernel's CTA c owns the units [c*U/P, (c+1)*U/P) of the line of (tile, k-block) units
// (U = tiles * nkb, one token tile); a CTA touches at most two tiles and leaves the partial
// of the tile in which its range begins in slot 0, of the other in slot 1, laid out
// [column][128 rows].  A consumer first builds, in shared memory, the list of contributors
// of every tile (PartialTable), then adds a tile's contributors in CTA order, which is K
// order, so the result does not depend on timing.
#pragma once
#include "common.cuh"

constexpr int PARTIAL_MAX_TILES = 256;
constexpr int PARTIAL_MAX_CONTRIB = 8;  // CTAs that may share one tile in deferred mode

struct PartialLayout {
  const float* ws;
  int nkb, tiles, n_ctas, acc_cols;
};

struct PartialTable {
  int first_and_count[PARTIAL_MAX_TILES];  // first contributor | count << 16
  unsigned slot_bits[PARTIAL_MAX_TILES];   // bit s: the s-th contributor's partial is in its slot 1
};

__device__ __forceinline__ int partial_owner(long long u, long long U, int P) { return (int)(((u + 1) * P + U - 1) / U) - 1; }

// Called by every thread of the block; ends with a __syncthreads().
__device__ __forceinline__ void build_partial_table(const PartialLayout& L, PartialTable& tab) {
  for (int tile = threadIdx.x; tile < L.tiles; tile += blockDim.x) {
    const long long U = (long long)L.tiles * L.nkb;
    const int c_first = partial_owner((long long)tile * L.nkb, U, L.n_ctas);
    const int c_last = partial_owner((long long)tile * L.nkb + L.nkb - 1, U, L.n_ctas);
    unsigned bits = 0;
    for (int cc = c_first; cc <= c_last && cc - c_first < 32; ++cc)
      if ((int)((U * cc / L.n_ctas) / L.nkb) != tile) bits |= 1u << (cc - c_first);
    tab.first_and_count[tile] = c_first | ((c_last - c_first + 1) << 16);
    tab.slot_bits[tile] = bits;
  }
  __syncthreads();
}

// Sum over contributors of element (column `col`, output feature `n`).
__device__ __forceinline__ float partial_sum(const PartialLayout& L, const PartialTable& tab, int col, int n) {
  const int tile = n >> 7, nl = n & 127;
  const int fc = tab.first_and_count[tile];
  const int c_first = fc & 0xFFFF, count = fc >> 16;
  const unsigned bits = tab.slot_bits[tile];
  const float* base = L.ws + (size_t)col * 128 + nl;
  const size_t slot_floats = (size_t)L.acc_cols * 128;
  // all loads first (they are independent), then the sum in contributor order
  float v[PARTIAL_MAX_CONTRIB];
#pragma unroll
  for (int s = 0; s < PARTIAL_MAX_CONTRIB; ++s)
    v[s] = s < count ? __ldcg(base + (size_t)((c_first + s) * 2 + ((bits >> s) & 1)) * slot_floats) : 0.f;
  float acc = 0.f;
#pragma unroll
  for (int s = 0; s < PARTIAL_MAX_CONTRIB; ++s) acc += v[s];
  return acc;
}
