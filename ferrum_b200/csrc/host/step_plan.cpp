#include "step_plan.hpp"

#include <algorithm>
#include <cstring>

namespace ferrum {

void copy_tables(const CacheManager& cache, int group, const std::vector<int>& slots, uintptr_t dst, int row_stride) {
  int32_t* out = reinterpret_cast<int32_t*>(dst);
  for (size_t r = 0; r < slots.size(); ++r) {
    const std::vector<int32_t>& row = cache.table(group, slots[r]);
    if ((int)row.size() > row_stride) throw CacheError("cache: block table row is wider than the staging buffer");
    std::memcpy(out + r * (size_t)row_stride, row.data(), row.size() * sizeof(int32_t));
  }
}

DecodePlan build_decode_plan(const std::vector<int>& kv_lo, const std::vector<int>& kv_hi, int Hkv, int cta_slots,
                             int min_tiles_per_cta, int item_cap, int cta_cap, bool pad, uintptr_t dst) {
  const int R = (int)kv_lo.size();
  if ((int)kv_hi.size() != R || Hkv <= 0 || cta_slots <= 0) throw CacheError("decode plan: bad arguments");
  int32_t* work = reinterpret_cast<int32_t*>(dst);
  int32_t* tile_info = work + (size_t)item_cap * 8;
  int32_t* req_tile0 = tile_info + (size_t)R * Hkv * 4;
  int32_t* cta_items = req_tile0 + R;

  std::vector<long long> kt(R);
  long long U = 0;
  for (int r = 0; r < R; ++r) {
    kt[r] = std::max(1, (kv_hi[r] - kv_lo[r] + 63) / 64);
    U += kt[r] * Hkv;
    req_tile0[r] = r;
  }
  const int P = (int)std::min<long long>(cta_slots, std::max<long long>(1, U / std::max(1, min_tiles_per_cta)));
  if (P > cta_cap) throw CacheError("decode plan: more CTAs than the capacity");
  // walk the pairs (request-major, head-minor) and the CTA bounds together
  int item = 0, slot = 0, cta = 0, split_requests = 0;
  long long pos = 0;  // position of the current pair's first unit on the line
  cta_items[0] = 0;
  long long next_bound = U / P;  // end of CTA 0's share: floor((c + 1) * U / P)
  for (int r = 0; r < R; ++r) {
    bool request_split = false;
    for (int h = 0; h < Hkv; ++h) {
      const long long pair_end = pos + kt[r];
      const int first_item = item;
      long long b = pos;
      while (b < pair_end) {
        const long long e = std::min(pair_end, next_bound);
        if (item >= item_cap) throw CacheError("decode plan: more items than the capacity");
        int32_t* w = work + (size_t)item * 8;
        w[0] = r;
        w[1] = 0;
        w[2] = kv_lo[r] + (int)(b - pos) * 64;
        w[3] = std::min<long long>(kv_hi[r], kv_lo[r] + (e - pos) * 64);
        w[6] = h;
        w[7] = 0;
        ++item;
        b = e;
        if (b == next_bound && cta + 1 < P) {
          ++cta;
          cta_items[cta] = item;
          next_bound = (long long)(cta + 1) * U / P;
        }
      }
      const int n = item - first_item;
      int32_t* info = tile_info + ((size_t)r * Hkv + h) * 4;
      info[0] = n > 1 ? slot : 0;
      info[1] = n;
      info[2] = 1;
      info[3] = 0;
      for (int i = first_item; i < item; ++i) {
        work[(size_t)i * 8 + 4] = n;
        work[(size_t)i * 8 + 5] = n > 1 ? slot++ : -1;
      }
      request_split |= n > 1;
      pos = pair_end;
    }
    split_requests += request_split;
  }
  cta_items[P] = item;
  DecodePlan out;
  out.n_items = item;
  out.n_ctas = P;
  out.n_slots = slot;
  out.n_split_requests = split_requests;
  if (pad) {
    std::memset(work + (size_t)item * 8, 0, (size_t)(item_cap - item) * 8 * sizeof(int32_t));
    for (int c = P + 1; c <= cta_cap; ++c) cta_items[c] = item;
  }
  return out;
}

}  // namespace ferrum
