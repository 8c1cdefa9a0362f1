// Host-side preparation of a step that is too hot for an interpreter: copying block-table
// rows into a staging buffer and cutting the decode attention work into balanced per-CTA
// lists.  Pointers are raw addresses of (pinned) host buffers owned by the caller.
#pragma once
#include <cstdint>
#include <vector>

#include "cache_manager.hpp"

namespace ferrum {

// dst[r * row_stride + i] = table(group, slots[r])[i] for i < width.
void copy_tables(const CacheManager& cache, int group, const std::vector<int>& slots, uintptr_t dst, int row_stride);

struct DecodePlan {
  int n_items = 0;    // work items written
  int n_ctas = 0;     // CTAs that own a non-empty share (before padding)
  int n_slots = 0;    // partial slots used
  int n_split_requests = 0;
};

// Balanced work lists for a batch in which every request brings ONE row tile (decoded
// tokens): the line of all (request, KV head, 64-key tile) units is cut into one equal share
// per CTA slot; a share is cut into items at (request, head) borders.  Writes, at `dst`
// (int32): work[item_cap][8], tile_info[R*Hkv][4], req_tile0[R], cta_items[cta_cap + 1], in
// this order, and returns the counts.  kv_lo/kv_hi give every request's key range.  When
// `pad` is set the work list is padded with empty items to item_cap and cta_items to
// cta_cap + 1 entries (fixed launch shapes for a captured graph).
DecodePlan build_decode_plan(const std::vector<int>& kv_lo, const std::vector<int>& kv_hi, int n_kv_heads, int cta_slots,
                             int min_tiles_per_cta, int item_cap, int cta_cap, bool pad, uintptr_t dst);

}  // namespace ferrum
