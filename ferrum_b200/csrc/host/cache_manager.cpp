#include "cache_manager.hpp"

#include <algorithm>

namespace ferrum {

CacheManager::CacheManager(std::vector<GroupSpec> groups, int max_requests)
    : groups_(std::move(groups)), max_requests_(max_requests) {
  if (max_requests_ <= 0) throw CacheError("cache: max_requests must be positive");
  for (auto& g : groups_) {
    if (g.page_size <= 0 || g.num_pages <= 0 || g.table_width <= 0 || g.window < 0)
      throw CacheError("cache: a group dimension is zero or negative");
  }
  reqs_.resize(max_requests_);
  for (auto& r : reqs_) {
    r.tables.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) r.tables[g].assign(groups_[g].table_width, -1);
  }
  // LIFO stacks; popping from the back hands out slot 0 / page 0 first
  for (int s = max_requests_ - 1; s >= 0; --s) free_slots_.push_back(s);
  free_.resize(groups_.size());
  in_use_.resize(groups_.size());
  for (size_t g = 0; g < groups_.size(); ++g) {
    for (int p = groups_[g].num_pages - 1; p >= 0; --p) free_[g].push_back(p);
    in_use_[g].assign(groups_[g].num_pages, 0);
  }
}

void CacheManager::check_slot(int slot) const {
  if (slot < 0 || slot >= max_requests_) throw CacheError("cache: slot id out of range");
  if (!reqs_[slot].open) throw CacheError("cache: slot is not open");
}

bool CacheManager::is_open(int slot) const { return slot >= 0 && slot < max_requests_ && reqs_[slot].open; }

int CacheManager::open() {
  if (free_slots_.empty()) throw Unavailable("no free request slots");
  const int slot = free_slots_.back();
  free_slots_.pop_back();
  Req& r = reqs_[slot];
  r.open = true;
  r.seq_len = 0;
  return slot;
}

void CacheManager::close(int slot) {
  if (slot < 0 || slot >= max_requests_ || !reqs_[slot].open) throw CacheError("cache: free of a slot that is not open");
  Req& r = reqs_[slot];
  for (size_t g = 0; g < groups_.size(); ++g) {
    for (auto& p : r.tables[g]) {
      if (p >= 0) {
        if (!in_use_[g][p]) throw CacheError("cache: page freed twice");
        in_use_[g][p] = 0;
        free_[g].push_back(p);
        p = -1;
      }
    }
  }
  r.open = false;
  r.seq_len = 0;
  free_slots_.push_back(slot);
}

int CacheManager::first_needed_page(int g, int pos0) const {
  const GroupSpec& s = groups_[g];
  if (s.window <= 0) return 0;
  const int lo = std::max(0, pos0 - s.window + 1);  // oldest key the query at pos0 reads
  return lo / s.page_size;
}

std::vector<int> CacheManager::pages_missing(int slot, int new_len) const {
  check_slot(slot);
  const Req& r = reqs_[slot];
  std::vector<int> need(groups_.size(), 0);
  if (new_len <= r.seq_len) return need;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& s = groups_[g];
    const int last = (new_len - 1) / s.page_size;
    if (last >= s.table_width) throw CacheError("cache: sequence length exceeds the block table");
    for (int lp = first_needed_page((int)g, r.seq_len); lp <= last; ++lp)
      if (r.tables[g][lp] < 0) ++need[g];
  }
  return need;
}

bool CacheManager::can_grow(int slot, int new_len) const {
  const auto need = pages_missing(slot, new_len);
  for (size_t g = 0; g < groups_.size(); ++g)
    if (need[g] > (int)free_[g].size()) return false;
  return true;
}

void CacheManager::grow(int slot, int new_len) {
  if (!can_grow(slot, new_len)) throw Unavailable("no free pages");
  Req& r = reqs_[slot];
  if (new_len <= r.seq_len) return;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& s = groups_[g];
    const int last = (new_len - 1) / s.page_size;
    for (int lp = first_needed_page((int)g, r.seq_len); lp <= last; ++lp) {
      if (r.tables[g][lp] >= 0) continue;
      const int p = free_[g].back();
      free_[g].pop_back();
      if (in_use_[g][p]) throw CacheError("cache: page handed out twice");
      in_use_[g][p] = 1;
      r.tables[g][lp] = p;
    }
  }
}

void CacheManager::commit(int slot, int new_len) {
  check_slot(slot);
  Req& r = reqs_[slot];
  if (new_len < r.seq_len) throw CacheError("cache: commit would shorten the sequence");
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& s = groups_[g];
    if (new_len > 0 && (new_len - 1) / s.page_size >= s.table_width)
      throw CacheError("cache: sequence length exceeds the block table");
    const int last = new_len > 0 ? (new_len - 1) / s.page_size : -1;
    for (int lp = first_needed_page((int)g, r.seq_len); lp <= last; ++lp)
      if (r.tables[g][lp] < 0) throw CacheError("cache: commit of positions that hold no page");
  }
  r.seq_len = new_len;
  // pages that no later query reaches: the next query stands at new_len
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int keep_from = first_needed_page((int)g, new_len);
    for (int lp = 0; lp < keep_from; ++lp) {
      int32_t& p = r.tables[g][lp];
      if (p >= 0) {
        in_use_[g][p] = 0;
        free_[g].push_back(p);
        p = -1;
      }
    }
  }
}

int CacheManager::max_growable(int slot, int want) const {
  check_slot(slot);
  const Req& r = reqs_[slot];
  if (want <= r.seq_len) return r.seq_len;
  if (can_grow(slot, want)) return want;
  int lo = r.seq_len, hi = want;  // can_grow(lo) holds, can_grow(hi) does not
  while (hi - lo > 1) {
    const int mid = lo + (hi - lo) / 2;
    if (can_grow(slot, mid)) lo = mid; else hi = mid;
  }
  return lo;
}

int CacheManager::seq_len(int slot) const {
  check_slot(slot);
  return reqs_[slot].seq_len;
}

int CacheManager::pages_held(int g, int slot) const {
  check_slot(slot);
  int n = 0;
  for (auto p : reqs_[slot].tables.at(g)) n += p >= 0;
  return n;
}

const std::vector<int32_t>& CacheManager::table(int g, int slot) const {
  check_slot(slot);
  return reqs_[slot].tables.at(g);
}

std::string CacheManager::check() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> seen(groups_[g].num_pages, 0);
    for (auto p : free_[g]) {
      if (p < 0 || p >= groups_[g].num_pages) return "free list holds an invalid page id";
      if (seen[p]++) return "page is twice in the free list";
      if (in_use_[g][p]) return "free page is marked in use";
    }
    for (int s = 0; s < max_requests_; ++s) {
      for (auto p : reqs_[s].tables[g]) {
        if (p < 0) continue;
        if (!reqs_[s].open) return "closed slot holds a page";
        if (p >= groups_[g].num_pages) return "table holds an invalid page id";
        if (seen[p]++) return "page is held twice";
        if (!in_use_[g][p]) return "held page is not marked in use";
      }
    }
    for (int p = 0; p < groups_[g].num_pages; ++p)
      if (!seen[p]) return "page lost: neither free nor held";
  }
  std::vector<int> slot_seen(max_requests_, 0);
  for (auto s : free_slots_) {
    if (s < 0 || s >= max_requests_ || slot_seen[s]++) return "slot free list is corrupt";
    if (reqs_[s].open) return "free slot is open";
  }
  for (int s = 0; s < max_requests_; ++s)
    if (!reqs_[s].open && !slot_seen[s]) return "slot lost: neither free nor open";
  return "";
}

long long CacheManager::capacity_tokens() const {
  long long cap = -1;
  for (auto& g : groups_) {
    long long c = (long long)std::min(g.num_pages, g.table_width) * g.page_size;
    if (g.window > 0) c = (long long)g.table_width * g.page_size;  // windowed groups recycle their pages
    if (cap < 0 || c < cap) cap = c;
  }
  return cap < 0 ? 0 : cap;
}

}  // namespace ferrum
