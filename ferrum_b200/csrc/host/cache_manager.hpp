// Paged cache bookkeeping: which page of which pool holds which positions of which request.
//
// The reference keeps one dense region per sequence ("slot") and finds a position by
// offset arithmetic (crates/kvcache/src/pool.rs:52-71).  Here the unit is a page of
// `page_size` positions.  Layers with the same needs form a group; every group has its own
// pool of pages and every request has one block table per group (logical page -> page id,
// -1 where it holds none).  A group with a window gives pages back as soon as no later
// query can reach them.  Beside the pages, every request owns one slot id, which indexes
// arrays of fixed-size per-request state.
//
// The manager owns integers only; the device memory the page ids index belongs to the caller.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace ferrum {

struct Unavailable : std::runtime_error { using std::runtime_error::runtime_error; };
struct CacheError : std::runtime_error { using std::runtime_error::runtime_error; };

struct GroupSpec {
  int page_size = 16;
  int window = 0;       // 0: every key is kept; w > 0: a query at p reads keys in (p - w, p]
  int num_pages = 0;
  int table_width = 0;  // logical pages a request may address
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, int max_requests);

  int n_groups() const { return (int)groups_.size(); }
  const GroupSpec& group(int g) const { return groups_.at(g); }
  int max_requests() const { return max_requests_; }

  // A new request: returns its slot id.  Throws Unavailable when every slot is taken
  // (the reference's "no free kv slots", crates/kvcache/src/pool.rs:83-88).
  int open();
  // Gives back the slot and every page it holds.  Closing twice is a CacheError
  // (crates/kvcache/src/pool.rs:103-112).
  void close(int slot);
  bool is_open(int slot) const;

  // Pages that `grow(slot, new_len)` would have to take, per group.
  std::vector<int> pages_missing(int slot, int new_len) const;
  bool can_grow(int slot, int new_len) const;
  // Makes sure the request holds every page that a step bringing positions
  // [seq_len, new_len) reads or writes.  All groups or nothing; throws Unavailable.
  void grow(int slot, int new_len);
  // The step ran: the request now holds new_len positions.  Pages a window has passed
  // go back to their pool.
  void commit(int slot, int new_len);
  // Largest new_len <= want that grow() can satisfy right now (>= seq_len).
  int max_growable(int slot, int want) const;

  int seq_len(int slot) const;
  int free_pages(int g) const { return (int)free_.at(g).size(); }
  int used_pages(int g) const { return groups_.at(g).num_pages - free_pages(g); }
  int free_slots() const { return (int)free_slots_.size(); }
  int pages_held(int g, int slot) const;
  const std::vector<int32_t>& table(int g, int slot) const;

  // Consistency: every page is either free or in exactly one table; returns a message
  // describing the first violation, or an empty string.
  std::string check() const;

  // Tokens a single request can hold when it has the cache to itself.
  long long capacity_tokens() const;

 private:
  struct Req {
    bool open = false;
    int seq_len = 0;
    std::vector<std::vector<int32_t>> tables;  // [group][logical page]
  };
  void check_slot(int slot) const;
  // first logical page a step starting at position pos0 still needs in group g
  int first_needed_page(int g, int pos0) const;

  std::vector<GroupSpec> groups_;
  int max_requests_;
  std::vector<Req> reqs_;
  std::vector<int> free_slots_;              // LIFO
  std::vector<std::vector<int32_t>> free_;   // per group, LIFO stack of page ids
  std::vector<std::vector<uint8_t>> in_use_; // per group, per page
};

}  // namespace ferrum
