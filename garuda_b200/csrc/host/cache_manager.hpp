// Paged cache bookkeeping on the host: pages, block tables, request slots.
//
// The reference keeps, per sequence and per layer, a map from block index to a
// block of 32 positions (garuda/src/cache/mod.rs:145-150, :221-241) and grows it
// lazily on append (:348-378); memory is bounded by a per-sequence position cap
// and by how many sequences run. Here all requests draw pages from one pool per
// group of layers, and a request's block table says which page holds which
// stretch of its positions. A group is a set of layers with the same needs
// (all keys, or a window of them: garuda/src/cache/mod.rs:333-338); groups have
// pages of their own because a windowed group gives pages back while the
// request is still running.
//
// Only numbers live here. The device memory behind the pages belongs to the
// Python side, which indexes it with the page ids handed out below.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace garuda {

struct CacheError : std::runtime_error {
  explicit CacheError(const std::string& what) : std::runtime_error(what) {}
};

// Raised when a reservation cannot be met; nothing has changed when it is thrown.
struct OutOfPages : CacheError {
  explicit OutOfPages(const std::string& what) : CacheError(what) {}
};

struct GroupConfig {
  int num_pages = 0;   // pages in this group's pool
  int window = 0;      // positions a query looks back over, itself included; 0: everything
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupConfig> groups, int page_size, int max_requests, int max_positions);

  // ---- request lifecycle -------------------------------------------------
  // A new request: takes a state slot. Throws if the id is known or no slot is free.
  int acquire(int64_t request);
  // Pages needed, per group, to take `request` from its length to `new_len`.
  std::vector<int> pages_needed(int64_t request, int new_len) const;
  // True if every (request, new_len) pair of a step can be reserved together.
  bool can_reserve(const std::vector<std::pair<int64_t, int>>& wants) const;
  // Back every live position below `new_len` with a page, in every group.
  // All or nothing: on OutOfPages (or a length beyond max_positions) nothing changed.
  void reserve(int64_t request, int new_len);
  // The step ran: the request now holds `new_len` positions. Pages that every
  // later query's window has passed go back to their pool.
  void commit(int64_t request, int new_len);
  // Everything the request holds goes back: pages (most recently used first,
  // so that they are handed out again at once) and the slot.
  void release(int64_t request);

  // ---- queries -------------------------------------------------------------
  bool known(int64_t request) const { return requests_.count(request) != 0; }
  int length(int64_t request) const { return get(request).len; }
  int slot(int64_t request) const { return get(request).slot; }
  int reserved_length(int64_t request) const { return get(request).reserved; }
  // Row of the block table: page id per stretch of page_size positions, -1 where none.
  void block_table_row(int64_t request, int group, int32_t* out, int width) const;
  int num_groups() const { return static_cast<int>(groups_.size()); }
  int page_size() const { return page_size_; }
  int max_pages_per_request() const { return max_pages_; }
  int max_positions() const { return max_positions_; }
  int max_requests() const { return max_requests_; }
  int free_pages(int group) const { return static_cast<int>(pools_[group].free.size()); }
  int total_pages(int group) const { return groups_[group].num_pages; }
  int free_slots() const { return static_cast<int>(free_slots_.size()); }
  int live_requests() const { return static_cast<int>(requests_.size()); }
  const GroupConfig& group(int g) const { return groups_[g]; }
  // First position that a query at position `len` (the next token) still reads.
  int first_live_position(int group, int len) const;
  // Throws CacheError naming the first violated invariant: every page is either
  // free or held by exactly one (request, group, index); no page is free twice.
  void check_invariants() const;
  uint64_t pages_handed_out() const { return pages_handed_out_; }
  uint64_t pages_reused() const { return pages_reused_; }

 private:
  struct Request {
    int slot = -1;
    int len = 0;        // positions committed
    int reserved = 0;   // positions backed by pages (>= len)
    // tables[group][logical page] = page id or -1
    std::vector<std::vector<int32_t>> tables;
  };
  struct Pool {
    std::vector<int32_t> free;        // stack: back() is handed out next
    std::vector<uint8_t> used_before; // page id -> has been handed out at least once
  };

  const Request& get(int64_t request) const;
  Request& get(int64_t request);
  int first_live_page(int group, int len) const { return first_live_position(group, len) / page_size_; }

  std::vector<GroupConfig> groups_;
  int page_size_, max_requests_, max_positions_, max_pages_;
  std::vector<Pool> pools_;
  std::vector<int> free_slots_;
  std::unordered_map<int64_t, Request> requests_;
  uint64_t pages_handed_out_ = 0, pages_reused_ = 0;
};

}  // namespace garuda
