#include "cache_manager.hpp"

#include <algorithm>
#include <sstream>

namespace garuda {

CacheManager::CacheManager(std::vector<GroupConfig> groups, int page_size, int max_requests,
                           int max_positions)
    : groups_(std::move(groups)),
      page_size_(page_size),
      max_requests_(max_requests),
      max_positions_(max_positions) {
  if (page_size_ < 1) throw CacheError("page_size must be at least 1");
  if (max_requests_ < 1) throw CacheError("max_requests must be at least 1");
  if (max_positions_ < 1) throw CacheError("max_positions must be at least 1");
  max_pages_ = (max_positions_ + page_size_ - 1) / page_size_;
  for (const auto& g : groups_) {
    if (g.num_pages < 0) throw CacheError("a group cannot have a negative number of pages");
    if (g.window < 0) throw CacheError("a window cannot be negative");
    Pool pool;
    pool.free.reserve(g.num_pages);
    // Highest id at the bottom, so that page 0 is handed out first.
    for (int p = g.num_pages - 1; p >= 0; --p) pool.free.push_back(p);
    pool.used_before.assign(g.num_pages, 0);
    pools_.push_back(std::move(pool));
  }
  for (int s = max_requests_ - 1; s >= 0; --s) free_slots_.push_back(s);
}

const CacheManager::Request& CacheManager::get(int64_t request) const {
  auto it = requests_.find(request);
  if (it == requests_.end())
    throw CacheError("request " + std::to_string(request) + " is not known to the cache");
  return it->second;
}

CacheManager::Request& CacheManager::get(int64_t request) {
  return const_cast<Request&>(static_cast<const CacheManager*>(this)->get(request));
}

int CacheManager::first_live_position(int group, int len) const {
  const int w = groups_[group].window;
  if (w <= 0) return 0;
  // The next query sits at position `len` and reads [len + 1 - w, len].
  return std::max(0, len + 1 - w);
}

int CacheManager::acquire(int64_t request) {
  if (requests_.count(request))
    throw CacheError("request " + std::to_string(request) + " already holds a slot");
  if (free_slots_.empty()) throw CacheError("no request slot is free");
  Request r;
  r.slot = free_slots_.back();
  free_slots_.pop_back();
  r.tables.assign(groups_.size(), std::vector<int32_t>(max_pages_, -1));
  requests_.emplace(request, std::move(r));
  return requests_.at(request).slot;
}

std::vector<int> CacheManager::pages_needed(int64_t request, int new_len) const {
  const Request& r = get(request);
  std::vector<int> need(groups_.size(), 0);
  if (new_len > max_positions_)
    throw CacheError(std::to_string(new_len) + " positions do not fit the " +
                     std::to_string(max_positions_) + "-position context");
  const int last = (new_len + page_size_ - 1) / page_size_;
  for (size_t g = 0; g < groups_.size(); ++g) {
    for (int p = first_live_page(static_cast<int>(g), r.len); p < last; ++p)
      if (r.tables[g][p] < 0) ++need[g];
  }
  return need;
}

bool CacheManager::can_reserve(const std::vector<std::pair<int64_t, int>>& wants) const {
  std::vector<int> total(groups_.size(), 0);
  for (const auto& w : wants) {
    if (w.second > max_positions_) return false;
    auto need = pages_needed(w.first, w.second);
    for (size_t g = 0; g < need.size(); ++g) total[g] += need[g];
  }
  for (size_t g = 0; g < total.size(); ++g)
    if (total[g] > static_cast<int>(pools_[g].free.size())) return false;
  return true;
}

void CacheManager::reserve(int64_t request, int new_len) {
  Request& r = get(request);
  if (new_len < r.len) throw CacheError("a request cannot shrink");
  auto need = pages_needed(request, new_len);  // throws beyond max_positions
  for (size_t g = 0; g < need.size(); ++g) {
    if (need[g] > static_cast<int>(pools_[g].free.size())) {
      std::ostringstream m;
      m << "request " << request << " needs " << need[g] << " more pages of group " << g
        << " to reach " << new_len << " positions, but only " << pools_[g].free.size() << " are free";
      throw OutOfPages(m.str());
    }
  }
  const int last = (new_len + page_size_ - 1) / page_size_;
  for (size_t g = 0; g < groups_.size(); ++g) {
    Pool& pool = pools_[g];
    for (int p = first_live_page(static_cast<int>(g), r.len); p < last; ++p) {
      if (r.tables[g][p] >= 0) continue;
      const int32_t page = pool.free.back();
      pool.free.pop_back();
      r.tables[g][p] = page;
      ++pages_handed_out_;
      if (pool.used_before[page]) ++pages_reused_;
      pool.used_before[page] = 1;
    }
  }
  r.reserved = std::max(r.reserved, new_len);
}

void CacheManager::commit(int64_t request, int new_len) {
  Request& r = get(request);
  if (new_len < r.len) throw CacheError("a request cannot shrink");
  if (new_len > r.reserved)
    throw CacheError("request " + std::to_string(request) + " commits " + std::to_string(new_len) +
                     " positions but only " + std::to_string(r.reserved) + " are backed by pages");
  r.len = new_len;
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (groups_[g].window <= 0) continue;
    const int first = first_live_page(static_cast<int>(g), r.len);
    for (int p = 0; p < first && p < max_pages_; ++p) {
      if (r.tables[g][p] >= 0) {
        pools_[g].free.push_back(r.tables[g][p]);
        r.tables[g][p] = -1;
      }
    }
  }
}

void CacheManager::release(int64_t request) {
  Request& r = get(request);
  for (size_t g = 0; g < groups_.size(); ++g)
    for (int p = 0; p < max_pages_; ++p)
      if (r.tables[g][p] >= 0) pools_[g].free.push_back(r.tables[g][p]);
  free_slots_.push_back(r.slot);
  requests_.erase(request);
}

void CacheManager::block_table_row(int64_t request, int group, int32_t* out, int width) const {
  const Request& r = get(request);
  if (group < 0 || group >= static_cast<int>(groups_.size())) throw CacheError("no such group");
  const auto& t = r.tables[group];
  for (int p = 0; p < width; ++p) out[p] = p < max_pages_ ? t[p] : -1;
}

void CacheManager::check_invariants() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> seen(groups_[g].num_pages, 0);
    for (int32_t p : pools_[g].free) {
      if (p < 0 || p >= groups_[g].num_pages)
        throw CacheError("group " + std::to_string(g) + ": free list holds page id out of range");
      if (seen[p]++) throw CacheError("group " + std::to_string(g) + ": page " + std::to_string(p) + " is free twice");
    }
    for (const auto& kv : requests_) {
      for (int32_t p : kv.second.tables[g]) {
        if (p < 0) continue;
        if (p >= groups_[g].num_pages)
          throw CacheError("group " + std::to_string(g) + ": a table holds page id out of range");
        if (seen[p]++)
          throw CacheError("group " + std::to_string(g) + ": page " + std::to_string(p) +
                           " is held twice (or held and free)");
      }
    }
    for (int p = 0; p < groups_[g].num_pages; ++p)
      if (seen[p] != 1)
        throw CacheError("group " + std::to_string(g) + ": page " + std::to_string(p) + " is lost");
  }
  std::vector<int> slot_seen(max_requests_, 0);
  for (int s : free_slots_) {
    if (s < 0 || s >= max_requests_ || slot_seen[s]++) throw CacheError("slot free twice or out of range");
  }
  for (const auto& kv : requests_) {
    const int s = kv.second.slot;
    if (s < 0 || s >= max_requests_ || slot_seen[s]++) throw CacheError("slot held twice or out of range");
    if (kv.second.len > kv.second.reserved) throw CacheError("a request is longer than its pages");
  }
  for (int s = 0; s < max_requests_; ++s)
    if (slot_seen[s] != 1) throw CacheError("slot " + std::to_string(s) + " is lost");
}

}  // namespace garuda
