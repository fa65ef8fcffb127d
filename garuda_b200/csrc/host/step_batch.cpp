#include "step_batch.hpp"

#include <algorithm>
#include <sstream>
#include <unordered_set>

namespace garuda {

namespace {

int align4(int n) { return (n + 3) / 4 * 4; }

std::string list_of(const std::vector<int>& v) {
  std::ostringstream s;
  s << "[";
  for (size_t i = 0; i < v.size(); ++i) s << (i ? ", " : "") << v[i];
  s << "]";
  return s.str();
}

}  // namespace

StepBuilder::StepBuilder(CacheManager* cache, int vocab) : cache_(cache), vocab_(vocab) {
  if (cache_ == nullptr) throw StepError("the step function needs a cache");
  if (vocab_ < 1) throw StepError("the vocabulary must hold at least one token");
}

Reserved StepBuilder::check_and_reserve(const std::vector<StepRequest>& entries) {
  CacheManager& mgr = *cache_;
  if (entries.empty()) throw StepError("a step needs at least one entry");
  std::unordered_set<int64_t> seen;
  Reserved res;
  std::vector<int64_t> fresh, starting;
  for (const StepRequest& e : entries) {
    const std::string id = std::to_string(e.request);
    if (!seen.insert(e.request).second) throw StepError("request " + id + " appears twice in one step");
    const int64_t n = static_cast<int64_t>(e.tokens.size());
    if (n == 0) throw StepError("request " + id + " brings no tokens");
    for (int64_t t : e.tokens)
      if (t < 0 || t >= vocab_)
        throw StepError("token " + std::to_string(t) + " of request " + id + " is outside the vocabulary of " +
                        std::to_string(vocab_));
    for (int64_t w : e.want)
      if (w < 0 || w >= n)
        throw StepError("request " + id + " wants logits at place " + std::to_string(w) + " of " +
                        std::to_string(n) + " tokens");
    const bool known = mgr.known(e.request);
    const int old = known ? mgr.length(e.request) : 0;
    if (old + n > mgr.max_positions())
      throw StepError(std::to_string(n) + " tokens do not fit the " + std::to_string(mgr.max_positions()) +
                      "-position context (" + std::to_string(old) + " used) of request " + id);
    if (!known) fresh.push_back(e.request);
    if (old == 0) starting.push_back(e.request);
    res.new_lens.emplace_back(e.request, old + static_cast<int>(n));
  }
  if (static_cast<int>(fresh.size()) > mgr.free_slots())
    throw StepError(std::to_string(fresh.size()) + " new requests but only " + std::to_string(mgr.free_slots()) +
                    " request slots are free");
  for (int64_t r : fresh) mgr.acquire(r);
  try {
    if (!mgr.can_reserve(res.new_lens)) {
      std::vector<int> total(mgr.num_groups(), 0), free(mgr.num_groups(), 0);
      for (const auto& w : res.new_lens) {
        const std::vector<int> need = mgr.pages_needed(w.first, w.second);
        for (int g = 0; g < mgr.num_groups(); ++g) total[g] += need[g];
      }
      for (int g = 0; g < mgr.num_groups(); ++g) free[g] = mgr.free_pages(g);
      throw OutOfPages("the step needs " + list_of(total) + " pages per group but only " + list_of(free) + " are free");
    }
    for (const auto& w : res.new_lens) mgr.reserve(w.first, w.second);
  } catch (...) {
    for (int64_t r : fresh) mgr.release(r);
    throw;
  }
  // A request that starts at position 0 starts from zeroed fixed-size state, whoever took its slot
  // (this call just now, or a scheduler that admitted it or readmitted it after a preemption) and
  // whoever held the slot before: the caller zeroes these.
  for (int64_t r : starting) res.starting_slots.push_back(mgr.slot(r));
  return res;
}

void StepBuilder::commit(const std::vector<std::pair<int64_t, int>>& new_lens) {
  for (const auto& w : new_lens) cache_->commit(w.first, w.second);
}

BatchLayout StepBuilder::arrange(int tokens, int rows, int wanted) const {
  BatchLayout l;
  l.tokens = tokens, l.rows = rows, l.wanted = wanted;
  l.groups = cache_->num_groups();
  l.table_width = cache_->max_pages_per_request();
  int cursor = 0;
  auto place = [&cursor](int& at, int n) {
    at = cursor;
    cursor += align4(n);
  };
  place(l.token_ids, tokens);
  place(l.positions, tokens);
  place(l.token_req, tokens);
  place(l.cu_q, rows + 1);
  place(l.kv_lens, rows);
  place(l.slots, rows);
  place(l.logit_rows, std::max(wanted, 1));
  place(l.tables, l.groups * rows * l.table_width);
  l.words = cursor;
  return l;
}

BatchLayout StepBuilder::layout(const std::vector<StepRequest>& entries) const {
  int tokens = 0, wanted = 0;
  for (const StepRequest& e : entries) {
    tokens += static_cast<int>(e.tokens.size());
    wanted += static_cast<int>(e.want.size());
  }
  return arrange(tokens, static_cast<int>(entries.size()), wanted);
}

BatchLayout StepBuilder::decode_layout(int rows) const { return arrange(rows, rows, rows); }

void StepBuilder::fill(const std::vector<StepRequest>& entries,
                       const std::vector<std::pair<int64_t, int>>& new_lens, BatchLayout& l, int32_t* out) const {
  if (entries.size() != new_lens.size() || static_cast<int>(entries.size()) != l.rows)
    throw StepError("fill: the layout was made for another batch");
  const CacheManager& mgr = *cache_;
  int32_t* token_ids = out + l.token_ids;
  int32_t* positions = out + l.positions;
  int32_t* token_req = out + l.token_req;
  int32_t* cu_q = out + l.cu_q;
  int32_t* kv_lens = out + l.kv_lens;
  int32_t* slots = out + l.slots;
  int32_t* logit_rows = out + l.logit_rows;
  std::fill(logit_rows, logit_rows + std::max(l.wanted, 1), 0);
  int t = 0, w = 0;
  cu_q[0] = 0;
  l.max_q = l.max_kv = 0;
  l.min_q = 1 << 30;
  for (size_t i = 0; i < entries.size(); ++i) {
    const StepRequest& e = entries[i];
    const int n = static_cast<int>(e.tokens.size()), new_len = new_lens[i].second, start = new_len - n;
    if (t + n > l.tokens || w + static_cast<int>(e.want.size()) > l.wanted)
      throw StepError("fill: the layout was made for another batch");
    for (int j = 0; j < n; ++j) {
      token_ids[t + j] = static_cast<int32_t>(e.tokens[j]);
      positions[t + j] = start + j;
      token_req[t + j] = static_cast<int32_t>(i);
    }
    for (int64_t place : e.want) logit_rows[w++] = t + static_cast<int32_t>(place);
    t += n;
    cu_q[i + 1] = t;
    kv_lens[i] = new_len;
    slots[i] = mgr.slot(e.request);
    l.max_q = std::max(l.max_q, n);
    l.max_kv = std::max(l.max_kv, new_len);
    l.min_q = std::min(l.min_q, n);
  }
  for (int g = 0; g < l.groups; ++g)
    for (int i = 0; i < l.rows; ++i)
      mgr.block_table_row(entries[i].request, g, out + l.tables + (static_cast<size_t>(g) * l.rows + i) * l.table_width,
                          l.table_width);
}

void StepBuilder::fill_decode(const std::vector<StepRequest>& entries,
                              const std::vector<std::pair<int64_t, int>>& new_lens, const BatchLayout& l,
                              int32_t* out) const {
  const int live = static_cast<int>(entries.size());
  if (entries.size() != new_lens.size() || live > l.rows || l.tokens != l.rows)
    throw StepError("fill_decode: more requests than the layout has rows");
  const CacheManager& mgr = *cache_;
  for (int i = 0; i < l.rows; ++i) {
    out[l.token_ids + i] = 0;
    out[l.positions + i] = 0;
    out[l.token_req + i] = i;
    out[l.cu_q + i] = i;
    out[l.kv_lens + i] = 1;
    out[l.slots + i] = -1;          // padding rows have no state slot
    out[l.logit_rows + i] = i;
  }
  out[l.cu_q + l.rows] = l.rows;
  std::fill(out + l.tables, out + l.tables + static_cast<size_t>(l.groups) * l.rows * l.table_width, -1);
  for (int i = 0; i < live; ++i) {
    const StepRequest& e = entries[i];
    if (e.tokens.size() != 1) throw StepError("fill_decode: every request brings one token");
    const int new_len = new_lens[i].second;
    out[l.token_ids + i] = static_cast<int32_t>(e.tokens[0]);
    out[l.positions + i] = new_len - 1;
    out[l.kv_lens + i] = new_len;
    out[l.slots + i] = mgr.slot(e.request);
    for (int g = 0; g < l.groups; ++g)
      mgr.block_table_row(e.request, g, out + l.tables + (static_cast<size_t>(g) * l.rows + i) * l.table_width,
                          l.table_width);
  }
}

}  // namespace garuda
