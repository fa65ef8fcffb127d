// The host half of the step function: a batch of (request, its next tokens, the places whose
// logits are wanted) is checked against the cache's bookkeeping, its pages are reserved, and the
// arrays that the kernels read are laid out in one buffer, which goes to the device in one copy.
//
// The reference's contract for a forward call (garuda/src/core/mod.rs:232-261): only positions
// not seen yet are consumed, an error and not a panic, and nothing is half-applied: a batch is
// checked before any cache is touched (garuda/src/llama/mod.rs:1160-1172, :1061-1067). Here a
// batch may mix portions of prompts with single decoded tokens, cut anywhere.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "cache_manager.hpp"

namespace garuda {

// A batch that was refused; no request and no page has changed.
struct StepError : std::invalid_argument {
  explicit StepError(const std::string& what) : std::invalid_argument(what) {}
};

struct StepRequest {
  int64_t request = 0;            // the caller's id of the request
  std::vector<int64_t> tokens;    // its next tokens, in order
  std::vector<int64_t> want;      // places among them whose logits are wanted
};

// Where each array lies in the buffer, in 32-bit words (every array starts on a multiple of
// four words, so that the device may read it in 16-byte pieces), and the batch's sizes.
//   token_ids[T], positions[T] (absolute: the request's length before the token,
//   garuda/src/llama/mod.rs:783), token_req[T] (row of the request within the batch),
//   cu_q[rows + 1] (prefix sums of the requests' token counts), kv_lens[rows] (length after the
//   step), slots[rows] (state slot; -1 in a padding row), logit_rows[max(W, 1)] (flat token rows
//   whose logits are wanted), tables[groups][rows][table_width] (page ids, -1 where none).
struct BatchLayout {
  int token_ids = 0, positions = 0, token_req = 0, cu_q = 0, kv_lens = 0, slots = 0, logit_rows = 0, tables = 0;
  int words = 0;           // the whole buffer
  int tokens = 0;          // T
  int rows = 0;            // request rows: the live requests, or a replayed decode step's padded count
  int wanted = 0;          // W
  int groups = 0, table_width = 0;
  int max_q = 0, max_kv = 0, min_q = 0;
};

struct Reserved {
  std::vector<std::pair<int64_t, int>> new_lens;   // (request, its length after the step), in the batch's order
  std::vector<int> starting_slots;                 // state slots of requests whose first token this step runs
};

class StepBuilder {
 public:
  StepBuilder(CacheManager* cache, int vocab);

  // Checks the whole batch, takes a slot for every request the cache does not know yet and
  // reserves every request's pages. Throws StepError or OutOfPages with nothing changed.
  Reserved check_and_reserve(const std::vector<StepRequest>& entries);
  // The step ran: every request now holds its new length.
  void commit(const std::vector<std::pair<int64_t, int>>& new_lens);

  // A step as it is: one row per entry.
  BatchLayout layout(const std::vector<StepRequest>& entries) const;
  // A step of single tokens padded to `rows` request rows (a captured graph's fixed shape).
  // Padding rows are requests of one token at position 0 with no page and no slot.
  BatchLayout decode_layout(int rows) const;

  // Writes the arrays; `out` holds at least layout.words words. Fills in max_q, max_kv, min_q.
  void fill(const std::vector<StepRequest>& entries, const std::vector<std::pair<int64_t, int>>& new_lens,
            BatchLayout& layout, int32_t* out) const;
  void fill_decode(const std::vector<StepRequest>& entries, const std::vector<std::pair<int64_t, int>>& new_lens,
                   const BatchLayout& layout, int32_t* out) const;

 private:
  BatchLayout arrange(int tokens, int rows, int wanted) const;

  CacheManager* cache_;
  int vocab_;
};

}  // namespace garuda
