// Continuous batching with chunked prefill, on the host.
//
// The reference's loop (garuda/src/scheduler/mod.rs:400-508) admits requests up
// to max_concurrent (:450-462), feeds every pending prompt a paced chunk
// (:538-593) and then advances every active sequence by one token (:596-696),
// as separate forward calls. Here one plan describes one mixed step: one token
// for every request that is decoding, and under what is left of the token budget,
// portions of the prompts that are still going in.
//
// When pages run out (the reference has no shared pool; it bounds each sequence
// and spills to disk, garuda/src/cache/mod.rs:383-421): nothing is admitted; a
// prompt portion is cut to the pages there are; a decoding request that cannot
// get its next page makes the most recently admitted request give up its pages
// and go back to the head of the queue, to be recomputed from its prompt and
// what it had generated; a request that cannot fit even alone ends with an error.
#pragma once

#include <chrono>
#include <cstdint>
#include <deque>
#include <limits>
#include <string>
#include <vector>

#include "cache_manager.hpp"

namespace garuda {

// splitmix64, as garuda/src/runtime/mod.rs:64-84.
class Rng {
 public:
  explicit Rng(uint64_t seed = 0) : state_(seed ^ 0x9E3779B97F4A7C15ull) {}
  uint64_t next_u64() {
    state_ += 0x9E3779B97F4A7C15ull;
    uint64_t z = state_;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  // Uniform in [0, 1) with 24 bits.
  float next_f32() { return static_cast<float>(next_u64() >> 40) / static_cast<float>(1u << 24); }
  uint64_t state() const { return state_; }

 private:
  uint64_t state_;
};

// garuda/src/runtime/mod.rs:15-59.
struct SamplingParams {
  float temperature = 0.8f;  // 0: greedy
  float top_p = 0.95f;       // 1: off
  int top_k = 40;            // 0: off
  int max_tokens = 128;
  bool has_seed = false;     // without a seed the request id seeds the generator (:612)
  uint64_t seed = 0;
  // Empty if valid, else the reason (:42-59).
  std::string problem() const;
};

struct SchedulerConfig {
  int max_concurrent = 4;       // requests running at once (garuda/src/config/mod.rs:166-167)
  int queue_capacity = 256;     // waiting requests before submit is refused (:168-169)
  int max_batch_tokens = 2048;  // tokens of one step, decode tokens and prompt portions together
  int prefill_chunk = 512;      // most tokens of one prompt in one step (scheduler/mod.rs:321)
  int max_context = 2048;       // min(configured context, the model's own)
  std::vector<int32_t> eos_token_ids;  // generation ends on any of them; empty: none
  int vocab_size = 0;           // prompts are checked against it at submit; 0: unchecked
  bool ignore_eos = false;
  // While something is decoding, a prompt goes in by portions that cost about one decode step, from
  // running estimates of both costs (garuda/src/scheduler/mod.rs:305-370); off: prefill_chunk alone.
  bool paced_prefill = false;
};

// Running estimates of what a decode step and a prompt token cost (exponential moving averages,
// weight 0.25 on the newest sample), and the portion that balances them: decode step / prompt
// token, held to [1, 512]; 32 until both are known (garuda/src/scheduler/mod.rs:319-370).
struct Pacing {
  static constexpr double kAlpha = 0.25;
  static constexpr int kInitial = 32, kMin = 1, kMax = 512;
  double decode_step = -1.0;    // seconds; negative: not known yet
  double prefill_token = -1.0;  // seconds per token
  static void blend(double* slot, double sample) {
    *slot = *slot < 0.0 ? sample : *slot * (1.0 - kAlpha) + sample * kAlpha;
  }
  void observe_decode(double seconds) { blend(&decode_step, seconds); }
  void observe_prefill(double seconds, int tokens) {
    if (tokens > 0) blend(&prefill_token, seconds / tokens);
  }
  int chunk() const {
    if (decode_step < 0.0 || !(prefill_token > 0.0)) return kInitial;
    const double c = decode_step / prefill_token;
    return c < kMin ? kMin : c > kMax ? kMax : static_cast<int>(c);
  }
};

struct SchedulerError : std::runtime_error {
  explicit SchedulerError(const std::string& what) : std::runtime_error(what) {}
};
struct Busy : SchedulerError {  // garuda/src/scheduler/mod.rs:287-295
  explicit Busy(const std::string& what) : SchedulerError(what) {}
};

struct PlanEntry {
  int64_t id = 0;
  int slot = 0;
  int start = 0;                 // position of the first token
  std::vector<int32_t> tokens;   // the tokens this step feeds
  bool decode = false;           // the request is decoding: this is its one next token
  bool sample = false;           // logits of the last token are wanted and a token is drawn
  float temperature = 0.f, top_p = 1.f;
  int top_k = 0;
  float u = 0.f;                 // the uniform draw for this token, from the request's generator
};

enum class EventKind { Token, Done, Error };

struct Event {
  int64_t id = 0;
  EventKind kind = EventKind::Token;
  int32_t token = -1;
  std::string detail;  // Done: "length" | "context_full" | "eos"; Error: the message ("cancelled", "timeout", ...)
};

struct StepPlan {
  std::vector<PlanEntry> entries;
  std::vector<int64_t> preempted;  // requests sent back to the queue while planning
  std::vector<Event> events;       // errors and cancellations decided while planning
  int num_tokens() const {
    int n = 0;
    for (const auto& e : entries) n += static_cast<int>(e.tokens.size());
    return n;
  }
};

struct SchedulerStats {  // garuda/src/scheduler/mod.rs:188-197, and what a page pool adds
  uint64_t submitted = 0, completed = 0, cancelled = 0, timed_out = 0, failed = 0, rejected_busy = 0;
  uint64_t preemptions = 0, steps = 0, tokens_fed = 0, tokens_generated = 0;
  int running = 0, queued = 0;
};

class Scheduler {
 public:
  Scheduler(SchedulerConfig config, CacheManager* cache);

  // Validates (garuda/src/runtime/mod.rs:578-589) and queues. priority: higher first, FIFO within.
  // timeout_seconds: the request ends with the error "timeout" at the first plan made that long
  // after it was submitted, waiting or running (the deadline is submission time + timeout and is
  // checked between steps: garuda/src/scheduler/mod.rs:520, :566-573, :623-631); 0: no limit.
  int64_t submit(std::vector<int32_t> prompt, SamplingParams params, int priority = 0, double timeout_seconds = 0.0);
  void cancel(int64_t id);
  // Decide the next step. Reserves the pages its entries need.
  StepPlan plan();
  // Seconds on the scheduler's clock: a steady clock that starts with the scheduler, or, once
  // set_time was called, the time given last (for tests and for replaying a schedule).
  double now() const;
  void set_time(double seconds) { manual_time_ = seconds; }
  // The uniform draw that the next plan will give a running request's sampling entry (its
  // generator is not advanced): for a decode step that is launched before that plan is made.
  float peek_uniform(int64_t id) const;
  // The step ran; `sampled` holds one token per entry with sample == true, in order.
  // elapsed_seconds: what the step took, for the pacing of prompt portions (negative: not measured).
  // A step of decode tokens only is a sample of the decode step's cost; a step of prompt tokens
  // only, of a prompt token's; a mixed step's time beyond the decode step's estimate is its prompt
  // tokens' (the reference times its two calls apart: garuda/src/scheduler/mod.rs:481-491).
  std::vector<Event> complete(const StepPlan& plan, const std::vector<int32_t>& sampled,
                              double elapsed_seconds = -1.0);
  const Pacing& pacing() const { return pacing_; }
  // The step failed: every request of the plan ends with this error.
  std::vector<Event> fail(const StepPlan& plan, const std::string& message);
  bool idle() const { return running_.empty() && queue_.empty(); }
  SchedulerStats stats() const;
  const SchedulerConfig& config() const { return config_; }

 private:
  struct Request {
    int64_t id = 0;
    std::vector<int32_t> tokens;  // prompt, then what was generated
    int prompt_len = 0;
    int fed = 0;                  // tokens whose positions are in the cache
    int generated = 0;
    SamplingParams params;
    Rng rng;
    int priority = 0;
    uint64_t arrival = 0;
    uint64_t admitted = 0;        // order of admission; larger is more recent
    bool cancelled = false;
    bool requeued = false;        // preempted: goes before every fresh request
    double deadline = std::numeric_limits<double>::infinity();   // on the scheduler's clock
  };

  void finish(Request& r, std::vector<Event>* events, EventKind kind, const std::string& detail);
  bool preempt_most_recent(StepPlan* plan, int64_t* victim);
  int largest_reservable(const Request& r, int want) const;

  SchedulerConfig config_;
  CacheManager* cache_;
  std::deque<Request> queue_;          // kept ordered: requeued first, then priority desc, arrival asc
  std::vector<Request> running_;       // in admission order
  int64_t next_id_ = 1;
  uint64_t arrivals_ = 0, admissions_ = 0;
  SchedulerStats stats_;
  Pacing pacing_;
  std::chrono::steady_clock::time_point started_ = std::chrono::steady_clock::now();
  double manual_time_ = -1.0;          // negative: the steady clock
};

}  // namespace garuda
