#include "scheduler.hpp"

#include <algorithm>
#include <cmath>

namespace garuda {

std::string SamplingParams::problem() const {
  if (!std::isfinite(temperature) || temperature < 0.f)
    return "temperature must be a non-negative number, got " + std::to_string(temperature);
  if (!std::isfinite(top_p) || top_p <= 0.f || top_p > 1.f)
    return "top_p must be in (0, 1], got " + std::to_string(top_p);
  if (top_k < 0) return "top_k must not be negative, got " + std::to_string(top_k);
  if (max_tokens < 1) return "max_tokens must be at least 1";
  return "";
}

Scheduler::Scheduler(SchedulerConfig config, CacheManager* cache) : config_(config), cache_(cache) {
  if (config_.max_concurrent < 1) throw SchedulerError("max_concurrent must be at least 1");
  if (config_.queue_capacity < 1) throw SchedulerError("queue_capacity must be at least 1");
  if (config_.max_batch_tokens < 1) throw SchedulerError("max_batch_tokens must be at least 1");
  if (config_.prefill_chunk < 0) throw SchedulerError("prefill_chunk must not be negative");
  if (config_.max_context < 2) throw SchedulerError("max_context must be at least 2");
  if (config_.max_context > cache_->max_positions())
    throw SchedulerError("max_context exceeds the positions the cache can hold per request");
  if (config_.max_concurrent > cache_->max_requests())
    throw SchedulerError("max_concurrent exceeds the cache's request slots");
}

double Scheduler::now() const {
  if (manual_time_ >= 0.0) return manual_time_;
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - started_).count();
}

int64_t Scheduler::submit(std::vector<int32_t> prompt, SamplingParams params, int priority, double timeout_seconds) {
  const std::string bad = params.problem();
  if (!bad.empty()) throw SchedulerError(bad);
  if (!(timeout_seconds >= 0.0)) throw SchedulerError("a timeout must not be negative");
  if (prompt.empty()) throw SchedulerError("prompt is empty");
  if (static_cast<int>(prompt.size()) >= config_.max_context)
    throw SchedulerError("prompt of " + std::to_string(prompt.size()) + " tokens does not fit the " +
                         std::to_string(config_.max_context) + "-token context window");
  if (config_.vocab_size > 0)
    for (int32_t t : prompt)
      if (t < 0 || t >= config_.vocab_size)
        throw SchedulerError("token " + std::to_string(t) + " is outside the vocabulary");
  int waiting = 0;
  for (const auto& q : queue_) waiting += q.requeued ? 0 : 1;
  if (waiting >= config_.queue_capacity) {
    ++stats_.rejected_busy;
    throw Busy("the queue is full");
  }
  Request r;
  r.id = next_id_++;
  r.prompt_len = static_cast<int>(prompt.size());
  r.tokens = std::move(prompt);
  r.params = params;
  r.rng = Rng(params.has_seed ? params.seed : static_cast<uint64_t>(r.id));
  r.priority = priority;
  if (timeout_seconds > 0.0) r.deadline = now() + timeout_seconds;
  r.arrival = arrivals_++;
  auto pos = std::find_if(queue_.begin(), queue_.end(), [&](const Request& q) {
    return !q.requeued && q.priority < r.priority;
  });
  const int64_t id = r.id;
  queue_.insert(pos, std::move(r));
  ++stats_.submitted;
  return id;
}

void Scheduler::cancel(int64_t id) {
  for (auto& q : queue_)
    if (q.id == id) q.cancelled = true;
  for (auto& r : running_)
    if (r.id == id) r.cancelled = true;
}

void Scheduler::finish(Request& r, std::vector<Event>* events, EventKind kind, const std::string& detail) {
  if (cache_->known(r.id)) cache_->release(r.id);
  Event e;
  e.id = r.id;
  e.kind = kind;
  e.detail = detail;
  events->push_back(e);
  if (kind == EventKind::Done) ++stats_.completed;
  else if (detail == "cancelled") ++stats_.cancelled;
  else if (detail == "timeout") ++stats_.timed_out;
  else ++stats_.failed;
  const int64_t id = r.id;
  running_.erase(std::remove_if(running_.begin(), running_.end(),
                                [id](const Request& x) { return x.id == id; }),
                 running_.end());
}

bool Scheduler::preempt_most_recent(StepPlan* plan, int64_t* victim) {
  if (running_.empty()) return false;
  auto it = std::max_element(running_.begin(), running_.end(),
                             [](const Request& a, const Request& b) { return a.admitted < b.admitted; });
  Request r = std::move(*it);
  running_.erase(it);
  cache_->release(r.id);
  r.fed = 0;
  r.requeued = true;
  *victim = r.id;
  plan->preempted.push_back(r.id);
  ++stats_.preemptions;
  queue_.push_front(std::move(r));
  return true;
}

int Scheduler::largest_reservable(const Request& r, int want) const {
  const int ps = cache_->page_size();
  int c = want;
  while (c > 0 && !cache_->can_reserve({{r.id, r.fed + c}})) {
    // the longest length that needs one page fewer
    const int len = ((r.fed + c - 1) / ps) * ps;
    c = len - r.fed;
  }
  return std::max(c, 0);
}

StepPlan Scheduler::plan() {
  StepPlan plan;
  // requests that were cancelled since the last step, or whose time has run out
  // (garuda/src/scheduler/mod.rs:554-573, :607-633): waiting or running, they end here, between steps
  const double t = now();
  for (auto it = queue_.begin(); it != queue_.end();) {
    if (it->cancelled || t >= it->deadline) {
      Event e;
      e.id = it->id;
      e.kind = EventKind::Error;
      e.detail = it->cancelled ? "cancelled" : "timeout";
      plan.events.push_back(e);
      ++(it->cancelled ? stats_.cancelled : stats_.timed_out);
      if (cache_->known(it->id)) cache_->release(it->id);
      it = queue_.erase(it);
    } else {
      ++it;
    }
  }
  for (size_t i = 0; i < running_.size();) {
    if (running_[i].cancelled) finish(running_[i], &plan.events, EventKind::Error, "cancelled");
    else if (t >= running_[i].deadline) finish(running_[i], &plan.events, EventKind::Error, "timeout");
    else ++i;
  }

  const int chunk_cap = config_.prefill_chunk > 0 ? config_.prefill_chunk : config_.max_batch_tokens;
  auto add_entry = [&](Request& r, int count, bool decode = false) {
    PlanEntry e;
    e.id = r.id;
    e.decode = decode;
    e.slot = cache_->slot(r.id);
    e.start = r.fed;
    e.tokens.assign(r.tokens.begin() + r.fed, r.tokens.begin() + r.fed + count);
    e.sample = (r.fed + count == static_cast<int>(r.tokens.size()));
    e.temperature = r.params.temperature;
    e.top_p = r.params.top_p;
    e.top_k = r.params.top_k;
    plan.entries.push_back(std::move(e));
  };

  for (;;) {
    plan.entries.clear();
    int budget = config_.max_batch_tokens;
    bool again = false;

    // one token for every request that is decoding
    for (size_t i = 0; i < running_.size() && budget > 0; ++i) {
      Request& r = running_[i];
      if (static_cast<int>(r.tokens.size()) - r.fed != 1) continue;
      try {
        cache_->reserve(r.id, r.fed + 1);
      } catch (const OutOfPages&) {
        if (running_.size() == 1) {
          finish(r, &plan.events, EventKind::Error,
                 "the request needs more pages than the cache holds");
        } else {
          int64_t victim;
          preempt_most_recent(&plan, &victim);
        }
        again = true;
        break;
      }
      add_entry(r, 1, true);
      budget -= 1;
    }
    if (again) continue;
    // while something is decoding, a prompt's portion costs about one decode step
    const int portion_cap = config_.paced_prefill && !plan.entries.empty() ? std::min(chunk_cap, pacing_.chunk())
                                                                          : chunk_cap;

    // portions of the prompts that are still going in, in order of admission
    for (size_t i = 0; i < running_.size() && budget > 0; ++i) {
      Request& r = running_[i];
      const int remaining = static_cast<int>(r.tokens.size()) - r.fed;
      if (remaining <= 1) continue;
      const int want = std::min({remaining, budget, portion_cap});
      const int got = largest_reservable(r, want);
      if (got <= 0) continue;
      cache_->reserve(r.id, r.fed + got);
      add_entry(r, got);
      budget -= got;
    }

    // admission (garuda/src/scheduler/mod.rs:450-462): a slot and the pages of a first portion
    // A request that was sent back in this very plan waits for the next one, and
    // comes back only when all it holds so far fits: otherwise it would take the
    // pages it just gave up and be sent back again.
    while (plan.preempted.empty() && static_cast<int>(running_.size()) < config_.max_concurrent &&
           !queue_.empty() && budget > 0 && cache_->free_slots() > 0) {
      Request& q = queue_.front();
      const int want = std::min({static_cast<int>(q.tokens.size()), budget, portion_cap});
      cache_->acquire(q.id);
      int got = largest_reservable(q, want);
      if (q.requeued && !running_.empty() &&
          !cache_->can_reserve({{q.id, std::min(static_cast<int>(q.tokens.size()) + 1, config_.max_context)}}))
        got = 0;
      if (got < want && !(running_.empty() && got > 0)) {
        cache_->release(q.id);
        if (running_.empty()) {
          // nothing else holds pages, and not one token of it fits
          Event e;
          e.id = q.id;
          e.kind = EventKind::Error;
          e.detail = "the request needs more pages than the cache holds";
          plan.events.push_back(e);
          ++stats_.failed;
          queue_.pop_front();
          continue;
        }
        break;
      }
      Request r = std::move(q);
      queue_.pop_front();
      r.admitted = ++admissions_;
      r.requeued = false;
      cache_->reserve(r.id, r.fed + got);
      running_.push_back(std::move(r));
      add_entry(running_.back(), got);
      budget -= got;
    }

    if (plan.entries.empty() && !running_.empty()) {
      // every running request waits for pages that only another running request can free
      if (running_.size() == 1) {
        finish(running_[0], &plan.events, EventKind::Error,
               "the request needs more pages than the cache holds");
      } else {
        int64_t victim;
        preempt_most_recent(&plan, &victim);
      }
      continue;
    }
    break;
  }

  for (auto& e : plan.entries) {
    if (!e.sample || e.temperature == 0.f) continue;
    for (auto& r : running_)
      if (r.id == e.id) e.u = r.rng.next_f32();
  }
  if (!plan.entries.empty()) ++stats_.steps;
  return plan;
}

float Scheduler::peek_uniform(int64_t id) const {
  for (const auto& r : running_)
    if (r.id == id) {
      Rng copy = r.rng;
      return copy.next_f32();
    }
  throw SchedulerError("request " + std::to_string(id) + " is not running");
}

std::vector<Event> Scheduler::complete(const StepPlan& plan, const std::vector<int32_t>& sampled,
                                       double elapsed_seconds) {
  std::vector<Event> events;
  if (elapsed_seconds >= 0.0) {
    int decoded = 0, prompt = 0;
    for (const auto& e : plan.entries) (e.decode ? decoded : prompt) += static_cast<int>(e.tokens.size());
    if (prompt == 0 && decoded > 0) pacing_.observe_decode(elapsed_seconds);
    else if (decoded == 0) pacing_.observe_prefill(elapsed_seconds, prompt);
    else if (pacing_.decode_step >= 0.0 && elapsed_seconds > pacing_.decode_step)
      pacing_.observe_prefill(elapsed_seconds - pacing_.decode_step, prompt);
  }
  size_t wanted = 0;
  for (const auto& e : plan.entries) wanted += e.sample ? 1 : 0;
  if (sampled.size() != wanted)
    throw SchedulerError("the step returned " + std::to_string(sampled.size()) + " tokens for " +
                         std::to_string(wanted) + " sampling entries");
  size_t k = 0;
  for (const auto& e : plan.entries) {
    auto it = std::find_if(running_.begin(), running_.end(), [&](const Request& r) { return r.id == e.id; });
    const int32_t tok = e.sample ? sampled[k++] : -1;
    if (it == running_.end()) continue;
    Request& r = *it;
    const int new_len = e.start + static_cast<int>(e.tokens.size());
    if (cache_->length(r.id) < new_len) cache_->commit(r.id, new_len);
    r.fed = new_len;
    stats_.tokens_fed += e.tokens.size();
    if (!e.sample) continue;
    r.tokens.push_back(tok);
    ++r.generated;
    ++stats_.tokens_generated;
    // The end-of-sequence token joins the context but is not emitted
    // (garuda/src/runtime/mod.rs:733-738).
    if (!config_.ignore_eos && std::find(config_.eos_token_ids.begin(), config_.eos_token_ids.end(), tok) !=
                                   config_.eos_token_ids.end()) {
      finish(r, &events, EventKind::Done, "eos");
      continue;
    }
    Event t;
    t.id = r.id;
    t.kind = EventKind::Token;
    t.token = tok;
    events.push_back(t);
    // garuda/src/runtime/mod.rs:703-711
    if (r.generated >= r.params.max_tokens) finish(r, &events, EventKind::Done, "length");
    else if (static_cast<int>(r.tokens.size()) >= config_.max_context)
      finish(r, &events, EventKind::Done, "context_full");
  }
  return events;
}

std::vector<Event> Scheduler::fail(const StepPlan& plan, const std::string& message) {
  std::vector<Event> events;
  for (const auto& e : plan.entries) {
    auto it = std::find_if(running_.begin(), running_.end(), [&](const Request& r) { return r.id == e.id; });
    if (it != running_.end()) finish(*it, &events, EventKind::Error, message);
  }
  return events;
}

SchedulerStats Scheduler::stats() const {
  SchedulerStats s = stats_;
  s.running = static_cast<int>(running_.size());
  s.queued = static_cast<int>(queue_.size());
  return s;
}

}  // namespace garuda
