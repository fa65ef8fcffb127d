// Python bindings of the host runtime: cache manager, step batches, scheduler, generator.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"
#include "step_batch.hpp"

namespace py = pybind11;
using namespace garuda;

namespace {

// A batch from Python, converted once for the check and for the arrays: any sequence of objects
// with `request`, `tokens` and `want`.
struct StepRequests {
  std::vector<StepRequest> items;
};

StepRequests step_requests(const py::sequence& entries) {
  StepRequests out;
  out.items.reserve(py::len(entries));
  try {
    for (const py::handle& e : entries) {
      StepRequest r;
      r.request = e.attr("request").cast<int64_t>();
      for (const py::handle& t : e.attr("tokens")) r.tokens.push_back(t.cast<int64_t>());
      for (const py::handle& w : e.attr("want")) r.want.push_back(w.cast<int64_t>());
      out.items.push_back(std::move(r));
    }
  } catch (const py::cast_error&) {
    throw StepError("a step's request ids, tokens and wanted places must be integers");
  }
  return out;
}

int32_t* words_of(py::array_t<int32_t, py::array::c_style>& buffer, int needed) {
  if (buffer.ndim() != 1 || buffer.shape(0) < needed)
    throw StepError("the batch's buffer holds " + std::to_string(buffer.size()) + " words, the batch needs " +
                    std::to_string(needed));
  return buffer.mutable_data();
}

}  // namespace

PYBIND11_MODULE(_garuda_host, m) {
  m.doc() = "garuda_b200 host runtime: paged-cache bookkeeping, scheduler, splitmix64";

  py::register_exception<CacheError>(m, "CacheError");
  py::register_exception<OutOfPages>(m, "OutOfPages", m.attr("CacheError").ptr());
  py::register_exception<SchedulerError>(m, "SchedulerError");
  py::register_exception<Busy>(m, "Busy", m.attr("SchedulerError").ptr());

  py::class_<GroupConfig>(m, "GroupConfig")
      .def(py::init([](int num_pages, int window) {
             GroupConfig g;
             g.num_pages = num_pages;
             g.window = window;
             return g;
           }),
           py::arg("num_pages"), py::arg("window") = 0)
      .def_readwrite("num_pages", &GroupConfig::num_pages)
      .def_readwrite("window", &GroupConfig::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupConfig>, int, int, int>(), py::arg("groups"), py::arg("page_size"),
           py::arg("max_requests"), py::arg("max_positions"))
      .def("acquire", &CacheManager::acquire)
      .def("pages_needed", &CacheManager::pages_needed)
      .def("can_reserve", &CacheManager::can_reserve)
      .def("reserve", &CacheManager::reserve)
      .def("commit", &CacheManager::commit)
      .def("release", &CacheManager::release)
      .def("known", &CacheManager::known)
      .def("length", &CacheManager::length)
      .def("slot", &CacheManager::slot)
      .def("reserved_length", &CacheManager::reserved_length)
      .def("block_table_row",
           [](const CacheManager& c, int64_t request, int group) {
             py::array_t<int32_t> out(c.max_pages_per_request());
             c.block_table_row(request, group, out.mutable_data(), c.max_pages_per_request());
             return out;
           })
      .def("fill_block_tables",
           // out: int32 [groups, rows, width]; row i is request ids[i]
           [](const CacheManager& c, const std::vector<int64_t>& ids,
              py::array_t<int32_t, py::array::c_style> out) {
             auto buf = out.mutable_unchecked<3>();
             if (buf.shape(0) != c.num_groups() || buf.shape(1) < static_cast<py::ssize_t>(ids.size()))
               throw CacheError("fill_block_tables: output has the wrong shape");
             const int width = static_cast<int>(buf.shape(2));
             for (int g = 0; g < c.num_groups(); ++g)
               for (size_t i = 0; i < ids.size(); ++i)
                 c.block_table_row(ids[i], g, &buf(g, i, 0), width);
           })
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def_property_readonly("page_size", &CacheManager::page_size)
      .def_property_readonly("max_pages_per_request", &CacheManager::max_pages_per_request)
      .def_property_readonly("max_positions", &CacheManager::max_positions)
      .def_property_readonly("max_requests", &CacheManager::max_requests)
      .def("free_pages", &CacheManager::free_pages)
      .def("total_pages", &CacheManager::total_pages)
      .def("window", [](const CacheManager& c, int g) { return c.group(g).window; })
      .def_property_readonly("free_slots", &CacheManager::free_slots)
      .def_property_readonly("live_requests", &CacheManager::live_requests)
      .def("first_live_position", &CacheManager::first_live_position)
      .def("check_invariants", &CacheManager::check_invariants)
      .def_property_readonly("pages_handed_out", &CacheManager::pages_handed_out)
      .def_property_readonly("pages_reused", &CacheManager::pages_reused);

  py::register_exception<StepError>(m, "StepError", PyExc_ValueError);

  py::class_<StepRequests>(m, "StepRequests")
      .def(py::init(&step_requests), py::arg("entries"))
      .def("__len__", [](const StepRequests& v) { return v.items.size(); })
      .def_property_readonly("requests", [](const StepRequests& v) {
        std::vector<int64_t> ids;
        for (const StepRequest& r : v.items) ids.push_back(r.request);
        return ids;
      });

  py::class_<BatchLayout>(m, "BatchLayout")
      .def_readonly("token_ids", &BatchLayout::token_ids)
      .def_readonly("positions", &BatchLayout::positions)
      .def_readonly("token_req", &BatchLayout::token_req)
      .def_readonly("cu_q", &BatchLayout::cu_q)
      .def_readonly("kv_lens", &BatchLayout::kv_lens)
      .def_readonly("slots", &BatchLayout::slots)
      .def_readonly("logit_rows", &BatchLayout::logit_rows)
      .def_readonly("tables", &BatchLayout::tables)
      .def_readonly("words", &BatchLayout::words)
      .def_readonly("tokens", &BatchLayout::tokens)
      .def_readonly("rows", &BatchLayout::rows)
      .def_readonly("wanted", &BatchLayout::wanted)
      .def_readonly("groups", &BatchLayout::groups)
      .def_readonly("table_width", &BatchLayout::table_width)
      .def_readonly("max_q", &BatchLayout::max_q)
      .def_readonly("max_kv", &BatchLayout::max_kv)
      .def_readonly("min_q", &BatchLayout::min_q);

  py::class_<Reserved>(m, "Reserved")
      .def_readonly("new_lens", &Reserved::new_lens)
      .def_readonly("starting_slots", &Reserved::starting_slots);

  py::class_<StepBuilder>(m, "StepBuilder")
      .def(py::init<CacheManager*, int>(), py::arg("cache"), py::arg("vocab"), py::keep_alive<1, 2>())
      .def("check_and_reserve", [](StepBuilder& b, const StepRequests& entries) { return b.check_and_reserve(entries.items); })
      .def("commit", &StepBuilder::commit)
      .def("layout", [](const StepBuilder& b, const StepRequests& entries) { return b.layout(entries.items); })
      .def("decode_layout", &StepBuilder::decode_layout)
      .def("fill",
           [](const StepBuilder& b, const StepRequests& entries,
              const std::vector<std::pair<int64_t, int>>& new_lens, BatchLayout& layout,
              py::array_t<int32_t, py::array::c_style> buffer) {
             b.fill(entries.items, new_lens, layout, words_of(buffer, layout.words));
           })
      .def("fill_decode",
           [](const StepBuilder& b, const StepRequests& entries,
              const std::vector<std::pair<int64_t, int>>& new_lens, const BatchLayout& layout,
              py::array_t<int32_t, py::array::c_style> buffer) {
             b.fill_decode(entries.items, new_lens, layout, words_of(buffer, layout.words));
           });

  py::class_<Rng>(m, "Rng")
      .def(py::init<uint64_t>(), py::arg("seed") = 0)
      .def("next_u64", &Rng::next_u64)
      .def("next_f32", &Rng::next_f32)
      .def_property_readonly("state", &Rng::state);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](float temperature, float top_p, int top_k, int max_tokens, py::object seed) {
             SamplingParams p;
             p.temperature = temperature;
             p.top_p = top_p;
             p.top_k = top_k;
             p.max_tokens = max_tokens;
             p.has_seed = !seed.is_none();
             p.seed = seed.is_none() ? 0 : seed.cast<uint64_t>();
             return p;
           }),
           py::arg("temperature") = 0.8f, py::arg("top_p") = 0.95f, py::arg("top_k") = 40,
           py::arg("max_tokens") = 128, py::arg("seed") = py::none())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("has_seed", &SamplingParams::has_seed)
      .def_readwrite("seed", &SamplingParams::seed)
      .def("problem", &SamplingParams::problem);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_concurrent", &SchedulerConfig::max_concurrent)
      .def_readwrite("queue_capacity", &SchedulerConfig::queue_capacity)
      .def_readwrite("max_batch_tokens", &SchedulerConfig::max_batch_tokens)
      .def_readwrite("prefill_chunk", &SchedulerConfig::prefill_chunk)
      .def_readwrite("max_context", &SchedulerConfig::max_context)
      .def_readwrite("eos_token_ids", &SchedulerConfig::eos_token_ids)
      // one id, or -1 for none: the list with that one entry
      .def_property("eos_token_id",
                    [](const SchedulerConfig& c) { return c.eos_token_ids.empty() ? -1 : c.eos_token_ids[0]; },
                    [](SchedulerConfig& c, int32_t id) {
                      c.eos_token_ids.clear();
                      if (id >= 0) c.eos_token_ids.push_back(id);
                    })
      .def_readwrite("vocab_size", &SchedulerConfig::vocab_size)
      .def_readwrite("ignore_eos", &SchedulerConfig::ignore_eos)
      .def_readwrite("paced_prefill", &SchedulerConfig::paced_prefill);

  py::class_<Pacing>(m, "Pacing")
      .def_readonly("decode_step", &Pacing::decode_step)
      .def_readonly("prefill_token", &Pacing::prefill_token)
      .def_property_readonly("chunk", &Pacing::chunk);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("id", &PlanEntry::id)
      .def_readonly("slot", &PlanEntry::slot)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("tokens", &PlanEntry::tokens)
      .def_readonly("decode", &PlanEntry::decode)
      .def_readonly("sample", &PlanEntry::sample)
      .def_readonly("temperature", &PlanEntry::temperature)
      .def_readonly("top_p", &PlanEntry::top_p)
      .def_readonly("top_k", &PlanEntry::top_k)
      .def_readonly("u", &PlanEntry::u);

  py::enum_<EventKind>(m, "EventKind")
      .value("Token", EventKind::Token)
      .value("Done", EventKind::Done)
      .value("Error", EventKind::Error);

  py::class_<Event>(m, "Event")
      .def_readonly("id", &Event::id)
      .def_readonly("kind", &Event::kind)
      .def_readonly("token", &Event::token)
      .def_readonly("detail", &Event::detail);

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("entries", &StepPlan::entries)
      .def_readonly("preempted", &StepPlan::preempted)
      .def_readonly("events", &StepPlan::events)
      .def_property_readonly("num_tokens", &StepPlan::num_tokens);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("submitted", &SchedulerStats::submitted)
      .def_readonly("completed", &SchedulerStats::completed)
      .def_readonly("cancelled", &SchedulerStats::cancelled)
      .def_readonly("timed_out", &SchedulerStats::timed_out)
      .def_readonly("failed", &SchedulerStats::failed)
      .def_readonly("rejected_busy", &SchedulerStats::rejected_busy)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("tokens_fed", &SchedulerStats::tokens_fed)
      .def_readonly("tokens_generated", &SchedulerStats::tokens_generated)
      .def_readonly("running", &SchedulerStats::running)
      .def_readonly("queued", &SchedulerStats::queued);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<SchedulerConfig, CacheManager*>(), py::arg("config"), py::arg("cache"),
           py::keep_alive<1, 3>())
      .def("submit", &Scheduler::submit, py::arg("prompt"), py::arg("params"), py::arg("priority") = 0,
           py::arg("timeout") = 0.0)
      .def("now", &Scheduler::now)
      .def("set_time", &Scheduler::set_time)
      .def("cancel", &Scheduler::cancel)
      .def("plan", &Scheduler::plan)
      .def("peek_uniform", &Scheduler::peek_uniform)
      .def("complete", &Scheduler::complete, py::arg("plan"), py::arg("sampled"), py::arg("elapsed") = -1.0)
      .def_property_readonly("pacing", [](const Scheduler& s) { return s.pacing(); })
      .def("fail", &Scheduler::fail)
      .def("idle", &Scheduler::idle)
      .def("stats", &Scheduler::stats);
}
