// pybind11 module `_control`: the control plane's classes for Python.
// InvalidArgument maps to ValueError, StateError to RuntimeError
// (the reference maps its errors the same way, crates/einf-control-py/src/lib.rs:5-14).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "control.h"

namespace py = pybind11;
using namespace einf;

namespace {

const char* state_name(RequestState s) {
  switch (s) {
    case RequestState::Waiting: return "waiting";
    case RequestState::Running: return "running";
    case RequestState::Finished: return "finished";
    case RequestState::Cancelled: return "cancelled";
    case RequestState::Failed: return "failed";
  }
  return "?";
}

const char* reason_name(CompletionReason r) {
  switch (r) {
    case CompletionReason::None: return "";
    case CompletionReason::Eos: return "eos";
    case CompletionReason::Length: return "length";
  }
  return "?";
}

}  // namespace

PYBIND11_MODULE(_control, m) {
  m.doc() = "einf_b200 control plane: page pool, cache manager, scheduler";

  py::register_exception<InvalidArgument>(m, "InvalidArgument", PyExc_ValueError);
  py::register_exception<StateError>(m, "StateError", PyExc_RuntimeError);

  py::class_<PagePool>(m, "PagePool")
      .def(py::init<int>(), py::arg("num_pages"))
      .def_property_readonly("capacity", &PagePool::capacity)
      .def_property_readonly("free_count", &PagePool::free_count)
      .def_property_readonly("held_count", &PagePool::held_count)
      .def_property_readonly("high_water", &PagePool::high_water)
      .def("is_held", &PagePool::is_held)
      .def("allocate",
           [](PagePool& pool, int n) -> py::object {
             std::vector<int> pages;
             if (!pool.allocate(n, &pages)) return py::none();
             return py::cast(pages);
           },
           py::arg("n"), "n pages, or None (and no change) if fewer are free")
      .def("release", &PagePool::release);

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int num_pages, int page_size, int window) {
             GroupSpec spec;
             spec.num_pages = num_pages;
             spec.page_size = page_size;
             spec.window = window;
             return spec;
           }),
           py::arg("num_pages"), py::arg("page_size"), py::arg("window") = 0)
      .def_readonly("num_pages", &GroupSpec::num_pages)
      .def_readonly("page_size", &GroupSpec::page_size)
      .def_readonly("window", &GroupSpec::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupSpec>, int>(), py::arg("groups"), py::arg("num_state_slots") = 0)
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def("free_pages", &CacheManager::free_pages, py::arg("group") = 0)
      .def("held_pages", &CacheManager::held_pages, py::arg("group") = 0)
      .def("high_water", &CacheManager::high_water, py::arg("group") = 0)
      .def_property_readonly("free_state_slots", &CacheManager::free_state_slots)
      .def_property_readonly("num_state_slots", &CacheManager::num_state_slots)
      .def("holds", &CacheManager::holds)
      .def("holders", &CacheManager::holders)
      .def("pages_needed", &CacheManager::pages_needed)
      .def("room_for", &CacheManager::room_for, py::arg("context_len"), py::arg("portion"))
      .def("reserve", [](CacheManager& c, const RequestId& id, int start, int end) { return c.reserve(id, start, end); },
           py::arg("id"), py::arg("start"), py::arg("end"))
      .def("advance", &CacheManager::advance)
      .def("release", &CacheManager::release)
      .def("block_table", &CacheManager::block_table, py::arg("id"), py::arg("group") = 0)
      .def("state_slot", &CacheManager::state_slot)
      .def("capacity_tokens", &CacheManager::capacity_tokens)
      .def("check_invariants", &CacheManager::check_invariants);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](float temperature, py::object top_k, float top_p, float min_p, uint64_t seed,
                       std::vector<int64_t> stop_token_ids, int num_logprobs) {
             SamplingParams p;
             p.temperature = temperature;
             if (!top_k.is_none()) {
               const int k = top_k.cast<int>();
               if (k <= 0) throw InvalidArgument("top_k must be positive when specified");
               p.top_k = k;
             }
             p.top_p = top_p;
             p.min_p = min_p;
             p.seed = seed;
             p.stop_token_ids = std::move(stop_token_ids);
             p.num_logprobs = num_logprobs;
             p.validate();
             return p;
           }),
           py::arg("temperature") = 0.f, py::arg("top_k") = py::none(), py::arg("top_p") = 1.f,
           py::arg("min_p") = 0.f, py::arg("seed") = 0, py::arg("stop_token_ids") = std::vector<int64_t>{},
           py::arg("num_logprobs") = 0)
      .def_readonly("temperature", &SamplingParams::temperature)
      .def_property_readonly("top_k", [](const SamplingParams& p) -> py::object {
        return p.top_k > 0 ? py::cast(p.top_k) : py::none();
      })
      .def_readonly("top_p", &SamplingParams::top_p)
      .def_readonly("min_p", &SamplingParams::min_p)
      .def_readonly("seed", &SamplingParams::seed)
      .def_readonly("stop_token_ids", &SamplingParams::stop_token_ids)
      .def_readonly("num_logprobs", &SamplingParams::num_logprobs)
      .def_property_readonly("is_greedy", &SamplingParams::greedy);

  py::class_<RequestSpec>(m, "RequestSpec")
      .def(py::init([](RequestId id, std::vector<int> prompt, int max_new_len, py::object sampling) {
             RequestSpec spec;
             spec.id = std::move(id);
             spec.prompt_token_ids = std::move(prompt);
             spec.max_new_len = max_new_len;
             if (!sampling.is_none()) spec.sampling = sampling.cast<SamplingParams>();
             return spec;
           }),
           py::arg("request_id"), py::arg("prompt_token_ids"), py::arg("max_new_len"),
           py::arg("sampling_params") = py::none())
      .def_readonly("request_id", &RequestSpec::id)
      .def_readonly("prompt_token_ids", &RequestSpec::prompt_token_ids)
      .def_readonly("max_new_len", &RequestSpec::max_new_len)
      .def_readonly("sampling_params", &RequestSpec::sampling);

  // A read-only view of a request (reference: RequestView, einf-control-py/src/lib.rs:537-617).
  py::class_<Request>(m, "RequestView")
      .def_property_readonly("request_id", [](const Request& r) { return r.spec.id; })
      .def_property_readonly("prompt_token_ids", [](const Request& r) { return r.spec.prompt_token_ids; })
      .def_property_readonly("max_new_len", [](const Request& r) { return r.spec.max_new_len; })
      .def_property_readonly("sampling_params", [](const Request& r) { return r.spec.sampling; })
      .def_property_readonly("state", [](const Request& r) { return std::string(state_name(r.state)); })
      .def_property_readonly("completion_reason", [](const Request& r) -> py::object {
        if (r.reason == CompletionReason::None) return py::none();
        return py::cast(std::string(reason_name(r.reason)));
      })
      .def_property_readonly("error", [](const Request& r) -> py::object {
        if (r.state != RequestState::Failed) return py::none();
        return py::cast(r.error);
      })
      .def_readonly("cached_len", &Request::cached_len)
      .def_readonly("generated_token_ids", &Request::generated)
      .def_readonly("arrival_index", &Request::arrival_index)
      .def_readonly("preemptions", &Request::preemptions)
      .def_property_readonly("is_decode", &Request::is_decode);

  py::class_<ScheduledRequest>(m, "ScheduledRequest")
      .def(py::init([](RequestId id, std::vector<int> tokens, int start_position,
                       std::vector<std::vector<int>> block_tables, bool need_sample, bool is_decode,
                       int state_slot, int64_t sample_index, py::object sampling) {
             ScheduledRequest s;
             s.id = std::move(id);
             s.input_token_ids = std::move(tokens);
             s.start_position = start_position;
             s.block_tables = std::move(block_tables);
             s.need_sample = need_sample;
             s.is_decode = is_decode;
             s.state_slot = state_slot;
             s.sample_index = sample_index;
             if (!sampling.is_none()) s.sampling = sampling.cast<SamplingParams>();
             return s;
           }),
           py::arg("request_id"), py::arg("input_token_ids"), py::arg("start_position"),
           py::arg("block_tables"), py::arg("need_sample") = false, py::arg("is_decode") = false,
           py::arg("state_slot") = -1, py::arg("sample_index") = 0, py::arg("sampling_params") = py::none())
      .def_readonly("request_id", &ScheduledRequest::id)
      .def_readonly("input_token_ids", &ScheduledRequest::input_token_ids)
      .def_readonly("is_decode", &ScheduledRequest::is_decode)
      .def_readonly("start_position", &ScheduledRequest::start_position)
      .def_readonly("block_tables", &ScheduledRequest::block_tables)
      .def_readonly("state_slot", &ScheduledRequest::state_slot)
      .def_readonly("need_sample", &ScheduledRequest::need_sample)
      .def_readonly("sample_index", &ScheduledRequest::sample_index)
      .def_readonly("sampling_params", &ScheduledRequest::sampling);

  py::class_<BatchPlan>(m, "BatchPlan")
      .def(py::init([](uint64_t step_id, std::vector<ScheduledRequest> requests) {
             BatchPlan plan;
             plan.step_id = step_id;
             plan.requests = std::move(requests);
             return plan;
           }),
           py::arg("step_id"), py::arg("requests"))
      .def_readonly("step_id", &BatchPlan::step_id)
      .def_readonly("requests", &BatchPlan::requests)
      .def_readonly("decode_steps", &BatchPlan::decode_steps)
      .def_property_readonly("num_tokens", &BatchPlan::num_tokens)
      .def("__len__", [](const BatchPlan& plan) { return plan.requests.size(); })
      // What an executor needs of each request, without copying tokens and block tables:
      // (request_id, number of tokens, need_sample, sample_index, sampling_params, start_position, state_slot)
      .def("summary", [](const BatchPlan& plan) {
        py::list out;
        for (const ScheduledRequest& r : plan.requests)
          out.append(py::make_tuple(r.id, r.input_token_ids.size(), r.need_sample, r.sample_index, r.sampling,
                                    r.start_position, r.state_slot));
        return out;
      });

  py::class_<PackConfig>(m, "PackConfig")
      .def(py::init([](int page_size, std::vector<int> pages_per_group, std::vector<int> windows, int vocab_size,
                       int table_width, int max_tokens, int max_requests, int q_tile) {
             PackConfig c;
             c.page_size = page_size;
             c.pages_per_group = std::move(pages_per_group);
             c.windows = std::move(windows);
             c.vocab_size = vocab_size;
             c.table_width = table_width;
             c.max_tokens = max_tokens;
             c.max_requests = max_requests;
             c.q_tile = q_tile;
             if (c.pages_per_group.size() != c.windows.size()) throw InvalidArgument("one window per cache group");
             return c;
           }),
           py::arg("page_size"), py::arg("pages_per_group"), py::arg("windows"), py::arg("vocab_size"),
           py::arg("table_width"), py::arg("max_tokens"), py::arg("max_requests"), py::arg("q_tile") = 128);

  py::class_<PackedStep>(m, "PackedStep")
      .def_readonly("total", &PackedStep::total)
      .def_readonly("num_tokens", &PackedStep::num_tokens)
      .def_readonly("num_requests", &PackedStep::num_requests)
      .def_readonly("num_wanted", &PackedStep::num_wanted)
      .def_readonly("num_tiles", &PackedStep::num_tiles)
      .def_readonly("num_single_tokens", &PackedStep::num_single_tokens)
      .def_readonly("max_q_len", &PackedStep::max_q_len)
      .def_readonly("max_context_len", &PackedStep::max_context_len)
      .def_readonly("max_portion_start", &PackedStep::max_portion_start)
      .def_readonly("decode_only", &PackedStep::decode_only)
      .def_readonly("q_lens", &PackedStep::q_lens)
      .def_readonly("starts", &PackedStep::starts)
      .def_readonly("rows_of_request", &PackedStep::rows_of_request)
      .def_property_readonly("fields", [](const PackedStep& p) {
        py::dict d;
        for (const StepField& f : p.fields) d[py::str(f.name)] = py::make_tuple(f.offset, f.count);
        return d;
      });

  m.def("step_buffer_size",
        [](int tokens, int requests, int wanted, int groups, int table_width, int tiles, int single_tokens) {
          int total = 0;
          step_layout(tokens, requests, wanted, groups, table_width, tiles, single_tokens, &total);
          return total;
        });

  // Pack the requests of a plan (or a list of ScheduledRequest) into `buffer`, an int32 array.
  auto pack = [](const std::vector<ScheduledRequest>& requests, py::object want,
                 py::array_t<int32_t, py::array::c_style> buffer, const PackConfig& config, int pad_requests_to) {
    std::vector<std::vector<int>> want_values;
    const std::vector<std::vector<int>>* want_ptr = nullptr;
    if (!want.is_none()) {
      want_values = want.cast<std::vector<std::vector<int>>>();
      want_ptr = &want_values;
    }
    return pack_step(requests, want_ptr, buffer.mutable_data(), static_cast<size_t>(buffer.size()), config,
                     pad_requests_to);
  };
  m.def("pack_plan",
        [pack](const BatchPlan& plan, py::object want, py::array_t<int32_t, py::array::c_style> buffer,
               const PackConfig& config, int pad_requests_to) {
          return pack(plan.requests, want, buffer, config, pad_requests_to);
        },
        py::arg("plan"), py::arg("want"), py::arg("buffer"), py::arg("config"), py::arg("pad_requests_to") = 0);

  py::class_<RequestResult>(m, "RequestResult")
      .def(py::init([](RequestId id, std::vector<int> tokens, int delta, bool is_eos) {
             RequestResult r;
             r.id = std::move(id);
             r.generated_token_ids = std::move(tokens);
             r.cached_len_delta = delta;
             r.is_eos = is_eos;
             return r;
           }),
           py::arg("request_id"), py::arg("generated_token_ids"), py::arg("cached_len_delta"),
           py::arg("is_eos") = false)
      .def_readonly("request_id", &RequestResult::id)
      .def_readonly("generated_token_ids", &RequestResult::generated_token_ids)
      .def_readonly("cached_len_delta", &RequestResult::cached_len_delta)
      .def_readonly("is_eos", &RequestResult::is_eos);

  py::class_<ExecutionResult>(m, "ExecutionResult")
      .def(py::init([](uint64_t step_id, std::vector<RequestResult> results) {
             ExecutionResult r;
             r.step_id = step_id;
             r.results = std::move(results);
             return r;
           }),
           py::arg("step_id"), py::arg("request_results"))
      .def_readonly("step_id", &ExecutionResult::step_id)
      .def_readonly("request_results", &ExecutionResult::results);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("prefill_tokens", &SchedulerStats::prefill_tokens)
      .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("failures", &SchedulerStats::failures)
      .def_readonly("finished", &SchedulerStats::finished)
      .def_readonly("window_pages_freed", &SchedulerStats::window_pages_freed);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init([](const std::string& policy, std::vector<GroupSpec> groups, int max_batch_len,
                       int max_prefill_chunk_len, int num_state_slots, int decode_lookahead, int max_requests) {
             return new Scheduler(policy_from_string(policy), std::move(groups), num_state_slots,
                                  max_batch_len, max_prefill_chunk_len, decode_lookahead, max_requests);
           }),
           py::arg("policy"), py::arg("groups"), py::arg("max_batch_len"), py::arg("max_prefill_chunk_len"),
           py::arg("num_state_slots") = 0, py::arg("decode_lookahead") = 1, py::arg("max_requests") = 0)
      .def("submit", &Scheduler::submit)
      .def("cancel", &Scheduler::cancel)
      .def("schedule", &Scheduler::schedule)
      .def("apply_result", &Scheduler::apply_result)
      .def("apply_step", &Scheduler::apply_step)
      .def_property_readonly("outstanding_steps_left", &Scheduler::outstanding_steps_left)
      .def("fail_batch",
           [](Scheduler& s, const BatchPlan& plan, const std::string& message) { s.fail_batch(plan.step_id, message); })
      .def("request", &Scheduler::request, py::return_value_policy::copy)
      .def("has_request", &Scheduler::has_request)
      .def("forget", &Scheduler::forget)
      .def("waiting_ids", &Scheduler::waiting_ids)
      .def("running_ids", &Scheduler::running_ids)
      .def_property_readonly("has_outstanding", &Scheduler::has_outstanding)
      .def_property_readonly("idle", &Scheduler::idle)
      .def_property_readonly("stats", &Scheduler::stats, py::return_value_policy::copy)
      .def_property_readonly("max_batch_len", &Scheduler::max_batch_len)
      .def_property_readonly("max_prefill_chunk_len", &Scheduler::max_prefill_chunk_len)
      .def_property_readonly("decode_lookahead", &Scheduler::decode_lookahead)
      .def_property_readonly("max_requests", &Scheduler::max_requests)
      .def("free_pages", [](const Scheduler& s, int g) { return s.cache().free_pages(g); }, py::arg("group") = 0)
      .def("free_blocks", [](const Scheduler& s) { return s.cache().free_pages(0); })
      .def("held_pages", [](const Scheduler& s, int g) { return s.cache().held_pages(g); }, py::arg("group") = 0)
      .def("high_water", [](const Scheduler& s, int g) { return s.cache().high_water(g); }, py::arg("group") = 0)
      .def("block_table", [](const Scheduler& s, const RequestId& id, int g) { return s.cache().block_table(id, g); },
           py::arg("id"), py::arg("group") = 0)
      .def("state_slot", [](const Scheduler& s, const RequestId& id) { return s.cache().state_slot(id); })
      .def("check_invariants", [](const Scheduler& s) { s.cache().check_invariants(); });
}
