// The control plane: page pool, cache manager, request lifecycle and scheduler.
// Plain C++17, no CUDA and no torch: it decides which tokens of which request run
// in a step and which cache pages they use; the step function executes the plan.
//
// The reference keeps this layer in Rust (crates/einf-control/src/*.rs, bound by
// crates/einf-control-py/src/lib.rs); this is a fresh C++ design of the same
// roles, bound with pybind11 (bindings.cpp).
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace einf {

using RequestId = std::string;

// Errors a caller can cause (bad arguments, unknown ids): Python ValueError.
struct InvalidArgument : std::invalid_argument {
  using std::invalid_argument::invalid_argument;
};
// Errors of state (a stale batch, a request in flight, a page freed twice): Python RuntimeError.
struct StateError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------------------------
// Page pool: ids 0..n-1, each free or held.  Allocation is all-or-nothing and
// takes the most recently freed pages first, lowest ids first on a fresh pool.
// (reference role: crates/einf-control/src/block_pool.rs:90-247)
// ---------------------------------------------------------------------------
class PagePool {
 public:
  explicit PagePool(int num_pages);
  int capacity() const { return static_cast<int>(held_.size()); }
  int free_count() const { return static_cast<int>(free_.size()); }
  int held_count() const { return capacity() - free_count(); }
  int high_water() const { return high_water_; }
  bool is_held(int page) const;
  // Returns false and changes nothing if fewer than n pages are free.
  bool allocate(int n, std::vector<int>* out);
  // Throws StateError for a page that is out of range or already free; in that
  // case no page of the call is released.
  void release(const std::vector<int>& pages);

 private:
  std::vector<int> free_;       // stack, next page at the back
  std::vector<uint8_t> held_;
  int high_water_ = 0;
};

// Fixed-size per-request state: slot ids 0..n-1.
class SlotPool {
 public:
  explicit SlotPool(int num_slots);
  int capacity() const { return static_cast<int>(held_.size()); }
  int free_count() const { return static_cast<int>(free_.size()); }
  int take();            // -1 if none is free
  void give_back(int slot);

 private:
  std::vector<int> free_;
  std::vector<uint8_t> held_;
};

// One group of layers with the same cache needs: pages of its own.
struct GroupSpec {
  int num_pages = 0;
  int page_size = 0;
  int window = 0;  // 0: every key is kept; n > 0: only the last n keys are needed
};

// ---------------------------------------------------------------------------
// Cache manager: per request, one block table per group (logical page -> physical
// page, -1 where a window has passed) and at most one state slot.
// (reference role: crates/einf-control/src/kv_cache.rs:48-250; groups, windows and
// state slots have no counterpart there.)
// ---------------------------------------------------------------------------
class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, int num_state_slots);

  int num_groups() const { return static_cast<int>(groups_.size()); }
  const GroupSpec& group(int g) const { return groups_.at(g); }
  int free_pages(int g) const { return pools_.at(g).free_count(); }
  int held_pages(int g) const { return pools_.at(g).held_count(); }
  int high_water(int g) const { return pools_.at(g).high_water(); }
  int free_state_slots() const { return slots_.free_count(); }
  int num_state_slots() const { return slots_.capacity(); }
  bool holds(const RequestId& id) const { return entries_.count(id) != 0; }
  std::vector<RequestId> holders() const;

  // Pages a request would still have to take, per group, to run tokens
  // [start, end) on top of what it already holds.
  std::vector<int> pages_needed(const RequestId& id, int start, int end) const;

  // Whether the free pages of every group could hold a request of `context_len` tokens that
  // is fed in portions of at most `portion` tokens (a windowed group holds at most the window
  // plus one portion).  The scheduler admits a waiting request only then, so that a request
  // that was preempted is not admitted again just to run out of pages once more.
  bool room_for(int context_len, int portion) const;

  // Make room for tokens [start, end) of the request in every group (and a state
  // slot on its first reservation).  All-or-nothing across groups: on false
  // nothing has changed.  `short_group`, if given, names the first group that was short
  // (-1: the state slots).
  bool reserve(const RequestId& id, int start, int end, int* short_group = nullptr);

  // The request now has `cached_len` tokens behind it: give back the pages a
  // window has passed.  Returns how many pages were freed.
  int advance(const RequestId& id, int cached_len);

  // Give back everything the request holds.  Unknown ids are ignored.
  void release(const RequestId& id);

  const std::vector<int>& block_table(const RequestId& id, int g) const;
  int state_slot(const RequestId& id) const;  // -1 if none
  // Tokens a request could hold if it had the whole pool of its tightest group.
  long long capacity_tokens() const;

  // Throws StateError if a page is lost, held twice, or held by nobody.
  void check_invariants() const;

 private:
  struct Entry {
    std::vector<std::vector<int>> tables;  // [group][logical page]
    int state_slot = -1;
  };
  int first_needed_page(const GroupSpec& spec, int start) const;

  std::vector<GroupSpec> groups_;
  std::vector<PagePool> pools_;
  SlotPool slots_;
  std::map<RequestId, Entry> entries_;
};

// ---------------------------------------------------------------------------
// Sampling parameters (reference: crates/einf-control/src/sample.rs:22-108).
// ---------------------------------------------------------------------------
struct SamplingParams {
  float temperature = 0.f;   // 0: greedy
  int top_k = 0;             // 0: off
  float top_p = 1.f;
  float min_p = 0.f;
  uint64_t seed = 0;
  std::vector<int64_t> stop_token_ids;
  int num_logprobs = 0;

  void validate() const;  // throws InvalidArgument
  bool greedy() const { return temperature == 0.f; }
};

struct RequestSpec {
  RequestId id;
  std::vector<int> prompt_token_ids;
  int max_new_len = 0;
  SamplingParams sampling;
};

enum class RequestState { Waiting, Running, Finished, Cancelled, Failed };
enum class CompletionReason { None, Eos, Length };

// (reference: crates/einf-control/src/request.rs:69-343)
struct Request {
  RequestSpec spec;
  RequestState state = RequestState::Waiting;
  CompletionReason reason = CompletionReason::None;
  uint64_t arrival_index = 0;
  int cached_len = 0;                // tokens whose keys and values are in the cache
  std::vector<int> generated;        // kept across preemption
  std::string error;
  int preemptions = 0;

  int context_len() const { return static_cast<int>(spec.prompt_token_ids.size() + generated.size()); }
  int token_at(int position) const;
  int pending() const { return context_len() - cached_len; }
  // A decode step feeds the one token that was sampled last.
  bool is_decode() const { return !generated.empty() && pending() == 1; }
  bool live() const { return state == RequestState::Waiting || state == RequestState::Running; }
};

// One request's share of a step (reference: crates/einf-control/src/execution_plan.rs:12-29).
struct ScheduledRequest {
  RequestId id;
  std::vector<int> input_token_ids;
  bool is_decode = false;
  int start_position = 0;
  std::vector<std::vector<int>> block_tables;  // per cache group
  int state_slot = -1;
  bool need_sample = false;
  int64_t sample_index = 0;   // tokens the request has generated so far
  SamplingParams sampling;
};

struct BatchPlan {
  uint64_t step_id = 0;
  std::vector<ScheduledRequest> requests;
  // Decode steps the executor may run on this plan before it reports back (1 unless the
  // scheduler was built with a lookahead).  More than 1 only when every request of the plan
  // decodes; pages for that many tokens are reserved and are in the block tables; from the
  // second step on, a request's input is the token it sampled in the step before.
  int decode_steps = 1;
  int num_tokens() const;
};

struct RequestResult {
  RequestId id;
  // empty, or the sampled token; with decode_steps > 1 the tokens of the steps that count for this
  // request, in order: all of them, or up to and including the one that ended it
  std::vector<int> generated_token_ids;
  int cached_len_delta = 0;              // input tokens whose keys and values are now cached
  bool is_eos = false;                   // the last of generated_token_ids ended the request
};

struct ExecutionResult {
  uint64_t step_id = 0;
  std::vector<RequestResult> results;
};

// ---------------------------------------------------------------------------
// Packing a batch plan into the int32 step buffer the kernels read.  The layout
// depends only on the counts, so that a CUDA graph captured for a bucket of decode
// steps finds every field where each later step's copy puts it.
// (reference role: ModelInputPool.build, src/einf/executors/torch/input.py:109-319)
// ---------------------------------------------------------------------------
struct PackConfig {
  int page_size = 0;
  std::vector<int> pages_per_group;
  std::vector<int> windows;       // 0: all keys
  int vocab_size = 0;
  int table_width = 0;
  int max_tokens = 0;
  int max_requests = 0;
  int q_tile = 128;               // query rows per tile of the prefill attention kernels
};

struct StepField {
  std::string name;
  int offset = 0;   // in int32 elements
  int count = 0;
};

// Fields in buffer order; every field starts on a 16-byte boundary.
std::vector<StepField> step_layout(int tokens, int requests, int wanted, int groups, int table_width, int tiles,
                                   int single_tokens, int* total);

struct PackedStep {
  std::vector<StepField> fields;
  int total = 0;
  int num_tokens = 0, num_requests = 0, num_wanted = 0;
  int num_tiles = 0;            // 128-row query tiles of the requests that bring more than one token
  int num_single_tokens = 0;    // requests that bring one token (decoding): their packed token indices
  int max_q_len = 0, max_context_len = 0;
  int max_portion_start = 0;    // most tokens that a request with more than one token here already holds
  bool decode_only = false;
  std::vector<int> q_lens, starts;
  std::vector<std::pair<int, int>> rows_of_request;   // per real request: first logits row, count
};

// `want`: per request the places among its tokens whose logits are wanted; null: the last
// token of every request that samples.  `pad_requests_to` appends one-token requests that
// write nothing (page 0 of every group, slot -1) up to that many requests.
// Throws InvalidArgument for a plan the step function must refuse.
PackedStep pack_step(const std::vector<ScheduledRequest>& requests, const std::vector<std::vector<int>>* want,
                     int32_t* buffer, size_t capacity, const PackConfig& config, int pad_requests_to);

enum class Policy { Fcfs, DecodeFirst };
Policy policy_from_string(const std::string& name);  // "fcfs" | "decode_first"

struct SchedulerStats {
  uint64_t steps = 0;
  uint64_t prefill_tokens = 0;
  uint64_t decode_tokens = 0;
  uint64_t preemptions = 0;
  uint64_t failures = 0;
  uint64_t finished = 0;
  uint64_t window_pages_freed = 0;
};

// ---------------------------------------------------------------------------
// Scheduler (reference: crates/einf-control/src/scheduler.rs:33-667).
//
// schedule():  running requests first, in policy order, each gets its next
//   portion under the token budget; then waiting requests are admitted from the
//   head of the queue while budget and pages last.
// When a running request cannot get its pages, the last request in policy order
//   that has not been scheduled in this step is preempted (pages given back,
//   generated tokens kept, front of the waiting queue) and the reservation is
//   tried again.  If that last request is the one asking, it preempts itself
//   when other requests hold pages (they will finish and free them), and fails
//   with "Insufficient memory to fulfill request <id>" when it is alone: then
//   the pool can never hold it.  (The reference fails it in both cases,
//   scheduler.rs:286-294.)  A waiting request that does not fit into an
//   otherwise idle engine fails the same way; otherwise admission just stops.
// ---------------------------------------------------------------------------
class Scheduler {
 public:
  // decode_lookahead: decode steps a plan may cover when every request of it decodes and none waits
  // for admission (1: every step reports back, as the reference does).
  // max_requests: most requests that run at a time, and so the most a plan holds (0: no limit
  // but the token budget and the pages).  The step buffer, the sampler and the block-table rows
  // of an engine are made for that many, so its scheduler must never plan more.
  Scheduler(Policy policy, std::vector<GroupSpec> groups, int num_state_slots, int max_batch_len,
            int max_prefill_chunk_len, int decode_lookahead = 1, int max_requests = 0);

  void submit(RequestSpec spec);
  void cancel(const RequestId& id);
  std::optional<BatchPlan> schedule();
  void apply_result(const ExecutionResult& result);
  // The outcome of the next decode step of an outstanding plan that covers several
  // (decode_steps > 1), for an executor that reports every step while later steps already run:
  // one sampled token for every request of the plan that has not ended on an earlier step of it,
  // an empty entry for one that has.  The plan stays outstanding until its last step has been
  // applied or every request of it has ended; what the device computes for a request after its
  // end-of-sequence token is never reported.  A plan is applied either step by step or whole.
  void apply_step(const ExecutionResult& result);
  void fail_batch(uint64_t step_id, const std::string& message);

  const Request& request(const RequestId& id) const;
  bool has_request(const RequestId& id) const { return requests_.count(id) != 0; }
  void forget(const RequestId& id);  // drop the record of a request that is no longer live
  std::vector<RequestId> waiting_ids() const;
  std::vector<RequestId> running_ids() const;
  bool has_outstanding() const { return outstanding_.has_value(); }
  // decode steps of the outstanding plan that apply_step has not seen yet (0: none outstanding)
  int outstanding_steps_left() const {
    return outstanding_ ? outstanding_->decode_steps - outstanding_steps_applied_ : 0;
  }
  bool idle() const;
  const CacheManager& cache() const { return cache_; }
  const SchedulerStats& stats() const { return stats_; }
  int max_batch_len() const { return max_batch_len_; }
  int max_prefill_chunk_len() const { return max_prefill_chunk_len_; }
  int decode_lookahead() const { return decode_lookahead_; }
  int max_requests() const { return max_requests_; }

 private:
  std::vector<RequestId> ordered_running() const;
  // How many decode steps the selected requests can run before they report back.
  int plan_lookahead(std::vector<ScheduledRequest>* selected);
  // 0: nothing to do or no budget; >0: tokens scheduled; -1: pages are short.
  int schedule_one(Request& request, int remaining, std::vector<ScheduledRequest>* selected);
  void preempt(Request& request);
  void fail(Request& request, const std::string& message);
  void finish(Request& request, CompletionReason reason);

  Policy policy_;
  CacheManager cache_;
  int max_batch_len_;
  int max_prefill_chunk_len_;
  int decode_lookahead_;
  int max_requests_;
  std::map<RequestId, Request> requests_;
  std::deque<RequestId> waiting_;
  std::vector<RequestId> running_;
  uint64_t next_arrival_ = 0;
  uint64_t next_step_ = 0;
  std::optional<BatchPlan> outstanding_;
  int outstanding_steps_applied_ = 0;          // steps of the outstanding plan applied by apply_step
  std::set<RequestId> outstanding_ended_;      // its requests that ended on one of those steps
  SchedulerStats stats_;
};

}  // namespace einf
