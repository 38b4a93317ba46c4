// Request lifecycle and the scheduler.
#include <algorithm>
#include <cmath>
#include <set>
#include <tuple>

#include "control.h"

namespace einf {

void SamplingParams::validate() const {
  // (reference: crates/einf-control/src/sample.rs:33-108)
  if (!std::isfinite(temperature) || temperature < 0.f)
    throw InvalidArgument("temperature must be finite and non-negative");
  if (top_k < 0) throw InvalidArgument("top_k must be positive when specified");
  if (!std::isfinite(top_p) || !(top_p > 0.f && top_p <= 1.f))
    throw InvalidArgument("top_p must be finite and in (0, 1]");
  if (!std::isfinite(min_p) || !(min_p >= 0.f && min_p <= 1.f))
    throw InvalidArgument("min_p must be finite and in [0, 1]");
  if (seed > static_cast<uint64_t>(INT64_MAX)) throw InvalidArgument("seed must fit in a signed 64-bit integer");
  if (num_logprobs < 0) throw InvalidArgument("num_logprobs must not be negative");
  if (temperature == 0.f && (top_k != 0 || top_p != 1.f || min_p != 0.f))
    throw InvalidArgument("greedy sampling (temperature 0) takes no top_k, top_p or min_p");
}

int Request::token_at(int position) const {
  const int prompt_len = static_cast<int>(spec.prompt_token_ids.size());
  return position < prompt_len ? spec.prompt_token_ids[position] : generated.at(position - prompt_len);
}

int BatchPlan::num_tokens() const {
  int total = 0;
  for (const ScheduledRequest& r : requests) total += static_cast<int>(r.input_token_ids.size());
  return total;
}

Policy policy_from_string(const std::string& name) {
  if (name == "fcfs") return Policy::Fcfs;
  if (name == "decode_first") return Policy::DecodeFirst;
  throw InvalidArgument("unknown policy '" + name + "'; known: fcfs, decode_first");
}

Scheduler::Scheduler(Policy policy, std::vector<GroupSpec> groups, int num_state_slots, int max_batch_len,
                     int max_prefill_chunk_len, int decode_lookahead, int max_requests)
    : policy_(policy),
      cache_(std::move(groups), num_state_slots),
      max_batch_len_(max_batch_len),
      max_prefill_chunk_len_(max_prefill_chunk_len),
      decode_lookahead_(decode_lookahead),
      max_requests_(max_requests) {
  if (max_requests < 0) throw InvalidArgument("max_requests must not be negative");
  if (max_batch_len <= 0) throw InvalidArgument("max_batch_len must be positive");
  if (max_prefill_chunk_len <= 0) throw InvalidArgument("max_prefill_chunk_len must be positive");
  if (decode_lookahead <= 0) throw InvalidArgument("decode_lookahead must be positive");
}

void Scheduler::submit(RequestSpec spec) {
  if (requests_.count(spec.id)) throw InvalidArgument("request '" + spec.id + "' already exists");
  if (spec.prompt_token_ids.empty()) throw InvalidArgument("a request needs at least one prompt token");
  if (spec.max_new_len <= 0) throw InvalidArgument("max_new_len must be positive");
  for (int token : spec.prompt_token_ids)
    if (token < 0) throw InvalidArgument("prompt token ids must not be negative");
  spec.sampling.validate();
  Request request;
  request.arrival_index = next_arrival_++;
  const RequestId id = spec.id;
  request.spec = std::move(spec);
  requests_.emplace(id, std::move(request));
  waiting_.push_back(id);
}

void Scheduler::cancel(const RequestId& id) {
  auto found = requests_.find(id);
  if (found == requests_.end()) throw InvalidArgument("unknown request '" + id + "'");
  Request& request = found->second;
  if (outstanding_) {
    for (const ScheduledRequest& scheduled : outstanding_->requests) {
      if (scheduled.id != id) continue;
      // A plan of one step is in the executor's hands: the caller cannot be here before its result
      // is (reference: scheduler.rs:100-102).  A plan of several decode steps is applied step by
      // step, and between two of them a request may be cancelled: it counts as ended in the
      // plan, and what the device still computes for it is dropped.
      if (outstanding_->decode_steps <= 1) throw StateError("request '" + id + "' is in flight");
      outstanding_ended_.insert(id);
    }
  }
  if (!request.live()) return;
  request.state = RequestState::Cancelled;
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  cache_.release(id);
}

std::vector<RequestId> Scheduler::ordered_running() const {
  std::vector<RequestId> ids = running_;
  auto key = [&](const RequestId& id) {
    const Request& r = requests_.at(id);
    const int cls = (policy_ == Policy::DecodeFirst && !r.is_decode()) ? 1 : 0;
    return std::make_tuple(cls, r.arrival_index, id);
  };
  std::sort(ids.begin(), ids.end(), [&](const RequestId& a, const RequestId& b) { return key(a) < key(b); });
  return ids;
}

int Scheduler::schedule_one(Request& request, int remaining, std::vector<ScheduledRequest>* selected) {
  const int pending = request.pending();
  const int portion = std::min({max_prefill_chunk_len_, pending, remaining});
  if (portion <= 0) return 0;
  const int start = request.cached_len;
  if (!cache_.reserve(request.spec.id, start, start + portion)) return -1;
  ScheduledRequest scheduled;
  scheduled.id = request.spec.id;
  scheduled.is_decode = request.is_decode();
  scheduled.start_position = start;
  scheduled.input_token_ids.reserve(portion);
  for (int i = 0; i < portion; ++i) scheduled.input_token_ids.push_back(request.token_at(start + i));
  for (int g = 0; g < cache_.num_groups(); ++g) scheduled.block_tables.push_back(cache_.block_table(request.spec.id, g));
  scheduled.state_slot = cache_.state_slot(request.spec.id);
  scheduled.need_sample = portion == pending;
  scheduled.sample_index = static_cast<int64_t>(request.generated.size());
  scheduled.sampling = request.spec.sampling;
  selected->push_back(std::move(scheduled));
  return portion;
}

void Scheduler::preempt(Request& request) {
  // (reference: crates/einf-control/src/request.rs:190-196, scheduler.rs:159-168)
  request.state = RequestState::Waiting;
  request.cached_len = 0;
  request.preemptions += 1;
  const RequestId& id = request.spec.id;
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  waiting_.push_front(id);
  cache_.release(id);
  stats_.preemptions += 1;
}

void Scheduler::fail(Request& request, const std::string& message) {
  request.state = RequestState::Failed;
  request.error = message;
  const RequestId& id = request.spec.id;
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  cache_.release(id);
  stats_.failures += 1;
}

void Scheduler::finish(Request& request, CompletionReason reason) {
  request.state = RequestState::Finished;
  request.reason = reason;
  const RequestId& id = request.spec.id;
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  cache_.release(id);
  stats_.finished += 1;
}

int Scheduler::plan_lookahead(std::vector<ScheduledRequest>* selected) {
  // Several decode steps in one plan spare the host a round trip per token.  Only when it costs
  // nobody anything: every request of the plan decodes (its next inputs are its own samples), no
  // request waits for admission (it would wait that many steps longer), no request runs that the
  // plan leaves out, none reaches its length limit on the way, and the pages are there: a step
  // that would have to preempt for them stays a single step.
  if (decode_lookahead_ <= 1 || !waiting_.empty() || selected->size() != running_.size()) return 1;
  int steps = decode_lookahead_;
  for (const ScheduledRequest& scheduled : *selected) {
    if (!scheduled.is_decode || !scheduled.need_sample || scheduled.input_token_ids.size() != 1) return 1;
    const Request& request = requests_.at(scheduled.id);
    steps = std::min(steps, request.spec.max_new_len - static_cast<int>(request.generated.size()));
  }
  if (steps <= 1) return 1;
  // All or nothing: the pages of every request's lookahead are counted before any is taken, so
  // that a step that cannot look ahead is the plain single step and holds no extra page.
  std::vector<int> wanted(cache_.num_groups(), 0);
  for (const ScheduledRequest& scheduled : *selected) {
    const std::vector<int> needed =
        cache_.pages_needed(scheduled.id, scheduled.start_position + 1, scheduled.start_position + steps);
    for (int g = 0; g < cache_.num_groups(); ++g) wanted[g] += needed[g];
  }
  for (int g = 0; g < cache_.num_groups(); ++g)
    if (wanted[g] > cache_.free_pages(g)) return 1;
  for (ScheduledRequest& scheduled : *selected) {
    if (!cache_.reserve(scheduled.id, scheduled.start_position + 1, scheduled.start_position + steps))
      throw StateError("lookahead pages were counted as free but could not be reserved");
  }
  for (ScheduledRequest& scheduled : *selected)
    for (int g = 0; g < cache_.num_groups(); ++g) scheduled.block_tables[g] = cache_.block_table(scheduled.id, g);
  return steps;
}

std::optional<BatchPlan> Scheduler::schedule() {
  if (outstanding_) throw StateError("a batch is outstanding: apply its result or fail it first");
  int remaining = max_batch_len_;
  std::vector<ScheduledRequest> selected;
  std::set<RequestId> protected_ids;

  // Pass 1: requests that already run, in policy order.
  for (const RequestId& id : ordered_running()) {
    if (remaining <= 0) break;
    auto found = requests_.find(id);
    if (found == requests_.end() || found->second.state != RequestState::Running) continue;  // preempted meanwhile
    Request& request = found->second;
    while (true) {
      const int used = schedule_one(request, remaining, &selected);
      if (used >= 0) {
        if (used > 0) {
          remaining -= used;
          protected_ids.insert(id);
        }
        break;
      }
      // Pages are short: the last unprotected request in policy order gives way.
      RequestId victim;
      bool have_victim = false;
      for (const RequestId& candidate : ordered_running()) {
        if (!protected_ids.count(candidate)) {
          victim = candidate;
          have_victim = true;
        }
      }
      if (!have_victim || victim == id) {
        const bool alone = running_.size() == 1;
        if (alone) {
          fail(request, "Insufficient memory to fulfill request " + id);
        } else {
          preempt(request);
        }
        break;
      }
      preempt(requests_.at(victim));
    }
  }

  // Pass 2: admit from the head of the waiting queue.
  while (remaining > 0 && !waiting_.empty()) {
    // Every running request takes a row of the step; the engine has max_requests of them.
    if (max_requests_ > 0 && static_cast<int>(running_.size()) >= max_requests_) break;
    const RequestId id = waiting_.front();
    auto found = requests_.find(id);
    if (found == requests_.end() || found->second.state != RequestState::Waiting) {
      waiting_.pop_front();
      continue;
    }
    Request& request = found->second;
    const bool room = cache_.room_for(request.context_len(), max_prefill_chunk_len_);
    const int used = room ? schedule_one(request, remaining, &selected) : -1;
    if (used > 0) {
      waiting_.pop_front();
      request.state = RequestState::Running;
      running_.push_back(id);
      remaining -= used;
      continue;
    }
    if (used < 0 && running_.empty() && selected.empty()) {
      // Nothing else holds pages, and still it does not fit: it never will.
      fail(request, "Insufficient memory to fulfill request " + id);
      continue;
    }
    break;
  }

  if (selected.empty()) return std::nullopt;
  BatchPlan plan;
  plan.step_id = next_step_++;
  plan.decode_steps = plan_lookahead(&selected);
  plan.requests = std::move(selected);
  outstanding_ = plan;
  return plan;
}

void Scheduler::apply_result(const ExecutionResult& result) {
  // Validate everything first, change state afterwards
  // (reference: crates/einf-control/src/scheduler.rs:416-535).
  if (!outstanding_) throw StateError("no batch is outstanding");
  const BatchPlan& plan = *outstanding_;
  if (result.step_id != plan.step_id)
    throw StateError("stale result: step " + std::to_string(result.step_id) + ", outstanding step " +
                     std::to_string(plan.step_id));
  if (outstanding_steps_applied_ > 0)
    throw StateError("the outstanding plan is being applied step by step: go on with apply_step");
  if (result.results.size() != plan.requests.size())
    throw InvalidArgument("the result has " + std::to_string(result.results.size()) + " entries, the batch " +
                          std::to_string(plan.requests.size()));
  std::set<RequestId> seen;
  for (size_t i = 0; i < plan.requests.size(); ++i) {
    const ScheduledRequest& scheduled = plan.requests[i];
    const RequestResult& r = result.results[i];
    if (r.id != scheduled.id) throw InvalidArgument("result " + std::to_string(i) + " is for '" + r.id + "', expected '" + scheduled.id + "'");
    if (!seen.insert(r.id).second) throw InvalidArgument("request '" + r.id + "' appears twice in the result");
    auto found = requests_.find(r.id);
    if (found == requests_.end()) throw InvalidArgument("unknown request '" + r.id + "'");
    if (found->second.state != RequestState::Running) throw StateError("request '" + r.id + "' is not running");
    const int sampled = static_cast<int>(r.generated_token_ids.size());
    if (plan.decode_steps > 1) {
      // every step that counts for the request took one input token and sampled one
      if (sampled < 1 || sampled > plan.decode_steps)
        throw InvalidArgument("request '" + r.id + "' must have 1 to " + std::to_string(plan.decode_steps) + " sampled tokens");
      if (r.cached_len_delta != sampled)
        throw InvalidArgument("cached_len_delta of '" + r.id + "' differs from the steps it ran");
      if (sampled < plan.decode_steps && !r.is_eos)
        throw InvalidArgument("request '" + r.id + "' stopped early without an end-of-sequence token");
    } else {
      if (r.cached_len_delta != static_cast<int>(scheduled.input_token_ids.size()))
        throw InvalidArgument("cached_len_delta of '" + r.id + "' differs from the tokens it was given");
      if (sampled > 1) throw InvalidArgument("a step generates at most one token per request");
      if (scheduled.need_sample != (sampled == 1))
        throw InvalidArgument("request '" + r.id + "' " + (scheduled.need_sample ? "needs" : "must not have") + " a sampled token");
    }
    if (static_cast<int64_t>(found->second.generated.size()) != scheduled.sample_index)
      throw StateError("sample index of '" + r.id + "' changed while the batch was out");
    if (static_cast<int>(found->second.generated.size()) + sampled > found->second.spec.max_new_len)
      throw InvalidArgument("request '" + r.id + "' would exceed max_new_len");
    if (r.is_eos && r.generated_token_ids.empty()) throw InvalidArgument("is_eos without a token");
  }
  for (size_t i = 0; i < plan.requests.size(); ++i) {
    const ScheduledRequest& scheduled = plan.requests[i];
    const RequestResult& r = result.results[i];
    Request& request = requests_.at(r.id);
    request.cached_len += r.cached_len_delta;
    if (scheduled.is_decode) stats_.decode_tokens += r.cached_len_delta;
    else stats_.prefill_tokens += r.cached_len_delta;
    request.generated.insert(request.generated.end(), r.generated_token_ids.begin(), r.generated_token_ids.end());
    // Eos wins over Length (reference: scheduler.rs:547-555).
    if (r.is_eos) {
      finish(request, CompletionReason::Eos);
    } else if (static_cast<int>(request.generated.size()) >= request.spec.max_new_len) {
      finish(request, CompletionReason::Length);
    } else {
      stats_.window_pages_freed += cache_.advance(r.id, request.cached_len);
    }
  }
  stats_.steps += plan.decode_steps;
  outstanding_.reset();
}

void Scheduler::apply_step(const ExecutionResult& result) {
  if (!outstanding_) throw StateError("no batch is outstanding");
  const BatchPlan& plan = *outstanding_;
  if (result.step_id != plan.step_id)
    throw StateError("stale result: step " + std::to_string(result.step_id) + ", outstanding step " +
                     std::to_string(plan.step_id));
  if (plan.decode_steps <= 1) throw StateError("the outstanding plan covers one step: use apply_result");
  if (result.results.size() != plan.requests.size())
    throw InvalidArgument("the result has " + std::to_string(result.results.size()) + " entries, the batch " +
                          std::to_string(plan.requests.size()));
  // Validate everything first, change state afterwards.
  for (size_t i = 0; i < plan.requests.size(); ++i) {
    const ScheduledRequest& scheduled = plan.requests[i];
    const RequestResult& r = result.results[i];
    if (r.id != scheduled.id) throw InvalidArgument("result " + std::to_string(i) + " is for '" + r.id + "', expected '" + scheduled.id + "'");
    const int sampled = static_cast<int>(r.generated_token_ids.size());
    if (outstanding_ended_.count(r.id)) {
      // ended by its own end-of-sequence token (the executor then reports nothing more for it) or
      // cancelled in between (the executor does not know: what it reports is dropped)
      auto ended = requests_.find(r.id);
      const bool cancelled = ended == requests_.end() || ended->second.state == RequestState::Cancelled;
      if (!cancelled && (sampled != 0 || r.cached_len_delta != 0 || r.is_eos))
        throw InvalidArgument("request '" + r.id + "' ended on an earlier step of this plan and takes no more tokens");
      continue;
    }
    auto found = requests_.find(r.id);
    if (found == requests_.end()) throw InvalidArgument("unknown request '" + r.id + "'");
    if (found->second.state != RequestState::Running) throw StateError("request '" + r.id + "' is not running");
    if (sampled != 1 || r.cached_len_delta != 1)
      throw InvalidArgument("a decode step of '" + r.id + "' takes one token in and gives one out");
    if (static_cast<int64_t>(found->second.generated.size()) != scheduled.sample_index + outstanding_steps_applied_)
      throw StateError("sample index of '" + r.id + "' changed while the batch was out");
    if (static_cast<int>(found->second.generated.size()) + 1 > found->second.spec.max_new_len)
      throw InvalidArgument("request '" + r.id + "' would exceed max_new_len");
  }
  size_t live = 0;
  for (size_t i = 0; i < plan.requests.size(); ++i) {
    const RequestResult& r = result.results[i];
    if (outstanding_ended_.count(r.id)) continue;
    Request& request = requests_.at(r.id);
    request.cached_len += 1;
    stats_.decode_tokens += 1;
    request.generated.push_back(r.generated_token_ids[0]);
    if (r.is_eos) {
      finish(request, CompletionReason::Eos);
      outstanding_ended_.insert(r.id);
    } else if (static_cast<int>(request.generated.size()) >= request.spec.max_new_len) {
      finish(request, CompletionReason::Length);
      outstanding_ended_.insert(r.id);
    } else {
      stats_.window_pages_freed += cache_.advance(r.id, request.cached_len);
      ++live;
    }
  }
  stats_.steps += 1;
  outstanding_steps_applied_ += 1;
  if (outstanding_steps_applied_ >= plan.decode_steps || live == 0) {
    outstanding_.reset();
    outstanding_steps_applied_ = 0;
    outstanding_ended_.clear();
  }
}

void Scheduler::fail_batch(uint64_t step_id, const std::string& message) {
  // (reference: crates/einf-control/src/scheduler.rs:623-667)
  if (!outstanding_ || outstanding_->step_id != step_id) throw StateError("stale batch: it is not the outstanding one");
  const BatchPlan plan = *outstanding_;
  outstanding_.reset();
  outstanding_steps_applied_ = 0;
  outstanding_ended_.clear();
  for (const ScheduledRequest& scheduled : plan.requests) {
    auto found = requests_.find(scheduled.id);
    if (found != requests_.end() && found->second.live()) fail(found->second, message);
  }
}

const Request& Scheduler::request(const RequestId& id) const {
  auto found = requests_.find(id);
  if (found == requests_.end()) throw InvalidArgument("unknown request '" + id + "'");
  return found->second;
}

void Scheduler::forget(const RequestId& id) {
  auto found = requests_.find(id);
  if (found == requests_.end()) return;
  if (found->second.live()) throw StateError("request '" + id + "' is still live");
  requests_.erase(found);
}

std::vector<RequestId> Scheduler::waiting_ids() const { return {waiting_.begin(), waiting_.end()}; }
std::vector<RequestId> Scheduler::running_ids() const { return running_; }

bool Scheduler::idle() const { return waiting_.empty() && running_.empty() && !outstanding_; }

}  // namespace einf
