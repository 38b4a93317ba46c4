"""The scheduler's decisions, with an executor that answers last token + 1 (no GPU).

Scenarios restate the reference's own tables (crates/einf-control/tests/tests.rs:192-584,
tests/test_server.py:78-763) for this scheduler; where this scheduler decides
otherwise (a request that runs out of pages while others hold some waits instead
of failing) the test says so.
"""
import pytest

from einf_b200.cache import GroupSpec
from einf_b200.engine import (
    ExecutionResult, FakeExecutor, LLMServer, RequestResult, RequestSpec, Scheduler,
)
from einf_b200.sampling import SamplingParams


def make(policy="fcfs", pages=16, page=4, budget=8, chunk=8, window=0, slots=0):
    return Scheduler(policy, [GroupSpec(pages, page, window)], budget, chunk, slots)


def shape(plan):
    return [(r.request_id, list(r.input_token_ids), r.start_position, r.need_sample) for r in plan.requests]


def test_prefill_then_decode_then_length():
    scheduler = make()
    scheduler.submit(RequestSpec("a", [10, 11, 12], 2))
    executor = FakeExecutor()
    plan = scheduler.schedule()
    assert shape(plan) == [("a", [10, 11, 12], 0, True)]
    assert plan.requests[0].block_tables == [[0]] and not plan.requests[0].is_decode
    assert plan.requests[0].sample_index == 0
    with pytest.raises(RuntimeError, match="outstanding"):
        scheduler.schedule()
    scheduler.apply_result(executor.execute(plan))
    view = scheduler.request("a")
    assert view.state == "running" and view.cached_len == 3 and view.generated_token_ids == [13]
    plan = scheduler.schedule()
    assert shape(plan) == [("a", [13], 3, True)] and plan.requests[0].is_decode
    assert plan.requests[0].sample_index == 1 and plan.step_id == 1
    scheduler.apply_result(executor.execute(plan))
    view = scheduler.request("a")
    assert view.state == "finished" and view.completion_reason == "length"
    assert view.generated_token_ids == [13, 14] and scheduler.free_pages() == 16
    assert scheduler.schedule() is None and scheduler.idle


def test_prompt_is_cut_under_chunk_and_budget():
    scheduler = make(budget=6, chunk=4)
    scheduler.submit(RequestSpec("a", list(range(10)), 1))
    scheduler.submit(RequestSpec("b", [50, 51, 52], 1))
    executor = FakeExecutor()
    seen = []
    while True:
        plan = scheduler.schedule()
        if plan is None:
            break
        seen.append(shape(plan))
        scheduler.apply_result(executor.execute(plan))
    assert seen == [
        [("a", [0, 1, 2, 3], 0, False), ("b", [50, 51], 0, False)],      # chunk 4, then what is left of 6
        [("a", [4, 5, 6, 7], 4, False), ("b", [52], 2, True)],           # only the last portion samples
        [("a", [8, 9], 8, True)],
    ]
    assert scheduler.request("a").generated_token_ids == [10]
    assert scheduler.stats.prefill_tokens == 13 and scheduler.stats.decode_tokens == 0


def test_new_prompt_joins_running_decodes():
    scheduler = make(budget=8, chunk=8)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", [1, 2], 4))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    scheduler.submit(RequestSpec("b", [7, 8, 9], 4))
    plan = scheduler.schedule()
    assert shape(plan) == [("a", [3], 2, True), ("b", [7, 8, 9], 0, True)]
    assert [r.is_decode for r in plan.requests] == [True, False]


def test_policies_order_running_requests():
    for policy, first in (("fcfs", "a"), ("decode_first", "b")):
        scheduler = make(policy=policy, budget=4, chunk=2)
        executor = FakeExecutor()
        scheduler.submit(RequestSpec("a", list(range(9)), 2))   # still prefilling
        scheduler.submit(RequestSpec("b", [5], 3))              # decodes after its first step
        scheduler.apply_result(executor.execute(scheduler.schedule()))
        plan = scheduler.schedule()
        assert plan.requests[0].request_id == first, policy


def test_eos_wins_over_length_and_stop_tokens_count():
    scheduler = make()
    scheduler.submit(RequestSpec("a", [4], 1))
    scheduler.submit(RequestSpec("b", [8], 5, SamplingParams(stop_token_ids=[9])))
    executor = FakeExecutor(eos_token_id=5)
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    a, b = scheduler.request("a"), scheduler.request("b")
    assert a.completion_reason == "eos" and a.generated_token_ids == [5]   # the end token is kept
    assert b.completion_reason == "eos" and b.generated_token_ids == [9]


def test_submit_checks():
    scheduler = make()
    scheduler.submit(RequestSpec("a", [1], 1))
    with pytest.raises(ValueError, match="already exists"):
        scheduler.submit(RequestSpec("a", [1], 1))
    with pytest.raises(ValueError, match="prompt"):
        scheduler.submit(RequestSpec("b", [], 1))
    with pytest.raises(ValueError, match="max_new_len"):
        scheduler.submit(RequestSpec("c", [1], 0))
    with pytest.raises(ValueError, match="unknown policy"):
        make(policy="lifo")


def test_sampling_params_validation():
    assert SamplingParams().is_greedy and SamplingParams().top_k is None
    p = SamplingParams(temperature=0.8, top_k=5, top_p=0.9, min_p=0.1, seed=3, stop_token_ids=[2])
    assert (p.top_k, p.seed, p.stop_token_ids) == (5, 3, [2]) and abs(p.top_p - 0.9) < 1e-6
    for bad in (dict(temperature=-1), dict(temperature=float("nan")), dict(temperature=1, top_k=0),
                dict(temperature=1, top_p=0.0), dict(temperature=1, top_p=1.5), dict(temperature=1, min_p=2),
                dict(top_k=3), dict(top_p=0.5), dict(min_p=0.5), dict(seed=2 ** 63)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_pages_run_out_fcfs_evicts_the_newest():
    # 4 pages of 4 tokens; a and b each hold 2 pages after their prompts.
    scheduler = make(pages=4, page=4, budget=32, chunk=32)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", list(range(8)), 6))
    scheduler.submit(RequestSpec("b", list(range(20, 27)), 6))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    assert scheduler.free_pages() == 0
    # a needs a third page for position 8: b, the newest, is preempted and waits in front
    plan = scheduler.schedule()
    assert shape(plan) == [("a", [8], 8, True)]
    b = scheduler.request("b")
    assert b.state == "waiting" and b.cached_len == 0 and b.generated_token_ids == [27] and b.preemptions == 1
    assert scheduler.waiting_ids() == ["b"] and scheduler.stats.preemptions == 1
    scheduler.check_invariants()
    scheduler.apply_result(executor.execute(plan))
    # b cannot come back while a holds 3 of 4 pages (it needs 2): admission just stops
    plan = scheduler.schedule()
    assert shape(plan) == [("a", [9], 9, True)]
    scheduler.apply_result(executor.execute(plan))
    LLMServer(scheduler, executor).run_until_idle()
    a, b = scheduler.request("a"), scheduler.request("b")
    assert a.state == b.state == "finished"
    assert a.generated_token_ids == [8, 9, 10, 11, 12, 13]
    # after the preemption b recomputed prompt + kept token and went on: same tokens as undisturbed
    assert b.generated_token_ids == [27, 28, 29, 30, 31, 32]
    assert scheduler.free_pages() == 4


def test_recompute_after_preemption_prefills_up_to_the_last_token():
    # 3 pages of 4 tokens.  a (older) grows into 2 pages, b into 2: b has to give way once,
    # with four tokens generated, and comes back through a chunked prefill of prompt + generated.
    scheduler = make(pages=3, page=4, budget=8, chunk=4)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", [1, 2, 3], 6))
    scheduler.submit(RequestSpec("b", [9], 6))
    steps = []
    for _ in range(40):
        plan = scheduler.schedule()
        if plan is None:
            break
        steps.append(shape(plan))
        scheduler.apply_result(executor.execute(plan))
        scheduler.check_invariants()
    a, b = scheduler.request("a"), scheduler.request("b")
    assert a.state == "finished" and a.generated_token_ids == [4, 5, 6, 7, 8, 9]
    assert b.state == "finished" and b.generated_token_ids == [10, 11, 12, 13, 14, 15]
    assert b.preemptions == 1 and a.preemptions == 0
    b_steps = [s for step in steps for s in step if s[0] == "b"]
    # before: prompt, then one token at a time; it gives way when position 4 needs a page
    assert b_steps[:4] == [("b", [9], 0, True), ("b", [10], 1, True), ("b", [11], 2, True), ("b", [12], 3, True)]
    # after: prompt + the four kept tokens, cut by the chunk; the first portion does not sample
    # (the reference would decode token by token from len(prompt) on and sample each time)
    assert b_steps[4:] == [
        ("b", [9, 10, 11, 12], 0, False),
        ("b", [13], 4, True),
        ("b", [14], 5, True),
    ]


def test_alone_and_too_large_fails_others_continue():
    scheduler = make(pages=2, page=4, budget=32, chunk=32)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("big", list(range(9)), 2))      # 3 pages, the pool has 2
    scheduler.submit(RequestSpec("ok", [1, 2], 2))
    LLMServer(scheduler, executor).run_until_idle()
    big = scheduler.request("big")
    assert big.state == "failed" and big.error == "Insufficient memory to fulfill request big"
    assert scheduler.request("ok").state == "finished" and scheduler.free_pages() == 2
    # a running request that outgrows the whole pool while alone fails the same way
    scheduler.submit(RequestSpec("grow", list(range(7)), 5))
    LLMServer(scheduler, executor).run_until_idle()
    grow = scheduler.request("grow")
    assert grow.state == "failed" and "Insufficient memory" in grow.error and scheduler.free_pages() == 2
    assert scheduler.stats.failures == 2


def test_last_in_order_waits_instead_of_failing():
    # decided here: the reference fails the asking request when it is itself the last in
    # policy order (scheduler.rs:286-294); this scheduler makes it wait for the others.
    scheduler = make(pages=4, page=4, budget=32, chunk=32)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", list(range(7)), 3))
    scheduler.submit(RequestSpec("b", list(range(40, 48)), 3))
    scheduler.apply_result(executor.execute(scheduler.schedule()))   # a: 2 pages, b: 2 pages
    plan = scheduler.schedule()   # a fits in its page; b needs a third page and is last in order
    assert shape(plan) == [("a", [7], 7, True)]
    assert scheduler.request("b").state == "waiting"
    scheduler.apply_result(executor.execute(plan))
    LLMServer(scheduler, executor).run_until_idle()
    assert scheduler.request("b").state == "finished"
    assert scheduler.request("b").generated_token_ids == [48, 49, 50]


def test_decode_first_evicts_a_prefilling_request_first():
    # "old" has a long prompt fed two tokens a step, "young" decodes meanwhile; five pages of
    # four tokens cannot hold both.  fcfs gives way the newest request, decode_first the one
    # that is still prefilling (reference: tests.rs:507-584).
    outcome = {}
    for policy in ("fcfs", "decode_first"):
        scheduler = make(policy=policy, pages=5, page=4, budget=6, chunk=2)
        executor = FakeExecutor()
        scheduler.submit(RequestSpec("old", list(range(14)), 2))
        scheduler.submit(RequestSpec("young", [70, 71], 9))
        server = LLMServer(scheduler, executor)
        while server.run_once():
            scheduler.check_invariants()
        old, young = scheduler.request("old"), scheduler.request("young")
        assert old.state == young.state == "finished"
        assert old.generated_token_ids == [14, 15]
        assert young.generated_token_ids == list(range(72, 81))
        assert scheduler.free_pages() == 5
        outcome[policy] = (old.preemptions, young.preemptions)
    assert outcome == {"fcfs": (0, 1), "decode_first": (1, 0)}


def test_cancel_frees_and_in_flight_is_refused():
    scheduler = make()
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", [1, 2, 3, 4, 5], 3))
    scheduler.submit(RequestSpec("b", [1], 3))
    plan = scheduler.schedule()
    with pytest.raises(RuntimeError, match="in flight"):
        scheduler.cancel("a")
    scheduler.apply_result(executor.execute(plan))
    scheduler.cancel("a")
    assert scheduler.request("a").state == "cancelled" and scheduler.free_pages() == 15
    assert scheduler.running_ids() == ["b"]
    scheduler.cancel("a")  # again: no effect
    with pytest.raises(ValueError, match="unknown"):
        scheduler.cancel("zzz")
    scheduler.forget("a")
    assert not scheduler.has_request("a")
    with pytest.raises(RuntimeError, match="still live"):
        scheduler.forget("b")


def test_failing_executor_fails_the_batch_and_the_server_goes_on():
    class Failing:
        def __init__(self):
            self.calls = 0

        def execute(self, batch):
            self.calls += 1
            if self.calls == 1:
                raise RuntimeError("boom")
            return FakeExecutor().execute(batch)

    scheduler = make()
    scheduler.submit(RequestSpec("a", [1, 2], 2))
    server = LLMServer(scheduler, Failing())
    assert server.run_once()
    a = scheduler.request("a")
    assert a.state == "failed" and a.error == "RuntimeError: boom" and scheduler.free_pages() == 16
    scheduler.submit(RequestSpec("b", [1, 2], 2))
    server.run_until_idle()
    assert scheduler.request("b").state == "finished"


def test_malformed_results_change_nothing():
    scheduler = make()
    scheduler.submit(RequestSpec("a", [1, 2], 2))
    plan = scheduler.schedule()
    good = FakeExecutor().execute(plan)
    bad_results = [
        ExecutionResult(plan.step_id + 1, good.request_results),                      # stale step
        ExecutionResult(plan.step_id, []),                                            # wrong count
        ExecutionResult(plan.step_id, [RequestResult("b", [3], 2)]),                  # other request
        ExecutionResult(plan.step_id, [RequestResult("a", [3], 1)]),                  # wrong delta
        ExecutionResult(plan.step_id, [RequestResult("a", [], 2)]),                   # token missing
        ExecutionResult(plan.step_id, [RequestResult("a", [3, 4], 2)]),               # two tokens
    ]
    for bad in bad_results:
        with pytest.raises((ValueError, RuntimeError)):
            scheduler.apply_result(bad)
        view = scheduler.request("a")
        assert view.cached_len == 0 and view.generated_token_ids == [] and scheduler.has_outstanding
    scheduler.apply_result(good)
    assert scheduler.request("a").cached_len == 2
    with pytest.raises(RuntimeError, match="no batch"):
        scheduler.apply_result(good)
    plan = scheduler.schedule()
    with pytest.raises(RuntimeError, match="stale"):
        scheduler.fail_batch(type("P", (), {"step_id": 99})(), "x") if False else scheduler.fail_batch(
            __import__("einf_b200.engine", fromlist=["BatchPlan"]).BatchPlan(99, []), "x")
    scheduler.fail_batch(plan, "stop")
    assert scheduler.request("a").state == "failed"


def test_windowed_group_frees_pages_while_decoding():
    scheduler = Scheduler("fcfs", [GroupSpec(64, 4), GroupSpec(6, 4, 5)], 16, 16, 0)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", list(range(10)), 40))
    LLMServer(scheduler, executor).run_until_idle()
    assert scheduler.request("a").state == "finished"
    assert scheduler.high_water(1) <= 4 and scheduler.stats.window_pages_freed > 5
    assert scheduler.free_pages(0) == 64 and scheduler.free_pages(1) == 6


def test_state_slots_in_the_plan():
    scheduler = make(slots=2)
    scheduler.submit(RequestSpec("a", [1], 2))
    scheduler.submit(RequestSpec("b", [1], 2))
    scheduler.submit(RequestSpec("c", [1], 2))
    plan = scheduler.schedule()
    assert [r.state_slot for r in plan.requests] == [0, 1]  # c waits for a slot
    assert scheduler.waiting_ids() == ["c"]
    executor = FakeExecutor()
    scheduler.apply_result(executor.execute(plan))
    LLMServer(scheduler, executor).run_until_idle()
    assert scheduler.request("c").state == "finished"


# ---------------------------------------------------------------------------
# Several decode steps per plan (decode_lookahead)
def make_ahead(lookahead, policy="fcfs", pages=16, page=4, budget=8, chunk=8, window=0):
    return Scheduler(policy, [GroupSpec(pages, page, window)], budget, chunk, 0, lookahead)


def test_lookahead_covers_steps_only_when_it_costs_nobody():
    scheduler = make_ahead(4)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    plan = scheduler.schedule()
    assert plan.decode_steps == 1                       # a prompt portion: one step
    scheduler.apply_result(executor.execute(plan))
    plan = scheduler.schedule()
    # one decoding request, nobody waits: four steps, pages for positions 3..6 in the table
    assert plan.decode_steps == 4 and shape(plan) == [("a", [13], 3, True)]
    assert len(plan.requests[0].block_tables[0]) == 2
    scheduler.apply_result(executor.execute(plan))
    view = scheduler.request("a")
    assert view.cached_len == 7 and view.generated_token_ids == [13, 14, 15, 16, 17]
    assert scheduler.stats.steps == 5 and scheduler.stats.decode_tokens == 4
    # a request that waits for admission: back to single steps until it decodes too
    scheduler.submit(RequestSpec("b", [50, 51], 3))
    plan = scheduler.schedule()
    assert plan.decode_steps == 1 and [r.request_id for r in plan.requests] == ["a", "b"]
    scheduler.apply_result(executor.execute(plan))
    plan = scheduler.schedule()
    # both decode; b has two tokens to go: the plan covers two steps
    assert plan.decode_steps == 2
    scheduler.apply_result(executor.execute(plan))
    assert scheduler.request("b").state == "finished" and scheduler.request("b").generated_token_ids == [52, 53, 54]
    plan = scheduler.schedule()
    assert plan.decode_steps == 1                       # a has one token to go
    scheduler.apply_result(executor.execute(plan))
    assert scheduler.request("a").state == "finished" and len(scheduler.request("a").generated_token_ids) == 9
    assert scheduler.free_pages() == 16 and scheduler.idle
    scheduler.check_invariants()


def test_lookahead_end_of_sequence_on_the_way_drops_the_rest():
    scheduler = make_ahead(4)
    executor = FakeExecutor(eos_token_id=15)
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    scheduler.submit(RequestSpec("b", [30], 9))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    plan = scheduler.schedule()
    assert plan.decode_steps == 4
    result = executor.execute(plan)
    assert [r.generated_token_ids for r in result.request_results] == [[14, 15], [32, 33, 34, 35]]
    scheduler.apply_result(result)
    a, b = scheduler.request("a"), scheduler.request("b")
    assert a.state == "finished" and a.completion_reason == "eos" and a.generated_token_ids == [13, 14, 15]
    assert b.state == "running" and b.cached_len == 5 and len(b.generated_token_ids) == 5
    LLMServer(scheduler, executor).run_until_idle()
    assert scheduler.free_pages() == 16
    scheduler.check_invariants()


def test_lookahead_needs_its_pages_and_never_preempts_for_them():
    scheduler = make_ahead(8, pages=3, page=4)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", list(range(6)), 20))
    scheduler.submit(RequestSpec("b", list(range(5)), 20))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    # three pages: a holds two, b holds... the pool has no page to look ahead with
    plan = scheduler.schedule()
    assert plan is not None and plan.decode_steps == 1
    assert scheduler.stats.preemptions <= 1


def test_lookahead_is_all_or_nothing_across_requests():
    # Pool of 7 pages of 4: a and b each hold two after their prompts, and each wants one more
    # page to look five steps ahead, c (longer prompt, three pages... ) wants two: together they
    # ask for more than what is free, so nobody gets any and the step is the plain single step.
    scheduler = make_ahead(6, pages=8, page=4, budget=32, chunk=16)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", list(range(7)), 20))
    scheduler.submit(RequestSpec("b", list(range(7)), 20))
    scheduler.submit(RequestSpec("c", list(range(7)), 20))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    assert scheduler.free_pages() == 2                # six held; tokens 7..12 need a third page each
    held = {i: list(scheduler.block_table(i)) for i in "abc"}
    plan = scheduler.schedule()
    assert plan.decode_steps == 1
    # the step's own token (position 7) still fits the second page: nobody took a page
    assert scheduler.free_pages() == 2
    assert {i: list(scheduler.block_table(i)) for i in "abc"} == held
    scheduler.apply_result(executor.execute(plan))
    scheduler.check_invariants()
    # with room for everybody's lookahead the plan does cover several steps
    roomy = make_ahead(6, pages=16, page=4, budget=32, chunk=16)
    for name in "abc":
        roomy.submit(RequestSpec(name, list(range(7)), 20))
    roomy.apply_result(executor.execute(roomy.schedule()))
    assert roomy.schedule().decode_steps == 6


def test_no_plan_holds_more_requests_than_the_engine_has_rows():
    # Token budget and pages would admit all of them at once; the engine's step buffer, sampler
    # and block-table rows are made for max_requests, so the scheduler must stop there.
    scheduler = Scheduler("fcfs", [GroupSpec(256, 16)], 128, 128, 0, 1, 8)
    assert scheduler.max_requests == 8
    for index in range(100):
        scheduler.submit(RequestSpec(f"r{index}", [1, 2, 3, 4], 3))
    executor = FakeExecutor()
    most = 0
    while True:
        plan = scheduler.schedule()
        if plan is None:
            break
        most = max(most, len(plan.requests))
        assert len(plan.requests) <= 8 and len(scheduler.running_ids()) <= 8
        scheduler.apply_result(executor.execute(plan))
    assert most == 8
    assert all(scheduler.request(f"r{index}").state == "finished" for index in range(100))
    assert scheduler.free_pages() == 256
    scheduler.check_invariants()
    with pytest.raises(ValueError, match="max_requests"):
        Scheduler("fcfs", [GroupSpec(4, 4)], 8, 8, 0, 1, -1)


def test_a_plan_of_several_steps_can_be_applied_step_by_step():
    """An executor that reports every step while the later steps of the plan run: the scheduler
    takes one token per live request and call, keeps the plan outstanding until its last step,
    ends a request at its end-of-sequence token and takes nothing for it afterwards."""
    scheduler = make_ahead(4)
    executor = FakeExecutor(eos_token_id=15)
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    scheduler.submit(RequestSpec("b", [30], 9))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    plan = scheduler.schedule()
    assert plan.decode_steps == 4 and scheduler.outstanding_steps_left == 4
    with pytest.raises(ValueError, match="one token in"):
        scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [14, 15], 2, False), RequestResult("b", [32], 1, False)]))
    scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [14], 1, False), RequestResult("b", [32], 1, False)]))
    assert scheduler.request("a").generated_token_ids == [13, 14] and scheduler.request("b").cached_len == 2
    assert scheduler.has_outstanding and scheduler.outstanding_steps_left == 3
    with pytest.raises(RuntimeError, match="outstanding"):
        scheduler.schedule()
    with pytest.raises(RuntimeError, match="step by step"):
        scheduler.apply_result(ExecutionResult(plan.step_id, [RequestResult("a", [15], 1, True), RequestResult("b", [33], 1, False)]))
    scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [15], 1, True), RequestResult("b", [33], 1, False)]))
    a = scheduler.request("a")
    assert a.state == "finished" and a.completion_reason == "eos" and a.generated_token_ids == [13, 14, 15]
    with pytest.raises(ValueError, match="ended on an earlier step"):
        scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [16], 1, False), RequestResult("b", [34], 1, False)]))
    scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [], 0, False), RequestResult("b", [34], 1, False)]))
    assert scheduler.has_outstanding
    scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [], 0, False), RequestResult("b", [35], 1, False)]))
    assert not scheduler.has_outstanding and scheduler.outstanding_steps_left == 0
    b = scheduler.request("b")
    assert b.state == "running" and b.cached_len == 5 and b.generated_token_ids == [31, 32, 33, 34, 35]
    assert scheduler.stats.steps == 5
    LLMServer(scheduler, executor).run_until_idle()       # the server reports every step too
    assert scheduler.request("b").state == "finished" and scheduler.free_pages() == 16
    scheduler.check_invariants()
    # a failure in the middle of a plan fails what is still live, not what has ended
    scheduler = make_ahead(4)
    executor = FakeExecutor(eos_token_id=15)
    scheduler.submit(RequestSpec("a", [10, 11, 13], 9))
    scheduler.submit(RequestSpec("b", [30], 9))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    plan = scheduler.schedule()
    scheduler.apply_step(ExecutionResult(plan.step_id, [RequestResult("a", [15], 1, True), RequestResult("b", [32], 1, False)]))
    scheduler.fail_batch(plan, "made-up fault")
    assert scheduler.request("a").state == "finished" and scheduler.request("b").state == "failed"
    assert scheduler.free_pages() == 16 and scheduler.idle


def test_a_request_can_be_cancelled_between_the_steps_of_a_streamed_plan():
    scheduler = make_ahead(4)
    executor = FakeExecutor()
    server = LLMServer(scheduler, executor)
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    scheduler.submit(RequestSpec("b", [30], 9))
    server.run_once()                                   # the prompts
    # while a plan of one step is out, its requests are in flight (as in the reference)
    single = make()
    single.submit(RequestSpec("x", [1, 2], 3))
    single.schedule()
    with pytest.raises(RuntimeError, match="in flight"):
        single.cancel("x")
    server.run_once()                                   # first step of a plan of four
    assert scheduler.has_outstanding and scheduler.outstanding_steps_left == 3
    scheduler.cancel("a")
    assert scheduler.request("a").state == "cancelled" and len(scheduler.request("a").generated_token_ids) == 2
    held = scheduler.free_pages()
    server.run_until_idle()                             # the executor still reports tokens for a: dropped
    assert len(scheduler.request("a").generated_token_ids) == 2
    b = scheduler.request("b")
    assert b.state == "finished" and b.generated_token_ids == list(range(31, 40))
    assert scheduler.free_pages() == 16 and scheduler.free_pages() > held and scheduler.idle
    scheduler.check_invariants()
    # cancelling every request of a plan ends the plan with its next step
    scheduler.submit(RequestSpec("c", [50, 51], 9))
    server.run_once()
    server.run_once()
    assert scheduler.has_outstanding
    scheduler.cancel("c")
    assert server.run_once() and not scheduler.has_outstanding
    assert not server.run_once() and scheduler.idle


def test_the_server_applies_a_streamed_plan_one_step_per_call():
    scheduler = make_ahead(4)
    executor = FakeExecutor()
    server = LLMServer(scheduler, executor)
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    assert server.run_once()                     # the prompt
    lengths = []
    while server.run_once():
        lengths.append(len(scheduler.request("a").generated_token_ids))
    assert lengths == list(range(2, 10))         # one more token after every call
    executor.report_every_step = False           # one report per plan
    scheduler.submit(RequestSpec("b", [10, 11, 12], 9))
    server.run_once()
    lengths = []
    while server.run_once():
        lengths.append(len(scheduler.request("b").generated_token_ids))
    assert lengths == [5, 9]


def test_lookahead_results_are_checked():
    scheduler = make_ahead(4)
    executor = FakeExecutor()
    scheduler.submit(RequestSpec("a", [10, 11, 12], 9))
    scheduler.apply_result(executor.execute(scheduler.schedule()))
    plan = scheduler.schedule()
    assert plan.decode_steps == 4
    with pytest.raises(ValueError, match="stopped early"):
        scheduler.apply_result(ExecutionResult(plan.step_id, [RequestResult("a", [14, 15], 2, False)]))
    with pytest.raises(ValueError, match="1 to 4"):
        scheduler.apply_result(ExecutionResult(plan.step_id, [RequestResult("a", [1, 2, 3, 4, 5], 5, False)]))
    with pytest.raises(ValueError, match="differs from the steps"):
        scheduler.apply_result(ExecutionResult(plan.step_id, [RequestResult("a", [14, 15, 16, 17], 1, False)]))
    assert scheduler.request("a").cached_len == 3        # nothing changed
    scheduler.apply_result(executor.execute(plan))
    assert scheduler.request("a").cached_len == 7


@pytest.mark.parametrize("window", [0, 6])
def test_lookahead_generates_the_same_tokens(window):
    outputs = []
    for lookahead in (1, 3, 8):
        scheduler = make_ahead(lookahead, policy="decode_first", pages=40, window=window)
        executor = FakeExecutor(eos_token_id=47)
        for name, prompt, new in (("a", [1, 2, 3], 17), ("b", [40], 30), ("c", list(range(20, 29)), 5)):
            scheduler.submit(RequestSpec(name, prompt, new))
        server = LLMServer(scheduler, executor)
        server.run_until_idle()
        outputs.append({n: (scheduler.request(n).generated_token_ids, scheduler.request(n).completion_reason) for n in "abc"})
        assert scheduler.free_pages() == 40
        scheduler.check_invariants()
    assert outputs[0] == outputs[1] == outputs[2]
    assert outputs[0]["b"][1] == "eos"


@pytest.mark.parametrize("seed", range(6))
def test_lookahead_under_random_arrivals_cancels_and_pressure(seed):
    """Random arrivals, lengths, policies, a small pool (so preemption happens) and cancels, with a
    lookahead: every request ends with exactly the tokens it must have (the fake executor answers
    last token + 1, so they are known in closed form), no page is lost, and the pool is whole again."""
    import random

    rng = random.Random(seed)
    eos = 1000
    scheduler = Scheduler(rng.choice(["fcfs", "decode_first"]), [GroupSpec(14, 4, rng.choice([0, 0, 9]))],
                          rng.choice([6, 12, 32]), rng.choice([3, 8]), 0, rng.choice([2, 3, 5]))
    executor = FakeExecutor(eos_token_id=eos)
    specs, cancelled, arrivals = {}, set(), []
    for index in range(14):
        prompt = [rng.randrange(2, 900) for _ in range(rng.randrange(1, 17))]
        if rng.random() < 0.3:
            prompt[-1] = eos - rng.randrange(1, 6)         # will hit the end-of-sequence token on the way
        specs[f"r{index}"] = (prompt, rng.randrange(1, 12))
        arrivals.append((rng.randrange(0, 30), f"r{index}"))
    arrivals.sort()
    step = 0
    while arrivals or not scheduler.idle:
        while arrivals and arrivals[0][0] <= step:
            _, name = arrivals.pop(0)
            scheduler.submit(RequestSpec(name, *specs[name]))
        if rng.random() < 0.05:
            live = scheduler.waiting_ids() + scheduler.running_ids()
            if live:
                victim = rng.choice(live)
                scheduler.cancel(victim)
                cancelled.add(victim)
        plan = scheduler.schedule()
        if plan is not None:
            assert 1 <= plan.decode_steps <= scheduler.decode_lookahead
            scheduler.apply_result(executor.execute(plan))
        scheduler.check_invariants()
        step += 1
        assert step < 2000
    assert scheduler.free_pages() == 14
    for name, (prompt, new) in specs.items():
        view = scheduler.request(name)
        if name in cancelled:
            assert view.state == "cancelled"
            continue
        if view.state == "failed":
            assert "Insufficient memory" in view.error
            continue
        expected = []
        for i in range(new):
            expected.append(prompt[-1] + 1 + i)
            if expected[-1] == eos:
                break
        assert view.state == "finished" and view.generated_token_ids == expected, name
        assert view.completion_reason == ("eos" if expected[-1] == eos else "length")
