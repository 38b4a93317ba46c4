"""Executors: turn a batch plan into an execution result.

:class:`GpuExecutor` is the product path: step function, sampler, one
device-to-host read of the sampled tokens and the status word, end-of-sequence
test (``src/einf/executors/torch/executor.py:28-117``).  :class:`FakeExecutor`
answers ``last input token + 1`` without a model, for tests of the control
plane (``src/einf/executors/fake.py:5-18``).
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from .. import ops
from ..cache.control import BatchPlan, ExecutionResult, RequestResult
from ..sampling.sampler import Sampler
from .runner import ModelRunner


class FakeExecutor:
    def __init__(self, eos_token_id: int = -1) -> None:
        self.eos_token_id = eos_token_id
        self.batches: list[BatchPlan] = []

    def execute(self, batch: BatchPlan) -> ExecutionResult:
        self.batches.append(batch)
        results = []
        for request in batch.requests:
            tokens, is_eos = [], False
            if request.need_sample:
                # with a lookahead: one token per step, each the input of the next, up to the one that ends it
                for step in range(batch.decode_steps):
                    tokens.append(request.input_token_ids[-1] + 1 + step)
                    is_eos = tokens[-1] == self.eos_token_id or tokens[-1] in request.sampling_params.stop_token_ids
                    if is_eos:
                        break
            consumed = len(tokens) if batch.decode_steps > 1 else len(request.input_token_ids)
            results.append(RequestResult(request.request_id, tokens, consumed, is_eos))
        return ExecutionResult(batch.step_id, results)

    # The step-by-step reports of a plan that covers several decode steps (see GpuExecutor.begin).
    report_every_step = True

    def begin(self, batch: BatchPlan) -> None:
        self._whole = self.execute(batch)
        self._cursor = 0

    def next_step(self) -> ExecutionResult:
        results = []
        for outcome in self._whole.request_results:
            tokens = list(outcome.generated_token_ids)
            if self._cursor < len(tokens):
                last = self._cursor == len(tokens) - 1
                results.append(RequestResult(outcome.request_id, [tokens[self._cursor]], 1, outcome.is_eos and last))
            else:
                results.append(RequestResult(outcome.request_id, [], 0, False))
        self._cursor += 1
        return ExecutionResult(self._whole.step_id, results)


class GpuExecutor:
    def __init__(self, runner: ModelRunner, eos_token_ids: Iterable[int] = ()) -> None:
        self.runner = runner
        self.eos_token_ids = frozenset(int(t) for t in eos_token_ids)
        self.sampler = Sampler(runner.runtime.device, runner.engine_config.max_requests)
        pin = runner.runtime.device.type == "cuda"
        self._host = torch.zeros(runner.engine_config.max_requests + 1, dtype=torch.int32, pin_memory=pin)
        self._device = torch.zeros_like(self._host, device=runner.runtime.device)
        self.d2h_bytes = 0
        #: plans that covered several decode steps
        self.ahead_batches = 0
        #: with a plan of several decode steps: report each step's tokens to the host as soon as
        #: that step is done, while the later steps of the plan already run (begin / next_step);
        #: false: one report at the end of the plan (execute)
        self.report_every_step = bool(getattr(runner.engine_config, "report_every_step", True))
        self._streams: Optional[dict] = None

    def execute(self, batch: BatchPlan) -> ExecutionResult:
        runner = self.runner
        # (request_id, tokens, need_sample, sample_index, sampling_params, start, state_slot)
        summary = batch.summary()
        sampling = [entry for entry in summary if entry[2]]
        count = len(sampling)
        steps = batch.decode_steps
        if steps > 1:
            return self._execute_ahead(batch, summary, steps)
        with runner._guard(), torch.inference_mode():
            output = runner.step(batch)
            tokens = self.sampler.sample(
                output.logits, [entry[4] for entry in sampling], [entry[3] for entry in sampling]
            )
            # one small kernel writes the tokens and the status word into pinned host memory
            ops.report(tokens, count, output.context.status, self._host)
            runner.synchronize()
        self.d2h_bytes += (count + 1) * 4
        host = self._host[:count + 1].tolist()
        runner.check_status(host[count])
        results = []
        cursor = 0
        for request_id, num_tokens, need_sample, _, params, _, _ in summary:
            if need_sample:
                token = host[cursor]
                cursor += 1
                is_eos = token in self.eos_token_ids or token in params.stop_token_ids
                results.append(RequestResult(request_id, [token], num_tokens, is_eos))
            else:
                results.append(RequestResult(request_id, [], num_tokens, False))
        return ExecutionResult(batch.step_id, results)

    def begin(self, batch: BatchPlan) -> None:
        """Start a plan that covers several decode steps and return at once: every step of it is
        put on the stream now (the step, the sampler, a kernel that moves the inputs on by one
        token, and a small kernel that writes the step's tokens and the status word into the
        step's own row of pinned host memory, followed by an event).  ``next_step`` then hands
        out one step's result at a time, waiting only for that step's event: the host reads step
        N and tells the scheduler while the device is at step N + 1."""
        runner = self.runner
        summary = batch.summary()
        steps, count = batch.decode_steps, len(summary)
        self.ahead_batches += 1
        params = [entry[4] for entry in summary]
        width = count + 1
        if self._streams is None or self._streams["rows"].shape[0] < steps or self._streams["rows"].shape[1] < width:
            pin = runner.runtime.device.type == "cuda"
            rows = torch.zeros((max(steps, 8), max(width, runner.engine_config.max_requests + 1)), dtype=torch.int32,
                               pin_memory=pin)
            tokens = torch.zeros(rows.shape, dtype=torch.int32, device=runner.runtime.device)
            events = [torch.cuda.Event() if pin else None for _ in range(rows.shape[0])]
            self._streams = {"rows": rows, "tokens": tokens, "events": events}
        rows, device_tokens, events = self._streams["rows"], self._streams["tokens"], self._streams["events"]
        with runner._guard(), torch.inference_mode():
            output = runner.step(batch)
            stream = ops.current_stream() if events[0] is not None else None
            for step in range(steps):
                if step > 0:
                    runner.advance_decode(output, device_tokens[step - 1, :count])
                    output = runner.repeat_step(output)
                sampled = self.sampler.sample(output.logits, params, [entry[3] + step for entry in summary])
                device_tokens[step, :count].copy_(sampled)
                ops.report(device_tokens[step], count, output.context.status, rows[step])
                if stream is not None:
                    events[step].record(stream)
        self._streams.update(batch=batch, summary=summary, steps=steps, cursor=0, ended=set())

    def next_step(self) -> ExecutionResult:
        """The result of the next step of the plan ``begin`` started: one token for every request
        that has not ended on an earlier step of the plan, nothing for one that has."""
        state = self._streams
        if state is None or state.get("batch") is None:
            raise RuntimeError("no plan is in flight")
        index, summary, count = state["cursor"], state["summary"], len(state["summary"])
        event = state["events"][index]
        if event is not None:
            event.synchronize()
        host = state["rows"][index, :count + 1].tolist()
        self.d2h_bytes += (count + 1) * 4
        try:
            self.runner.check_status(host[count])
        except Exception:
            state["batch"] = None
            raise
        ended = state["ended"]
        results = []
        for position, (request_id, _, _, _, params, _, _) in enumerate(summary):
            if request_id in ended:
                results.append(RequestResult(request_id, [], 0, False))
                continue
            token = host[position]
            is_eos = token in self.eos_token_ids or token in params.stop_token_ids
            if is_eos:
                ended.add(request_id)
            results.append(RequestResult(request_id, [token], 1, is_eos))
        state["cursor"] = index + 1
        step_id = state["batch"].step_id
        if state["cursor"] >= state["steps"] or len(ended) == count:
            state["batch"] = None
        return ExecutionResult(step_id, results)

    def _execute_ahead(self, batch: BatchPlan, summary, steps: int) -> ExecutionResult:
        """Several decode steps before the host looks: after each step a small kernel moves the
        step's inputs on by one token on the device (the sampled token becomes the input, position
        and cache slot advance through the block table, which already holds the pages), and the
        same step runs again.  One read at the end brings every step's tokens; what a request
        sampled after its end-of-sequence token is dropped."""
        runner = self.runner
        self.ahead_batches += 1
        count = len(summary)
        params = [entry[4] for entry in summary]
        need = steps * count + 1
        if self._host.numel() < need:
            pin = runner.runtime.device.type == "cuda"
            self._host = torch.zeros(need, dtype=torch.int32, pin_memory=pin)
            self._device = torch.zeros_like(self._host, device=runner.runtime.device)
        with runner._guard(), torch.inference_mode():
            output = runner.step(batch)
            for step in range(steps):
                if step > 0:
                    runner.advance_decode(output, self._device[(step - 1) * count:step * count])
                    output = runner.repeat_step(output)
                tokens = self.sampler.sample(output.logits, params, [entry[3] + step for entry in summary])
                self._device[step * count:(step + 1) * count].copy_(tokens)
            self._device[steps * count:need].copy_(output.context.status)
            self._host[:need].copy_(self._device[:need], non_blocking=True)
            runner.synchronize()
        self.d2h_bytes += need * 4
        host = self._host[:need].tolist()
        runner.check_status(host[steps * count])
        results = []
        for index, (request_id, _, _, _, request_params, _, _) in enumerate(summary):
            tokens, is_eos = [], False
            for step in range(steps):
                token = host[step * count + index]
                tokens.append(token)
                is_eos = token in self.eos_token_ids or token in request_params.stop_token_ids
                if is_eos:
                    break
            results.append(RequestResult(request_id, tokens, len(tokens), is_eos))
        return ExecutionResult(batch.step_id, results)
