"""The serving loop and the Python entry point.

``LLMServer(scheduler, executor)`` with ``run_once`` and ``run_until_idle`` is
the reference's loop (``src/einf/lib.py:5-27``): schedule, execute, apply; an
executor that raises fails the batch and the server goes on.  :class:`Engine`
builds scheduler, runner and executor from a model folder and adds ``submit``
and ``generate``.
"""
from __future__ import annotations

import itertools
from pathlib import Path
from typing import Iterable, Optional, Sequence

from ..cache.control import RequestSpec, SamplingParams, Scheduler
from ..config.base import ModelConfig
from ..config.engine import EngineConfig
from .executor import GpuExecutor
from .runner import ModelRunner


class LLMServer:
    def __init__(self, scheduler: Scheduler, executor) -> None:
        self.scheduler = scheduler
        self.executor = executor

        #: a plan of several decode steps whose steps are reported one by one (its later steps run
        #: on the device while the host applies the earlier ones)
        self._in_flight = None

    def run_once(self) -> bool:
        """One step: schedule, execute, apply (``lib.py:10-23``).  A plan that covers several decode
        steps is started whole on the device and applied one step per call, if the executor
        reports every step; otherwise it is applied whole."""
        batch = self._in_flight
        if batch is None:
            batch = self.scheduler.schedule()
            if batch is None:
                return False
            streaming = batch.decode_steps > 1 and getattr(self.executor, "report_every_step", False) \
                and hasattr(self.executor, "begin")
            if not streaming:
                try:
                    result = self.executor.execute(batch)
                except Exception as error:  # the batch fails, the server lives (lib.py:16-20)
                    self.scheduler.fail_batch(batch, f"{type(error).__name__}: {error}")
                    return True
                self.scheduler.apply_result(result)
                return True
            try:
                self.executor.begin(batch)
            except Exception as error:
                self.scheduler.fail_batch(batch, f"{type(error).__name__}: {error}")
                return True
            self._in_flight = batch
        try:
            result = self.executor.next_step()
        except Exception as error:
            self._in_flight = None
            self.scheduler.fail_batch(batch, f"{type(error).__name__}: {error}")
            return True
        self.scheduler.apply_step(result)
        if not self.scheduler.has_outstanding:
            self._in_flight = None
        return True

    def run_until_idle(self) -> None:
        while self.run_once():
            pass


class Engine:
    """A model on one GPU with its cache, scheduler and sampler."""

    def __init__(self, runner: ModelRunner, eos_token_ids: Optional[Iterable[int]] = None,
                 decode_lookahead: Optional[int] = None) -> None:
        """``decode_lookahead`` overrides the engine configuration's (a second engine over the same
        runner, and so the same weights and cache, may differ in it)."""
        self.runner = runner
        cfg = runner.engine_config
        # Several decode steps per report only for models whose parts all run from device memory
        # alone: the steps after the first run on inputs that a kernel moved on, which the host
        # has not seen (a mixer with per-request state keeps it in its slot on the device and is
        # fine; one that reads its slots on the host is not).
        from .. import ops

        lookahead = cfg.decode_lookahead if decode_lookahead is None else int(decode_lookahead)
        if not runner.device_driven or len(runner.group_specs()) > ops.ADVANCE_MAX_GROUPS:
            lookahead = 1
        self.scheduler = Scheduler(
            cfg.policy,
            runner.group_specs(),
            cfg.max_batch_len,
            cfg.max_prefill_chunk_len,
            runner.num_state_slots,
            lookahead,
            cfg.max_requests,
        )
        if eos_token_ids is None:
            eos_token_ids = runner.config.eos_token_ids
        self.executor = GpuExecutor(runner, eos_token_ids)
        self.server = LLMServer(self.scheduler, self.executor)
        self._ids = itertools.count()

    @classmethod
    def from_folder(cls, folder: str | Path, engine_config: Optional[EngineConfig] = None, **kwargs) -> "Engine":
        return cls(ModelRunner.from_folder(folder, engine_config or EngineConfig()), **kwargs)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, engine_config: Optional[EngineConfig] = None, **kwargs) -> "Engine":
        return cls(ModelRunner.from_random(config, seed, engine_config or EngineConfig()), **kwargs)

    # ------------------------------------------------------------------
    def submit(
        self,
        prompt_token_ids: Sequence[int],
        max_new_len: int,
        sampling_params: Optional[SamplingParams] = None,
        request_id: Optional[str] = None,
    ) -> str:
        if request_id is None:
            request_id = f"request-{next(self._ids)}"
        total = len(prompt_token_ids) + max_new_len
        if total > self.runner.max_sequence_len:
            raise ValueError(
                f"request {request_id!r} may reach {total} tokens; the engine holds at most "
                f"{self.runner.max_sequence_len} per request"
            )
        vocab = self.runner.vocab_size
        if any(not 0 <= int(t) < vocab for t in prompt_token_ids):
            raise ValueError(f"request {request_id!r} has a token id outside the vocabulary of {vocab}")
        self.scheduler.submit(RequestSpec(request_id, list(prompt_token_ids), max_new_len, sampling_params))
        return request_id

    def step(self) -> bool:
        return self.server.run_once()

    def run_until_idle(self) -> None:
        self.server.run_until_idle()

    def request(self, request_id: str):
        return self.scheduler.request(request_id)

    def cancel(self, request_id: str) -> None:
        self.scheduler.cancel(request_id)

    def generate(
        self,
        prompts: Sequence[Sequence[int]],
        max_new_len: int,
        sampling_params: Optional[SamplingParams] = None,
    ) -> list[list[int]]:
        """Token ids in, token ids out: run the prompts to completion."""
        ids = [self.submit(prompt, max_new_len, sampling_params) for prompt in prompts]
        self.run_until_idle()
        outputs, errors = [], []
        for request_id in ids:
            view = self.scheduler.request(request_id)
            if view.state == "failed":
                errors.append(f"{request_id} failed: {view.error}")
            outputs.append(list(view.generated_token_ids))
            # every record is dropped before an error is raised, so the ids can be used again
            self.scheduler.forget(request_id)
        if errors:
            raise RuntimeError("; ".join(errors))
        return outputs
