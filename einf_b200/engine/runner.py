"""The step function: run the tokens of one batch through the model, from the cache.

A step takes requests that each bring their next tokens (a portion of a prompt
or one decoded token, cut anywhere), runs only those tokens as one packed
batch, reads earlier tokens from the pages earlier steps wrote, and returns the
logits at the wanted places.  It is the role of ``TorchExecutor`` +
``QwenModelRunner.forward`` in the reference
(``src/einf/executors/torch/executor.py:28-117``, ``qwen.py:742-778``), without
its per-request Python loop inside every layer (``qwen.py:426-487``): every
kernel here takes the whole batch.

There is no CPU path: a runner refuses a device that is not CUDA.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import torch

from .. import ops
from ..cache.control import GroupSpec
from ..cache.storage import CacheStorage
from ..config.base import ModelConfig
from ..config.engine import EngineConfig
from ..config.registry import load_config
from ..parts.base import Part, Runtime, StateNeed, StepContext
from ..parts.model import DecoderModel, expected_tensors, kernel_libraries
from ..weights.loader import load_tensors
from ..weights.random import random_tensors
from .batch import StepInputBuilder, as_plan

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class StepError(RuntimeError):
    """A kernel reported a fault through the status word."""


@dataclass
class StepOutput:
    logits: torch.Tensor                     # [S, vocab] float32 on the device
    rows_of_request: list[tuple[int, int]]   # per request: (first row, count) in logits
    context: StepContext
    #: for a step that was a graph replay: (graph, its logits, its kernel count, live requests)
    replay: Optional[tuple] = None


_NO_GUARD = contextlib.nullcontext()


class ModelRunner:
    def __init__(self, config: ModelConfig, tensors, engine_config: EngineConfig) -> None:
        device = torch.device(engine_config.device)
        self._check_device(device)
        self.config = config
        self.engine_config = engine_config
        self.runtime = Runtime(_TORCH_DTYPES[engine_config.dtype], device)
        if self.runtime.dtype == torch.float32:
            # The 32-bit path rounds nothing: no TF32 in any library call either.
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        spec = config.model_spec()
        ops.ensure_built(kernel_libraries(spec, self.runtime))
        with self._guard():
            self.model = DecoderModel(spec, tensors, self.runtime)
        plan = self.model.cache_plan
        page = engine_config.block_len
        if engine_config.max_tokens is not None:
            # Every live request may leave its last page partly empty.
            base_pages = -(-engine_config.max_tokens // page)
        else:
            base_pages = engine_config.num_blocks
        self.pages_per_group = []
        for window in plan.group_windows:
            pages = base_pages
            if window:
                per_request = -(-(window + engine_config.max_prefill_chunk_len) // page) + 1
                pages = min(pages, engine_config.max_requests * per_request)
            self.pages_per_group.append(pages)
        self.page_size = page
        self.num_state_slots = engine_config.max_requests if plan.has_state else 0
        self.storage = CacheStorage(
            plan, self.pages_per_group, page, self.num_state_slots, self.runtime.dtype, device
        )
        self._state_tensors = self.storage.state_tensors
        full_pages = [p for p, w in zip(self.pages_per_group, plan.group_windows) if not w]
        max_len = (min(full_pages) if full_pages else base_pages) * page
        max_position = getattr(config, "max_position_embeddings", None)
        if max_position:
            max_len = min(max_len, int(max_position))
        if engine_config.max_sequence_len:
            max_len = min(max_len, int(engine_config.max_sequence_len))
        #: longest sequence one request may reach
        self.max_sequence_len = max_len
        self.table_width = -(-max_len // page)
        self.inputs = StepInputBuilder(
            device,
            page,
            self.pages_per_group,
            plan.group_windows,
            spec.vocab_size,
            self.table_width,
            max_tokens=max(engine_config.max_batch_len, engine_config.max_requests),
            max_requests=engine_config.max_requests,
        )
        self.vocab_size = spec.vocab_size
        self.steps = 0
        #: every part runs from device memory alone (none reads device values on the host): its
        #: steps can be captured in CUDA graphs and repeated on inputs that a kernel moved on
        self.device_driven = all(
            getattr(part, "graph_safe", True) for block in self.model.blocks for part in vars(block).values()
        )
        #: decode-only steps replay a CUDA graph captured per batch-size bucket
        self.graphs_enabled = (
            bool(engine_config.use_cuda_graphs) and self.runtime.device.type == "cuda" and self.device_driven
        )
        #: one part of every group whose launches take more from a step than its tensors' shapes
        keyed = {}
        for block in self.model.blocks:
            for part in vars(block).values():
                if isinstance(part, Part) and type(part).launch_key is not Part.launch_key:
                    keyed.setdefault(part.launch_group(), part)
        self._keyed_parts = tuple(keyed.values())
        self._graphs: dict[tuple, tuple] = {}    # (requests padded to a bucket, the keyed parts' launch keys)
        self._shape_graphs: dict[tuple, tuple] = {}
        self._shapes_seen: dict[tuple, int] = {}
        self.graph_replays = 0
        #: kernels of this package inside the graphs replayed so far (for launch accounting)
        self.graph_kernel_launches = 0

    # ------------------------------------------------------------------
    @staticmethod
    def _check_device(device: torch.device) -> None:
        if device.type != "cuda":
            raise RuntimeError(
                f"einf_b200 runs on a CUDA device only (asked for {device}); there is no CPU path"
            )
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; einf_b200 has no CPU path")

    def _guard(self):
        """Make the model's device the current one (nothing to do when it already is)."""
        device = self.runtime.device
        index = device.index if device.index is not None else 0
        if torch.cuda.current_device() == index:
            return _NO_GUARD
        return torch.cuda.device(device)

    def synchronize(self) -> None:
        with self._guard():
            ops.current_stream().synchronize()

    @classmethod
    def from_folder(cls, folder: str | Path, engine_config: EngineConfig) -> "ModelRunner":
        config = load_config(folder)
        expected, optional = expected_tensors(config.model_spec())
        tensors = load_tensors(folder, expected, device="cpu", optional=optional)
        return cls(config, tensors, engine_config)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, engine_config: EngineConfig) -> "ModelRunner":
        """Random weights drawn on the device (no folder is written)."""
        expected, _ = expected_tensors(config.model_spec())
        tensors = random_tensors(
            expected, seed, config.init_std, config.init_scale_std, torch.bfloat16, engine_config.device
        )
        return cls(config, tensors, engine_config)

    def group_specs(self) -> list[GroupSpec]:
        return [
            GroupSpec(pages, self.page_size, int(window or 0))
            for pages, window in zip(self.pages_per_group, self.model.cache_plan.group_windows)
        ]

    # ------------------------------------------------------------------
    def _forward(self, ctx) -> torch.Tensor:
        """The launches of one step: per-request state of the requests that start at position 0
        is cleared by a kernel that reads the step's own inputs (state is read before it is
        written; pages are not), then the model runs.  Everything is on the device, so the
        same launches can be captured in a graph."""
        for state in self._state_tensors:
            ops.zero_fresh_state(state, ctx.state_slots, ctx.q_start, ctx.positions)
        return self.model.forward(ctx, self.storage.views)

    def step(self, requests: Sequence, want: Optional[Sequence[Sequence[int]]] = None) -> StepOutput:
        """Run one batch.  ``requests`` is a ``BatchPlan`` or ``ScheduledRequest``-like objects;
        see :meth:`StepInputBuilder.build` for ``want``."""
        plan = as_plan(requests)
        summary = plan.summary()
        with self._guard(), torch.inference_mode():
            if self.graphs_enabled and want is None and self._graphable(summary):
                return self._graph_step(plan, len(summary))
            ctx, rows = self.inputs.build(plan, want)
            self.steps += 1
            if self.graphs_enabled and want is None:
                return self._shape_graph_step(ctx, rows)
            logits = self._forward(ctx)
        return StepOutput(logits, rows, ctx)

    def _launch_keys(self, ctx) -> tuple:
        page = self.page_size
        return tuple(part.launch_key(ctx, page) for part in self._keyed_parts)

    def advance_decode(self, output: StepOutput, sampled: torch.Tensor) -> None:
        """Move the inputs of a decode-only step on by one token, on the device: every request's
        sampled token becomes its input, its position and context grow by one and its cache slots
        follow its block table (which must already hold the page).  Padding requests stay."""
        ctx = output.context
        if len(ctx.slots) > ops.ADVANCE_MAX_GROUPS:
            raise StepError(f"advance_decode takes at most {ops.ADVANCE_MAX_GROUPS} cache groups")
        ops.advance_decode(ctx.token_ids, ctx.positions, ctx.context_lens, sampled, ctx.slots, ctx.block_tables,
                           self.page_size)

    def repeat_step(self, output: StepOutput) -> StepOutput:
        """Run the step of ``output`` again on what its device inputs hold now."""
        self.steps += 1
        with self._guard(), torch.inference_mode():
            if output.replay is not None:
                graph, static_logits, launches, count = output.replay
                graph.replay()
                self.graph_replays += 1
                self.graph_kernel_launches += launches
                return StepOutput(static_logits[:count], output.rows_of_request, output.context, output.replay)
            logits = self._forward(output.context)
        return StepOutput(logits, output.rows_of_request, output.context)

    #: graphs kept for steps that are not decode-only (each holds its own activations)
    MAX_SHAPE_GRAPHS = 8

    def _shape_graph_step(self, ctx, rows) -> StepOutput:
        """Steps with prompt portions: the layout of the step buffer and every launch depend
        only on the counts below, so a step whose counts were seen before (a server cutting
        prompts into portions of one size does this all the time) replays a graph, which spares
        the host some three hundred launches; a shape is captured the second time it comes."""
        from .. import ops

        # The longest cached prefix of a portion and the longest context are host values that
        # launches read too (the attention kernels pick their cluster sizes from them), so what
        # is made of them belongs to the key: a shape first seen with short contexts must not pin
        # the choice made for them.
        key = (ctx.num_tokens, ctx.num_requests, ctx.logit_rows.shape[0], ctx.q_tiles.shape[0],
               ctx.single_tokens.shape[0], ops.prefill_prefix_bucket(ctx.max_portion_start), self._launch_keys(ctx))
        entry = self._shape_graphs.get(key)
        if entry is not None:
            graph, static_logits, launches = entry
            graph.replay()
            self.graph_replays += 1
            self.graph_kernel_launches += launches
            return StepOutput(static_logits, rows, ctx)
        logits = self._forward(ctx)
        seen = self._shapes_seen.get(key, 0) + 1
        self._shapes_seen[key] = seen
        if seen >= 2 and len(self._shape_graphs) < self.MAX_SHAPE_GRAPHS:
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                static_logits = self._forward(ctx)
            self._shape_graphs[key] = (graph, static_logits, ops.launch_count - before)
        return StepOutput(logits, rows, ctx)

    # ------------------------------------------------------------------
    # CUDA graphs for decode-only steps.  The step buffer has the same layout for
    # every step of a bucket, so a graph captured once finds tokens, positions,
    # slots and block tables where each later step's single copy puts them.  The
    # batch is padded to the bucket with requests that write nothing.  (The
    # reference captures whole decode steps per bucket too, tied to FlashInfer's
    # plan: src/einf/executors/torch/decode_graph.py.)
    @staticmethod
    def _graphable(summary) -> bool:
        """Every request brings one token that is not its first and wants its logits."""
        return all(tokens == 1 and start > 0 and need_sample for (_, tokens, need_sample, _, _, start, _) in summary)

    def _bucket(self, count: int) -> int:
        bucket = 1
        while bucket < count:
            bucket *= 2
        return min(bucket, self.engine_config.max_requests)

    def _graph_step(self, plan, count: int) -> StepOutput:
        from .. import ops

        bucket = self._bucket(count)
        ctx, rows = self.inputs.build(plan, None, pad_requests_to=bucket)
        self.steps += 1
        # what the parts' launches make of the step's host-side figures (the decode attention cuts
        # the keys by the bucket of the longest context): a graph for each
        bucket = (bucket, self._launch_keys(ctx))
        entry = self._graphs.get(bucket)
        if entry is None:
            # This step runs eagerly (it also sizes every workspace); the capture that
            # follows records the same launches without running them.
            logits = self._forward(ctx)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                static_logits = self._forward(ctx)
            entry = (graph, static_logits, ops.launch_count - before)
            self._graphs[bucket] = entry
            return StepOutput(logits[:count], rows, ctx, entry + (count,))
        graph, static_logits, launches = entry
        graph.replay()
        self.graph_replays += 1
        self.graph_kernel_launches += launches
        return StepOutput(static_logits[:count], rows, ctx, entry + (count,))

    @staticmethod
    def check_status(status: int) -> None:
        if status == 0:
            return
        faults = []
        if status & ops.STATUS_BAD_TOKEN:
            faults.append("a token id outside the embedding table")
        if status & ops.STATUS_BAD_PAGE:
            faults.append("a block-table entry outside the page pool")
        if status & ops.STATUS_WAIT_EXPIRED:
            faults.append("a bounded wait inside a kernel expired")
        raise StepError("the step's kernels reported: " + "; ".join(faults or [f"status {status}"]))
