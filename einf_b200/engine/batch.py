"""From a batch plan to the device tensors a step needs.

The plan (``BatchPlan`` of the control plane, or one made by hand) lists, per
request, its next tokens, where they start, its block tables and state slot.
:class:`StepInputBuilder` has the C++ packer (``csrc/control/pack.cpp``) write
them into one int32 staging buffer in pinned host memory, copies it to the
device in one transfer and hands out views.  For a given number of tokens,
requests and wanted rows the layout is always the same, so a captured CUDA graph
finds its inputs where it left them.

The reference packs seven int64 tensors with one copy each
(``src/einf/executors/torch/input.py:109-319``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from ..cache.control import BatchPlan, PackConfig, ScheduledRequest, pack_plan, step_buffer_size
from ..parts.base import StepContext

#: query rows per tile of the prefill attention kernel (einf_b200.ops.Q_TILE)
Q_TILE = 128


class BatchError(ValueError):
    """A plan the step function refuses."""


def as_plan(requests) -> BatchPlan:
    """A :class:`BatchPlan` from a plan or from request-like objects (``input_token_ids``,
    ``start_position``, ``block_tables``, optional ``state_slot``, ``need_sample``,
    ``request_id``): hand-made batches take the same road as the scheduler's."""
    if isinstance(requests, BatchPlan):
        return requests
    converted = []
    for index, r in enumerate(requests):
        if isinstance(r, ScheduledRequest):
            converted.append(r)
            continue
        converted.append(
            ScheduledRequest(
                str(getattr(r, "request_id", index)),
                [int(t) for t in r.input_token_ids],
                int(r.start_position),
                [[int(p) for p in table] for table in r.block_tables],
                bool(getattr(r, "need_sample", False)),
                False,
                int(getattr(r, "state_slot", -1)),
                int(getattr(r, "sample_index", 0)),
                getattr(r, "sampling_params", None),
            )
        )
    return BatchPlan(0, converted)


class StepInputBuilder:
    def __init__(
        self,
        device: torch.device,
        page_size: int,
        pages_per_group: Sequence[int],
        group_windows: Sequence[Optional[int]],
        vocab_size: int,
        table_width: int,
        max_tokens: int,
        max_requests: int,
    ) -> None:
        self.device = torch.device(device)
        self.table_width = table_width
        self.groups = len(pages_per_group)
        self.config = PackConfig(
            page_size, list(pages_per_group), [int(w or 0) for w in group_windows], vocab_size, table_width,
            max_tokens, max_requests, Q_TILE,
        )
        capacity = step_buffer_size(
            max_tokens, max_requests, max_tokens, self.groups, table_width, max_tokens, max_requests
        )
        pin = self.device.type == "cuda"
        self._staging = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._staging_np = [t.numpy() for t in self._staging]
        self._events = [None, None]
        self._turn = 0
        self._device_buffer = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        self._views: dict[tuple, dict] = {}
        self.h2d_bytes = 0

    def build(
        self,
        requests,
        want: Optional[Sequence[Sequence[int]]] = None,
        pad_requests_to: int = 0,
    ) -> tuple[StepContext, list[tuple[int, int]]]:
        """Pack one step.  ``requests`` is a ``BatchPlan`` or a sequence of request-like objects.

        ``want[i]`` lists the places among request i's tokens whose logits are wanted; by
        default the last token of every request that samples.  Returns the context and, per
        request, ``(first_row, count)`` into the logits.  ``pad_requests_to`` appends harmless
        one-token requests (no cache write, output unused) up to that count, so that decode
        steps of similar size share a CUDA graph.
        """
        plan = as_plan(requests)
        turn = self._turn
        self._turn ^= 1
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        try:
            packed = pack_plan(
                plan, None if want is None else [list(w) for w in want], self._staging_np[turn], self.config,
                pad_requests_to,
            )
        except ValueError as error:
            raise BatchError(str(error)) from None
        total = packed.total
        self._device_buffer[:total].copy_(self._staging[turn][:total], non_blocking=True)
        if self.device.type == "cuda":
            if self._events[turn] is None:
                self._events[turn] = torch.cuda.Event()
            self._events[turn].record(ops.current_stream())
        self.h2d_bytes += total * 4
        num_requests, num_tiles = packed.num_requests, packed.num_tiles
        # The views are made once per layout (offset and length of every field).
        fields = packed.fields
        key = tuple(v for span in fields.values() for v in span)
        views = self._views.get(key)
        if views is None:
            buffer = self._device_buffer

            def dev(name: str) -> torch.Tensor:
                offset, count = fields[name]
                return buffer[offset:offset + count]

            views = dict(
                token_ids=dev("token_ids"),
                positions=dev("positions"),
                seq_of_token=dev("seq_of_token"),
                q_start=dev("q_start"),
                context_lens=dev("context_lens"),
                block_tables=[dev(f"block_table{g}").view(num_requests, self.table_width) for g in range(self.groups)],
                slots=[dev(f"slots{g}") for g in range(self.groups)],
                state_slots=dev("state_slots"),
                logit_rows=dev("logit_rows"),
                q_tiles=dev("q_tiles").view(num_tiles, 4),
                single_tokens=dev("single_tokens"),
                status=dev("status"),
            )
            if len(self._views) >= 256:
                self._views.clear()
            self._views[key] = views
        ctx = StepContext(
            num_tokens=packed.num_tokens,
            num_requests=num_requests,
            q_lens=tuple(packed.q_lens),
            start_positions=tuple(packed.starts),
            max_q_len=packed.max_q_len,
            max_context_len=packed.max_context_len,
            max_portion_start=packed.max_portion_start,
            decode_only=packed.decode_only,
            **views,
        )
        return ctx, list(packed.rows_of_request)
