"""From a batch plan to the device tensors a step needs.

The plan (``BatchPlan`` of the control plane, or one made by hand) lists, per
request, its next tokens, where they start, its block tables and state slot.
:class:`StepInputBuilder` packs them into one int32 staging buffer in pinned
host memory, copies it to the device in one transfer and hands out views.  For
a given number of tokens, requests and wanted rows the layout is always the
same, so a captured CUDA graph finds its inputs where it left them.

The reference packs seven int64 tensors with one copy each
(``src/einf/executors/torch/input.py:109-319``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..parts.base import StepContext

#: query rows per tile of the prefill attention kernel (einf_b200.ops.Q_TILE)
Q_TILE = 64


class BatchError(ValueError):
    """A plan the step function refuses."""


@dataclass(frozen=True)
class StepLayout:
    """Offsets (in int32 elements) of each field inside the step buffer."""

    tokens: int
    requests: int
    wanted: int
    groups: int
    table_width: int
    tiles: int = 0

    def fields(self) -> dict[str, tuple[int, int]]:
        offset = 0
        out: dict[str, tuple[int, int]] = {}

        def add(name: str, count: int) -> None:
            nonlocal offset
            out[name] = (offset, count)
            offset += (count + 3) // 4 * 4  # keep every field 16-byte aligned

        add("status", 1)
        add("token_ids", self.tokens)
        add("positions", self.tokens)
        add("seq_of_token", self.tokens)
        add("q_start", self.requests + 1)
        add("context_lens", self.requests)
        add("state_slots", self.requests)
        add("logit_rows", self.wanted)
        add("q_tiles", 4 * self.tiles)
        for g in range(self.groups):
            add(f"slots{g}", self.tokens)
        for g in range(self.groups):
            add(f"block_table{g}", self.requests * self.table_width)
        out["_total"] = (offset, 0)
        return out


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
        self.page_size = page_size
        self.pages_per_group = tuple(pages_per_group)
        self.group_windows = tuple(group_windows)
        self.vocab_size = vocab_size
        self.table_width = table_width
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        groups = len(self.pages_per_group)
        capacity = StepLayout(max_tokens, max_requests, max_tokens, groups, table_width, max_tokens).fields()["_total"][0]
        self._capacity = capacity
        pin = self.device.type == "cuda"
        self._staging = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._staging_np = [t.numpy() for t in self._staging]
        self._events = [None, None]
        self._turn = 0
        self._device_buffer = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        self.h2d_bytes = 0

    # ------------------------------------------------------------------
    def build(
        self,
        requests: Sequence,
        want: Optional[Sequence[Sequence[int]]] = None,
        pad_requests_to: int = 0,
    ) -> tuple[StepContext, list[tuple[int, int]]]:
        """Pack ``requests`` (objects with ``input_token_ids``, ``start_position``,
        ``block_tables``, ``state_slot``, ``need_sample``) for one step.

        ``want[i]`` lists the places among request i's tokens whose logits are
        wanted; by default the last token of every request that samples.
        Returns the context and, per request, ``(first_row, count)`` into the logits.

        ``pad_requests_to`` appends harmless one-token requests (no cache write, output
        unused) up to that count, so that decode steps of similar size share a CUDA graph.
        """
        if not requests:
            raise BatchError("a step needs at least one request")
        page = self.page_size
        groups = len(self.pages_per_group)
        q_lens = [len(r.input_token_ids) for r in requests]
        if min(q_lens) <= 0:
            raise BatchError("every request of a step brings at least one token")
        real_requests = len(requests)
        pad = max(0, pad_requests_to - real_requests)
        num_requests = real_requests + pad
        num_tokens = sum(q_lens) + pad
        if num_tokens > self.max_tokens:
            raise BatchError(f"the step has {num_tokens} tokens, the engine was built for {self.max_tokens}")
        if num_requests > self.max_requests:
            raise BatchError(f"the step has {num_requests} requests, the engine was built for {self.max_requests}")
        if want is None:
            want = [[q - 1] if getattr(r, "need_sample", False) else [] for r, q in zip(requests, q_lens)]
        elif len(want) != real_requests:
            raise BatchError("want must have one entry per request")
        num_wanted = sum(len(w) for w in want) + pad

        num_tiles = sum(-(-q // Q_TILE) for q in q_lens) + pad
        layout = StepLayout(num_tokens, num_requests, num_wanted, groups, self.table_width, num_tiles)
        fields = layout.fields()
        total = fields["_total"][0]
        turn = self._turn
        self._turn ^= 1
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        host = self._staging_np[turn]

        def view(name: str) -> np.ndarray:
            offset, count = fields[name]
            return host[offset:offset + count]

        view("status")[:] = 0
        token_ids, positions, seq_of_token = view("token_ids"), view("positions"), view("seq_of_token")
        q_start, context_lens, state_slots = view("q_start"), view("context_lens"), view("state_slots")
        logit_rows = view("logit_rows")
        q_tiles = view("q_tiles").reshape(num_tiles, 4)
        tile_cursor = 0
        slots = [view(f"slots{g}") for g in range(groups)]
        tables = [view(f"block_table{g}").reshape(num_requests, self.table_width) for g in range(groups)]
        for table in tables:
            table[:] = -1

        rows_of_request: list[tuple[int, int]] = []
        cursor = 0
        row_cursor = 0
        q_start[0] = 0
        starts = []
        for index, (request, q_len) in enumerate(zip(requests, q_lens)):
            start = int(request.start_position)
            if start < 0:
                raise BatchError(f"request {index}: negative start position")
            starts.append(start)
            end = start + q_len
            tokens = np.asarray(request.input_token_ids, dtype=np.int64)
            if tokens.min() < 0 or tokens.max() >= self.vocab_size:
                raise BatchError(
                    f"request {index}: token id outside the vocabulary of {self.vocab_size}"
                )
            token_ids[cursor:cursor + q_len] = tokens
            pos = np.arange(start, end, dtype=np.int32)
            positions[cursor:cursor + q_len] = pos
            seq_of_token[cursor:cursor + q_len] = index
            q_start[index + 1] = cursor + q_len
            context_lens[index] = end
            state_slots[index] = getattr(request, "state_slot", -1)
            for first in range(0, q_len, Q_TILE):
                q_tiles[tile_cursor] = (index, cursor + first, min(Q_TILE, q_len - first), start + first)
                tile_cursor += 1
            if len(request.block_tables) != groups:
                raise BatchError(f"request {index}: {len(request.block_tables)} block tables for {groups} cache groups")
            for g in range(groups):
                table = np.asarray(request.block_tables[g], dtype=np.int32)
                needed_pages = (end + page - 1) // page
                if table.shape[0] < needed_pages:
                    raise BatchError(
                        f"request {index}: block table of group {g} has {table.shape[0]} pages, "
                        f"{needed_pages} are needed for {end} tokens"
                    )
                if table.shape[0] > self.table_width:
                    raise BatchError(
                        f"request {index}: {table.shape[0]} pages exceed the table width {self.table_width}"
                    )
                if table.max(initial=-1) >= self.pages_per_group[g]:
                    raise BatchError(f"request {index}: page id outside the pool of group {g}")
                tables[g][index, : table.shape[0]] = table
                page_of_token = table[pos // page]
                window = self.group_windows[g]
                first_key = 0 if not window else max(0, start - window + 1)
                if page_of_token.min() < 0 or table[first_key // page: needed_pages].min() < 0:
                    raise BatchError(f"request {index}: a page it needs in group {g} is missing from its block table")
                slots[g][cursor:cursor + q_len] = page_of_token * page + pos % page
            wanted = list(want[index])
            for place in wanted:
                if not 0 <= place < q_len:
                    raise BatchError(f"request {index}: wanted place {place} outside its {q_len} tokens")
            logit_rows[row_cursor:row_cursor + len(wanted)] = np.asarray(wanted, dtype=np.int32) + cursor
            rows_of_request.append((row_cursor, len(wanted)))
            row_cursor += len(wanted)
            cursor += q_len
        for extra in range(pad):
            index = real_requests + extra
            token_ids[cursor] = 0
            positions[cursor] = 0
            seq_of_token[cursor] = index
            q_start[index + 1] = cursor + 1
            context_lens[index] = 1
            state_slots[index] = -1
            q_tiles[tile_cursor] = (index, cursor, 1, 0)
            tile_cursor += 1
            for g in range(groups):
                tables[g][index, :] = 0      # any valid page: what is read there is never used
                slots[g][cursor] = -1        # and nothing is written
            logit_rows[row_cursor] = cursor
            row_cursor += 1
            cursor += 1
            q_lens.append(1)
            starts.append(0)

        device_view = self._device_buffer[:total]
        device_view.copy_(self._staging[turn][:total], non_blocking=True)
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
            self._events[turn] = event
        self.h2d_bytes += total * 4

        def dev(name: str) -> torch.Tensor:
            offset, count = fields[name]
            return self._device_buffer[offset:offset + count]

        ctx = StepContext(
            num_tokens=num_tokens,
            num_requests=num_requests,
            token_ids=dev("token_ids"),
            positions=dev("positions"),
            seq_of_token=dev("seq_of_token"),
            q_start=dev("q_start"),
            context_lens=dev("context_lens"),
            block_tables=[dev(f"block_table{g}").view(num_requests, self.table_width) for g in range(groups)],
            slots=[dev(f"slots{g}") for g in range(groups)],
            state_slots=dev("state_slots"),
            logit_rows=dev("logit_rows"),
            q_tiles=dev("q_tiles").view(num_tiles, 4),
            status=dev("status"),
            q_lens=tuple(q_lens),
            start_positions=tuple(starts),
            max_q_len=max(q_lens),
            max_context_len=max(s + q for s, q in zip(starts, q_lens)),
            decode_only=all(q == 1 for q in q_lens),
        )
        return ctx, rows_of_request
