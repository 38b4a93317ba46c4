"""Token selection on the device.

A batch whose rows are all greedy takes the argmax kernel (ties to the lowest
index, as ``logits.argmax`` in ``src/einf/executors/torch/sampler.py:31-32``);
otherwise one kernel filters and draws every row from its own parameters and a
uniform number keyed by ``(seed, sample_index)``, so a request's tokens do not
depend on the batch it shares (``sampler.py:93-94`` seeds a generator per row
for the same reason).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import ops


class Sampler:
    def __init__(self, device: torch.device | str, max_rows: int) -> None:
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.tokens = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        pin = self.device.type == "cuda"
        # [temperature, top_p, min_p] as float32, [top_k] as int32, [seed, sample_index] as int64.
        # The copies to the device are asynchronous and a caller may sample several steps before it
        # waits for the device, so the pinned staging is a ring: a slot is written again only after
        # the copy that read it last has run (its event).
        self._ring = 8
        self._turn = 0
        self._events = [None] * self._ring
        self._host_f = torch.zeros((self._ring, 3, max_rows), dtype=torch.float32, pin_memory=pin)
        self._host_i = torch.zeros((self._ring, 1, max_rows), dtype=torch.int32, pin_memory=pin)
        self._host_l = torch.zeros((self._ring, 2, max_rows), dtype=torch.int64, pin_memory=pin)
        self._dev_f = torch.zeros((3, max_rows), dtype=torch.float32, device=self.device)
        self._dev_i = torch.zeros((1, max_rows), dtype=torch.int32, device=self.device)
        self._dev_l = torch.zeros((2, max_rows), dtype=torch.int64, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence, sample_indices: Sequence[int]) -> torch.Tensor:
        """One token per row of ``logits`` (float32 ``[rows, vocab]``); returns an
        int32 device tensor of ``rows`` tokens (a view of an internal buffer)."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(sample_indices):
            raise ValueError("one set of sampling parameters per logits row is needed")
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the sampler's {self.max_rows}")
        if rows == 0:
            return self.tokens[:0]
        if all(p.temperature == 0 for p in params):
            ops.argmax(logits, self.tokens)
            return self.tokens[:rows]
        turn = self._turn
        self._turn = (turn + 1) % self._ring
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        f, i, l = self._host_f[turn].numpy(), self._host_i[turn].numpy(), self._host_l[turn].numpy()
        for r, (p, index) in enumerate(zip(params, sample_indices)):
            f[0, r] = p.temperature
            f[1, r] = p.top_p
            f[2, r] = p.min_p
            i[0, r] = p.top_k or 0
            l[0, r] = np.int64(p.seed)
            l[1, r] = index
        self._dev_f.copy_(self._host_f[turn], non_blocking=True)
        self._dev_i.copy_(self._host_i[turn], non_blocking=True)
        self._dev_l.copy_(self._host_l[turn], non_blocking=True)
        if self.device.type == "cuda":
            if self._events[turn] is None:
                self._events[turn] = torch.cuda.Event()
            self._events[turn].record(ops.current_stream())
        ops.sample(
            logits, self.tokens, self._dev_f[0], self._dev_i[0], self._dev_f[1], self._dev_f[2],
            self._dev_l[0], self._dev_l[1],
        )
        return self.tokens[:rows]
