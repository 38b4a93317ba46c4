"""Trace replay: feed given token ids through the model step by step, write logits.

It samples nothing and owns no model code: it drives the same
:class:`ModelRunner` step function, cache manager and kernels that generation
uses.  Each line of the trace is one step::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch; a request's position is where its
earlier steps left it; ``end`` names requests whose pages are given back after
the step.  For a step that wants logits, ``<out>/<step>.f32`` holds them as
little-endian float32 ``[wanted, vocab]`` in the order of the entries and of
``want``.  The reference has no such program (its ``scripts/README.md:3`` only
reserves the place).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import IO, Iterable

import numpy as np
import torch

from ..cache.control import CacheManager, ScheduledRequest
from ..config.engine import EngineConfig
from .runner import ModelRunner


class ReplayError(RuntimeError):
    pass


class TraceReplayer:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, block_len: int = 16,
                 device: str = "cuda:0", max_requests: int = 8) -> None:
        """``max_requests``: most requests one step may hold (rows of the step buffer)."""
        pages = -(-max_tokens // block_len)
        engine_config = EngineConfig(
            dtype=dtype,
            block_len=block_len,
            num_blocks=pages,
            max_batch_len=max(max_tokens, 8),
            max_prefill_chunk_len=max(max_tokens, 8),
            max_requests=max_requests,
            device=device,
            use_cuda_graphs=False,
        )
        self.runner = ModelRunner.from_folder(model_dir, engine_config)
        self.manager = CacheManager(self.runner.group_specs(), self.runner.num_state_slots)
        self.lengths: dict[str, int] = {}

    def run_step(self, record: dict) -> np.ndarray | None:
        entries = record.get("entries", [])
        requests, want = [], []
        for entry in entries:
            request_id = str(entry["id"])
            tokens = [int(t) for t in entry["tokens"]]
            start = self.lengths.get(request_id, 0)
            end = start + len(tokens)
            if not self.manager.reserve(request_id, start, end):
                raise ReplayError(
                    f"step {record.get('step')}: no pages left for request {request_id!r} "
                    f"({end} tokens); --max-tokens is too small for this trace"
                )
            requests.append(
                ScheduledRequest(
                    request_id,
                    tokens,
                    start,
                    [self.manager.block_table(request_id, g) for g in range(self.manager.num_groups)],
                    False,
                    False,
                    self.manager.state_slot(request_id),
                )
            )
            want.append([int(w) for w in entry.get("want", [])])
        logits = None
        if requests:
            output = self.runner.step(requests, want)
            status = output.context.status
            if output.logits.shape[0] > 0:
                logits = output.logits.cpu().numpy().astype("<f4", copy=False)
            self.runner.check_status(int(status.cpu()[0]))
            for entry in entries:
                request_id = str(entry["id"])
                self.lengths[request_id] = self.lengths.get(request_id, 0) + len(entry["tokens"])
                self.manager.advance(request_id, self.lengths[request_id])
        for request_id in record.get("end", []):
            request_id = str(request_id)
            self.manager.release(request_id)
            self.lengths.pop(request_id, None)
        return logits


def replay(lines: Iterable[str], replayer: TraceReplayer, out_dir: Path, log: IO[str]) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = replayer.run_step(record)
        if logits is not None:
            logits.tofile(out_dir / f"{step}.f32")
        print(f"done {step}", file=log, flush=True)


def main(argv: list[str] | None = None) -> int:
    import argparse

    parser = argparse.ArgumentParser(
        prog="trace_run", description="Replay token ids through the engine step by step and write logits"
    )
    parser.add_argument("--model", required=True, type=Path, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, type=Path, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", required=True, type=int,
                        help="most tokens live requests hold at any time; the cache pool is made for this many")
    parser.add_argument("--block-len", type=int, default=16, help="tokens per cache page")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--max-requests", type=int, default=8, help="most requests in one step")
    args = parser.parse_args(argv)
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, args.block_len, args.device,
                             args.max_requests)
    # readline, not iteration: a step must be answered before the next one is read
    replay(iter(sys.stdin.readline, ""), replayer, args.out, sys.stdout)
    return 0
