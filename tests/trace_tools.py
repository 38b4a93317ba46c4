"""Builders of replay traces and the comparison with the plain implementation.

A trace is a list of steps in the format ``bin/trace_run`` reads.  Every
builder asks for the logits at every position it feeds, so each mode checks
every position of every request.
"""
from __future__ import annotations

import random
from typing import Sequence

import numpy as np
import torch


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, all its tokens in one step."""
    steps = []
    for name, tokens in requests.items():
        steps.append({"step": len(steps), "entries": [
            {"id": name, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [name]})
    return steps


def last_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for name, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [
            {"id": name, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        for position in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [
                {"id": name, "tokens": [tokens[position]], "want": [0]}], "end": []})
        steps[-1]["end"] = [name]
    return steps


def cut(length: int, sizes: Sequence[int]) -> list[int]:
    """Cut ``length`` into portions that cycle through ``sizes``."""
    out, i = [], 0
    while length > 0:
        size = min(sizes[i % len(sizes)], length)
        out.append(size)
        length -= size
        i += 1
    return out


def in_portions(requests: dict[str, list[int]], sizes: Sequence[int] = (7, 2, 5, 3, 2, 11, 4)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for index, (name, tokens) in enumerate(requests.items()):
        rotated = list(sizes[index % len(sizes):]) + list(sizes[:index % len(sizes)])
        start = 0
        for size in cut(len(tokens), rotated):
            steps.append({"step": len(steps), "entries": [
                {"id": name, "tokens": tokens[start:start + size], "want": list(range(size))}], "end": []})
            start += size
        steps[-1]["end"] = [name]
    return steps


def mixed(requests: dict[str, list[int]], seed: int = 0, max_live: int = 4,
          page_round: int = 64) -> tuple[list[dict], int]:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of
    others, requests pausing for a step now and then, new ones starting as others end.
    Returns the steps and the most tokens (each request rounded up to ``page_round``)
    that live requests ever hold: the pool size at which pages must be used again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}            # name -> tokens fed so far
    steps: list[dict] = []
    most = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            name, _ = waiting.pop(0)
            live[name] = 0
        entries, ended = [], []
        for name in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                 # this request sits the step out
            tokens = requests[name]
            fed = live[name]
            left = len(tokens) - fed
            # the tail of a request is fed token by token, like decoding
            if left <= 6 or rng.random() < 0.35:
                size = 1
            else:
                size = min(left, rng.choice([2, 3, 5, 8, 13, 21]))
            entries.append({"id": name, "tokens": tokens[fed:fed + size], "want": list(range(size))})
            live[name] = fed + size
            if live[name] == len(tokens):
                ended.append(name)
        if not entries:
            continue
        held = sum(-(-count // page_round) * page_round for count in live.values())
        most = max(most, held)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for name in ended:
            del live[name]
    return steps, most


def run_steps(replayer, steps: list[dict]) -> dict[tuple[str, int], np.ndarray]:
    """Feed the steps to a ``TraceReplayer``; logits row of every (request, position)."""
    position: dict[str, int] = {}
    rows: dict[tuple[str, int], np.ndarray] = {}
    for record in steps:
        logits = replayer.run_step(record)
        cursor = 0
        for entry in record["entries"]:
            start = position.get(entry["id"], 0)
            for place in entry["want"]:
                rows[(entry["id"], start + place)] = logits[cursor]
                cursor += 1
            position[entry["id"]] = start + len(entry["tokens"])
        for name in record["end"]:
            position.pop(name, None)
    return rows


def expected_rows(plain_impl, folder, requests: dict[str, list[int]], rounding=None, schedule=None):
    config, tensors = plain_impl.read_folder(folder)
    out: dict[tuple[str, int], np.ndarray] = {}
    for name, tokens in requests.items():
        logits = plain_impl.forward(config, tensors, tokens, schedule=schedule, rounding=rounding).numpy()
        for position in range(len(tokens)):
            out[(name, position)] = logits[position]
    return out


def compare(rows, expected, rtol: float, atol: float) -> None:
    """Every row within tolerance; on failure, name the first wrong token and its place."""
    assert set(rows) == set(expected), "the trace did not cover every position"
    worst = None
    for key in sorted(expected):
        got, want = rows[key], expected[key]
        excess = np.abs(got - want) - (atol + rtol * np.abs(want))
        if not np.isfinite(got).all() or excess.max() > 0:
            worst = (key, float(np.abs(got - want).max()))
            break
    if worst is not None:
        (name, position), error = worst
        raise AssertionError(
            f"first wrong token: request {name!r} position {position}, max |difference| {error:.3e} "
            f"(rtol {rtol}, atol {atol})"
        )


def max_error(rows, expected) -> float:
    return max(float(np.abs(rows[k] - expected[k]).max()) for k in expected)
