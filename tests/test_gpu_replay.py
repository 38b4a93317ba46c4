"""Replay on the GPU against the plain implementation: whole, tail one by one, portions, mixed.

32-bit runs are held to rtol 1e-4 / atol 2e-5 against the plain float32 model;
bfloat16 runs to 2e-2 / 2e-2 against the plain model with bfloat16 rounding at
the places where the engine stores activations.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_impl
import trace_tools
from conftest import ROOT, TINY, TINY_PAGE, random_tokens

pytestmark = pytest.mark.gpu

TOLERANCE = {"float32": dict(rtol=1e-4, atol=2e-5), "bfloat16": dict(rtol=2e-2, atol=2e-2)}
LENGTHS = {"A": [1, 2, 5, 9, 13, 37, 70], "B": [3, 7, 17, 30, 64, 101], "C": [4, 16, 33, 50, 97, 150]}


def make_requests(name, lengths, seed=0):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed * 100 + i) for i, n in enumerate(lengths)}


def expected_for(name, folder, requests, dtype):
    rounding = "bfloat16" if dtype == "bfloat16" else None
    return trace_tools.expected_rows(plain_impl, folder, requests, rounding=rounding)


def replayer_for(folder, dtype, max_tokens, page):
    from einf_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, block_len=page)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_modes(name, dtype, tiny_folders):
    requests = make_requests(name, LENGTHS[name])
    expected = expected_for(name, tiny_folders[name], requests, dtype)
    page = TINY_PAGE[name]
    longest = -(-max(LENGTHS[name]) // 64) * 64
    mixed_steps, most = trace_tools.mixed(requests, seed=7, page_round=page)
    traces = {
        "whole": (trace_tools.whole(requests), longest),
        "tail": (trace_tools.last_one_by_one(requests, tail=32), longest),
        "portions": (trace_tools.in_portions(requests), longest),
        "mixed": (mixed_steps, most),
    }
    for mode, (steps, max_tokens) in traces.items():
        replayer = replayer_for(tiny_folders[name], dtype, max_tokens, page)
        rows = trace_tools.run_steps(replayer, steps)
        try:
            trace_tools.compare(rows, expected, **TOLERANCE[dtype])
        except AssertionError as error:
            raise AssertionError(f"{name} {dtype} {mode}: {error}") from None
        assert replayer.manager.free_pages(0) == replayer.manager.group(0).num_pages
        if mode == "mixed":
            assert sum(len(t) for t in requests.values()) > most  # pages had to be used again


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_modes_agree_with_each_other_bit_for_bit_where_they_must(dtype, tiny_folders):
    """The same tokens through the same kernels: cutting a prompt differently changes only
    the order of nothing, because each row's arithmetic does not depend on the batch."""
    requests = make_requests("C", [97, 41], seed=4)
    page = TINY_PAGE["C"]
    a = trace_tools.run_steps(replayer_for(tiny_folders["C"], dtype, 128, page), trace_tools.whole(requests))
    b = trace_tools.run_steps(replayer_for(tiny_folders["C"], dtype, 128, page), trace_tools.in_portions(requests))
    tolerance = dict(rtol=1e-5, atol=2e-6) if dtype == "float32" else TOLERANCE[dtype]
    trace_tools.compare(b, a, **tolerance)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, tiny_folders):
    requests = make_requests("A", [330], seed=9)
    steps = trace_tools.last_one_by_one(requests, tail=322)   # 8 tokens of prompt, then 322 single tokens
    assert len(steps) == 323
    rows = trace_tools.run_steps(replayer_for(tiny_folders["A"], dtype, 384, 4), steps)
    trace_tools.compare(rows, expected_for("A", tiny_folders["A"], requests, dtype), **TOLERANCE[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_a_window(dtype, tiny_folders):
    requests = make_requests("C", [140], seed=10)
    steps = trace_tools.last_one_by_one(requests, tail=120)
    replayer = replayer_for(tiny_folders["C"], dtype, 192, 16)
    rows = trace_tools.run_steps(replayer, steps)
    trace_tools.compare(rows, expected_for("C", tiny_folders["C"], requests, dtype), **TOLERANCE[dtype])
    assert replayer.manager.high_water(1) <= 3   # the windowed group gave pages back on the way


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(name, tiny_folders):
    requests = make_requests(name, [1, 2, 3], seed=5)
    for dtype in ("float32", "bfloat16"):
        rows = trace_tools.run_steps(replayer_for(tiny_folders[name], dtype, 64, TINY_PAGE[name]),
                                     trace_tools.last_one_by_one(requests, tail=32))
        trace_tools.compare(rows, expected_for(name, tiny_folders[name], requests, dtype), **TOLERANCE[dtype])


def test_trace_run_program(tiny_folders, tmp_path):
    """The program itself: stdin in, files and `done` lines out, exit 0."""
    requests = make_requests("B", [19, 40], seed=6)
    steps, most = trace_tools.mixed(requests, seed=1, page_round=64)
    steps.append({"step": len(steps), "entries": [{"id": "z", "tokens": [1, 2], "want": []}], "end": ["z"]})
    text = "".join(json.dumps(s) + "\n" for s in steps)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        done = subprocess.run(
            [str(ROOT / "bin" / "trace_run"), "--model", str(tiny_folders["B"]), "--dtype", dtype,
             "--out", str(out), "--max-tokens", str(most)],
            input=text, capture_output=True, text=True, timeout=600,
        )
        assert done.returncode == 0, done.stderr[-2000:]
        assert done.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
        expected = expected_for("B", tiny_folders["B"], requests, dtype)
        position = {}
        for record in steps:
            path = out / f"{record['step']}.f32"
            wanted = sum(len(e["want"]) for e in record["entries"])
            assert path.exists() == (wanted > 0)
            if not wanted:
                continue
            logits = np.fromfile(path, dtype="<f4").reshape(wanted, 384)
            cursor = 0
            for entry in record["entries"]:
                start = position.get(entry["id"], 0)
                for place in entry["want"]:
                    np.testing.assert_allclose(logits[cursor], expected[(entry["id"], start + place)], **TOLERANCE[dtype])
                    cursor += 1
                position[entry["id"]] = start + len(entry["tokens"])


def test_run_qwen_program(tiny_folders, tmp_path):
    """``bin/run_qwen`` as a user runs it (``scripts/run_qwen.py`` of the reference): from a model
    folder and from a bare config.json with random weights, its ``key: value`` lines parsed and
    the tokens compared with the plain model; then ``--compare-reference`` on a bfloat16 run."""
    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    program = str(ROOT / "bin" / "run_qwen")

    def run(*options):
        done = subprocess.run([sys.executable, program, *options], capture_output=True, text=True, timeout=600)
        fields = dict(line.split(": ", 1) for line in done.stdout.splitlines() if ": " in line)
        return done, fields

    done, fields = run("--model-dir", str(tiny_folders["A"]), "--prompt-ids", "5,17,3,99,4", "--dtype", "float32",
                       "--max-new-len", "8", "--block-len", "4", "--max-prefill-chunk-len", "3", "--ignore-eos")
    assert done.returncode == 0, done.stderr[-2000:]
    assert json.loads(fields["generated_ids"]) == plain_impl.greedy_generate(config, tensors, [5, 17, 3, 99, 4], 8)
    assert json.loads(fields["prompt_ids"]) == [5, 17, 3, 99, 4] and fields["completion_reason"] == "length"
    assert "tokens_per_gen_s=" in done.stdout

    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(TINY["B"]))
    done, fields = run("--random-weights", "--config", str(config_path), "--seed", "1", "--prompt-ids", "7,8,9",
                       "--dtype", "float32", "--max-new-len", "5", "--block-len", "8", "--ignore-eos")
    assert done.returncode == 0, done.stderr[-2000:]
    config_b, tensors_b = plain_impl.read_folder(tiny_folders["B"])      # seed 1 is tiny B's own
    assert json.loads(fields["generated_ids"]) == plain_impl.greedy_generate(config_b, tensors_b, [7, 8, 9], 5)

    done, fields = run("--model-dir", str(tiny_folders["C"]), "--prompt-ids", "5,17,3,99,4,8,1", "--max-new-len", "6",
                       "--decode-lookahead", "4", "--ignore-eos", "--compare-reference")
    assert done.returncode == 0, done.stderr[-2000:]
    generated, reference = json.loads(fields["generated_ids"]), json.loads(fields["reference_generated_ids"])
    assert len(generated) == len(reference) == 6 and fields["tokens_equal"] == str(generated == reference)
    # no tokenizer in the folder and no --prompt-ids: refused with exit code 2
    done, _ = run("--model-dir", str(tiny_folders["A"]))
    assert done.returncode == 2 and "--prompt-ids" in done.stderr
