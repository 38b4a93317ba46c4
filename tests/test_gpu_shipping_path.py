"""The path that ships, against the plain model, at the layer sizes the tensor-core kernels serve.

Generation through ``Engine.generate`` runs decode steps as CUDA-graph replays per batch-size
bucket (padded with requests that write nothing), prompt portions as graphs per shape, every
kernel chained to the one before it by programmatic dependent launch, and, with a lookahead,
several decode steps per report with the inputs moved on by a kernel.  Replay runs eagerly, so
these paths need tests of their own: here their tokens are checked against the plain model at
the layer sizes of Qwen2.5-0.5B (head size 64), 1.5B (head size 128) and 7B (seven query heads
per key/value head, the widest products, an output matrix of its own), including steps of 33
to 64 single tokens, whose products go to the library and whose consumers read dense rows.
"""
import numpy as np
import pytest
import torch

import plain_impl
import trace_tools
from conftest import SIZED, random_tokens

pytestmark = pytest.mark.gpu


def check_generated(config, tensors, prompt, generated, dtype):
    """Every generated token is the plain model's choice given the tokens before it (one whole
    forward over prompt + generated, teacher forced).  32-bit: the largest logit, or one within 1e-4
    of it.  bfloat16: the largest logit of the plain model with bfloat16 rounding at the engine's
    storage points, or one that is closer to it than four times what that rounding moves a logit
    (rows' root mean square): a skipped key or a wrong page moves logits by tens of times that."""
    context = list(prompt) + list(generated[:-1])
    rows = list(range(len(prompt) - 1, len(context)))
    exact = plain_impl.forward(config, tensors, context, rows=rows)
    if dtype == "float32":
        for row, token in zip(exact, generated):
            best = int(torch.argmax(row))
            assert token == best or float(row[best] - row[token]) < 1e-4, (len(prompt), token, best)
        return
    rounded = plain_impl.forward(config, tensors, context, rows=rows, rounding="bfloat16")
    for row, truth, token in zip(rounded, exact, generated):
        best = int(torch.argmax(row))
        yardstick = float(torch.sqrt(torch.mean((row - truth) ** 2)))
        assert token == best or float(row[best] - row[token]) <= 4.0 * yardstick, (
            len(prompt), token, best, float(row[best] - row[token]), yardstick)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", ["0.5b", "1.5b", "7b"])
def test_generation_with_graphs_and_lookahead_matches_the_plain_model(size, dtype, sized_folders):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine, ModelRunner

    folder = sized_folders(size)
    config, tensors = plain_impl.read_folder(folder)
    vocab = SIZED[size]["vocab_size"]
    lengths = (5, 33, 129, 260, 700) if size != "7b" else (5, 33, 129, 300)
    prompts = [random_tokens(vocab, n, 500 + n) for n in lengths]
    runner = ModelRunner.from_folder(folder, EngineConfig(
        dtype=dtype, block_len=16, num_blocks=256, max_batch_len=512, max_prefill_chunk_len=256,
        max_requests=8, policy="decode_first"))
    assert runner.graphs_enabled
    outputs = {}
    for lookahead in (1, 4):
        engine = Engine(runner, eos_token_ids=(), decode_lookahead=lookahead)
        replays = runner.graph_replays
        outputs[lookahead] = engine.generate(prompts, 21)
        assert runner.graph_replays - replays >= 15
        assert (engine.executor.ahead_batches > 0) == (lookahead > 1)
        assert engine.scheduler.free_pages() == 256
        # a second time: every graph exists from the first step on (prompt portions included)
        assert engine.generate(prompts, 21) == outputs[lookahead]
    assert outputs[1] == outputs[4]
    for prompt, generated in zip(prompts, outputs[1]):
        assert len(generated) == 21
        check_generated(config, tensors, prompt, generated, dtype)


@pytest.mark.parametrize("size, dtype", [("0.5b", "bfloat16"), ("0.5b", "float32"), ("1.5b", "bfloat16"), ("7b", "bfloat16")])
def test_steps_of_more_than_32_single_tokens_match_the_plain_model(size, dtype, sized_folders):
    """44 live requests: once they all decode, a step is 44 single tokens in the 64-request graph
    bucket with 20 padding requests; the bfloat16 products run in the library, rotary, activation
    and norms read dense rows, attention serves 64 rows."""
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    folder = sized_folders(size)
    config, tensors = plain_impl.read_folder(folder)
    vocab = SIZED[size]["vocab_size"]
    prompts = [random_tokens(vocab, 2 + (7 * n) % 23, 900 + n) for n in range(44)]
    for lookahead in (1, 3):
        engine = Engine.from_folder(folder, EngineConfig(
            dtype=dtype, block_len=16, num_blocks=44 * 3 + 8, max_batch_len=256, max_prefill_chunk_len=64,
            max_requests=64, policy="fcfs", decode_lookahead=lookahead), eos_token_ids=())
        outputs = engine.generate(prompts, 9)
        assert any(key[0] == 64 for key in engine.runner._graphs) and engine.runner.graph_replays >= 5   # (requests, launch keys)
        for prompt, generated in zip(prompts, outputs):
            check_generated(config, tensors, prompt, generated, dtype)
        assert engine.scheduler.free_pages() == 44 * 3 + 8


@pytest.mark.parametrize("size, dtype", [("1.5b", "bfloat16"), ("1.5b", "float32"), ("7b", "bfloat16")])
def test_replay_of_a_step_with_forty_single_tokens(size, dtype, sized_folders):
    """The same through the replay program's class (eager steps, logits compared, not tokens): forty
    requests fed in portions, ten requests a step, then their last three tokens as steps of forty
    single tokens."""
    from einf_b200.engine.replay import TraceReplayer

    folder = sized_folders(size)
    vocab = SIZED[size]["vocab_size"]
    requests = {f"r{n:02d}": random_tokens(vocab, 6 + (5 * n) % 17, 1200 + n) for n in range(40)}
    names = list(requests)
    steps = []
    for first in range(0, 40, 10):
        entries = []
        for name in names[first:first + 10]:
            head = len(requests[name]) - 3
            entries.append({"id": name, "tokens": requests[name][:head], "want": list(range(head))})
        steps.append({"step": len(steps), "entries": entries, "end": []})
    for back in (3, 2, 1):
        entries = [{"id": name, "tokens": [requests[name][-back]], "want": [0]} for name in names]
        steps.append({"step": len(steps), "entries": entries, "end": names if back == 1 else []})
    rows = trace_tools.run_steps(TraceReplayer(folder, dtype, 40 * 64, max_requests=48), steps)
    if dtype == "float32":
        trace_tools.compare(rows, trace_tools.expected_rows(plain_impl, folder, requests), rtol=1e-4, atol=2e-5)
        return
    compare_with_the_rounding_yardstick(rows, folder, requests)


def compare_with_the_rounding_yardstick(rows, folder, requests):
    """bfloat16: the plain model with bfloat16 rounding at the engine's storage points misses the
    plain 32-bit model by some amount per row; the engine may miss it by at most twice that."""
    config, tensors = plain_impl.read_folder(folder)
    checked = 0
    for name, tokens in requests.items():
        places = sorted(i for (n, i) in rows if n == name)
        if not places:
            continue
        exact = plain_impl.forward(config, tensors, tokens, rows=places).numpy()
        rounded = plain_impl.forward(config, tensors, tokens, rows=places, rounding="bfloat16").numpy()
        for k, i in enumerate(places):
            got, truth = rows[(name, i)], exact[k]
            scale = float(np.sqrt(np.mean(truth ** 2)))
            rounding_error = float(np.sqrt(np.mean((rounded[k] - truth) ** 2))) / scale
            engine_error = float(np.sqrt(np.mean((got - truth) ** 2))) / scale
            assert np.isfinite(got).all() and engine_error <= 2.0 * rounding_error + 1e-3, (
                name, i, engine_error, rounding_error)
            checked += 1
    assert checked == len(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_seven_billion_layer_sizes_mixed_trace(dtype, sized_folders):
    """Hidden 3,584, 28 query heads over 4 key/value heads of 128, intermediate 18,944, untied
    output matrix: portions of some requests beside single tokens of others, pages used again."""
    from einf_b200.engine.replay import TraceReplayer

    folder = sized_folders("7b")
    vocab = SIZED["7b"]["vocab_size"]
    requests = {"r0": random_tokens(vocab, 150, 21), "r1": random_tokens(vocab, 70, 22), "r2": random_tokens(vocab, 9, 23),
                "r3": random_tokens(vocab, 45, 24), "r4": random_tokens(vocab, 110, 25)}
    steps, most = trace_tools.mixed(requests, seed=13, page_round=64)
    assert sum(-(-len(t) // 64) * 64 for t in requests.values()) > most     # pages are used again
    rows = trace_tools.run_steps(TraceReplayer(folder, dtype, most), steps)
    if dtype == "float32":
        trace_tools.compare(rows, trace_tools.expected_rows(plain_impl, folder, requests), rtol=1e-4, atol=2e-5)
    else:
        compare_with_the_rounding_yardstick(rows, folder, requests)
