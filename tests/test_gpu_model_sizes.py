"""The engine at the layer sizes of Qwen2.5-0.5B (two layers of them) against the plain model.

The tiny configurations exercise every option; this one exercises the kernels at the sizes
they are tuned for: hidden 896, 14 query heads over 2 key/value heads of size 64, intermediate
4,864, a vocabulary of 151,936 that is no power of two, page size 16.
"""
import pytest

import plain_impl
import trace_tools
from conftest import random_tokens

pytestmark = pytest.mark.gpu

@pytest.fixture(scope="module")
def folder_128(sized_folders):
    """Qwen2.5-1.5B layer sizes: head size 128, the other compiled variant of the attention kernels."""
    return sized_folders("1.5b")


def test_head_size_128_matches_the_plain_model(folder_128):
    """bfloat16 at the 1.5B layer sizes: a 1,200-token prompt in large portions (whose few row tiles
    make the prefill kernel split their keys over a cluster) beside other requests' portions and
    single tokens, then the tails token by token (the tcgen05 decode kernel and the split-K products
    at head size 128); every position of the short request and the last 64 of the two long ones
    against the plain model."""
    import numpy as np

    from einf_b200.engine.replay import TraceReplayer

    requests = {"r0": random_tokens(3001, 1200, 6), "r1": random_tokens(3001, 40, 7), "r2": random_tokens(3001, 300, 8)}
    r0, r1, r2 = requests["r0"], requests["r1"], requests["r2"]
    steps = [
        {"entries": [{"id": "r0", "tokens": r0[:600], "want": []}], "end": []},
        {"entries": [{"id": "r0", "tokens": r0[600:1112], "want": []},
                     {"id": "r1", "tokens": r1[:30], "want": list(range(30))}], "end": []},
        {"entries": [{"id": "r0", "tokens": r0[1112:1194], "want": list(range(1136 - 1112, 1194 - 1112))},
                     {"id": "r1", "tokens": r1[30:31], "want": [0]},
                     {"id": "r2", "tokens": r2[:294], "want": list(range(236, 294))}], "end": []},
    ]
    fed = {"r0": 1194, "r1": 31, "r2": 294}
    while any(fed[name] < len(requests[name]) for name in requests):
        entries, ended = [], []
        for name, tokens in requests.items():
            if fed[name] < len(tokens):
                entries.append({"id": name, "tokens": [tokens[fed[name]]], "want": [0]})
                fed[name] += 1
                if fed[name] == len(tokens):
                    ended.append(name)
        steps.append({"entries": entries, "end": ended})
    for index, record in enumerate(steps):
        record["step"] = index
    rows = trace_tools.run_steps(TraceReplayer(folder_128, "bfloat16", 1216 + 64 + 320), steps)
    config, tensors = plain_impl.read_folder(folder_128)
    checked = 0
    for name, tokens in requests.items():
        exact = plain_impl.forward(config, tensors, tokens).numpy()
        rounded = plain_impl.forward(config, tensors, tokens, rounding="bfloat16").numpy()
        for i in range(len(tokens)):
            if (name, i) not in rows:
                continue
            got, truth = rows[(name, i)], exact[i]
            scale = float(np.sqrt(np.mean(truth ** 2)))
            rounding_error = float(np.sqrt(np.mean((rounded[i] - truth) ** 2))) / scale
            engine_error = float(np.sqrt(np.mean((got - truth) ** 2))) / scale
            assert np.isfinite(got).all() and engine_error <= 2.0 * rounding_error + 1e-3, (name, i, engine_error, rounding_error)
            checked += 1
    assert checked == 64 + 40 + 64


@pytest.fixture(scope="module")
def folder(sized_folders):
    return sized_folders("0.5b")


@pytest.mark.parametrize("dtype, decode_shapes", [("float32", None), ("bfloat16", None), ("bfloat16", ((4, 2),)),
                                                  ("bfloat16", ((16, 1),)), ("bfloat16", ((3, 8),))])
def test_half_billion_sizes_match_the_plain_model(folder, dtype, decode_shapes, monkeypatch):
    """``decode_shapes``: the only (cluster size, clusters per token) the decode attention may
    choose from, instead of all: short contexts never get several clusters per token or a cluster
    above eight by themselves, and this way the whole step (its graphs, the scratch space the
    clusters meet in, layer after layer and step after step) runs with them."""
    from einf_b200 import ops
    from einf_b200.engine.replay import TraceReplayer

    if decode_shapes is not None:
        monkeypatch.setattr(ops, "DECODE_SHAPES", decode_shapes)

    requests = {"r0": random_tokens(151936, 150, 1), "r1": random_tokens(151936, 70, 2), "r2": random_tokens(151936, 9, 3)}
    rounding = "bfloat16" if dtype == "bfloat16" else None
    config, tensors = plain_impl.read_folder(folder)
    # the output matrix is large: compare the last 24 positions of each request
    steps, most = trace_tools.mixed(requests, seed=11, page_round=64)
    keep = {name: set(range(max(0, len(tokens) - 24), len(tokens))) for name, tokens in requests.items()}
    position = {}
    for record in steps:
        for entry in record["entries"]:
            start = position.get(entry["id"], 0)
            entry["want"] = [i for i in range(len(entry["tokens"])) if start + i in keep[entry["id"]]]
            position[entry["id"]] = start + len(entry["tokens"])
    rows = trace_tools.run_steps(TraceReplayer(folder, dtype, most), steps)
    expected = {}
    for name, tokens in requests.items():
        logits = plain_impl.forward(config, tensors, tokens, rounding=rounding)
        for i in keep[name]:
            expected[(name, i)] = logits[i].numpy()
    if dtype == "float32":
        trace_tools.compare(rows, expected, rtol=1e-4, atol=2e-5)
        return
    # bfloat16: with 152k logits per row, the largest of millions of rounding differences is no
    # measure.  The yardstick is the rounding itself: the plain model with bfloat16 rounding at
    # the engine's storage points misses the plain 32-bit model by some amount per row; the
    # engine may miss it by at most twice that (a skipped key or a wrong page misses it by
    # tens of times that).
    import numpy as np
    for name, tokens in requests.items():
        exact = plain_impl.forward(config, tensors, tokens).numpy()
        for i in keep[name]:
            got, rounded, truth = rows[(name, i)], expected[(name, i)], exact[i]
            scale = float(np.sqrt(np.mean(truth ** 2)))
            rounding_error = float(np.sqrt(np.mean((rounded - truth) ** 2))) / scale
            engine_error = float(np.sqrt(np.mean((got - truth) ** 2))) / scale
            assert np.isfinite(got).all() and engine_error <= 2.0 * rounding_error + 1e-3, (
                name, i, engine_error, rounding_error)


def test_generation_repeats_itself_whatever_the_host_does(folder):
    """At these sizes every step is a chain of kernels that start before the one before them has
    ended (programmatic dependent launch) and most steps are graph replays; a kernel that read
    something too early would show as tokens that change from run to run.  The same prompts
    three times, with one decode step per report and with four, long and short prompts cut into
    portions beside decoding requests: always the same tokens."""
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    prompts = [random_tokens(151936, n, 400 + n) for n in (700, 33, 1100, 129, 5, 260, 64, 1, 17, 300)]
    seen = []
    for lookahead in (1, 4):
        engine = Engine.from_folder(folder, EngineConfig(
            dtype="bfloat16", block_len=16, num_blocks=1024, max_batch_len=512, max_prefill_chunk_len=256,
            max_requests=16, policy="decode_first", decode_lookahead=lookahead), eos_token_ids=())
        for _ in range(3 if lookahead == 1 else 2):
            seen.append(engine.generate(prompts, 48))
        assert engine.runner.graph_replays > 40 and engine.scheduler.free_pages() == 1024
    assert all(outputs == seen[0] for outputs in seen[1:])


@pytest.mark.parametrize("lookahead", [1, 4])
def test_decoding_across_a_bucket_of_context_lengths(folder_128, lookahead):
    """The decode attention cuts a request's keys by the bucket of the longest context (a power of
    two from 4,096 on).  A request that decodes from 4,090 to 4,104 tokens crosses one; the cut
    stays the same there, so the one graph goes on being replayed.  Token for token like the plain
    model on the engine's own choices, except where the plain model's two best logits are closer
    than bfloat16 tells apart."""
    import torch

    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    config, tensors = plain_impl.read_folder(folder_128)
    prompt = random_tokens(3001, 4090, 77)
    engine = Engine.from_folder(folder_128, EngineConfig(
        dtype="bfloat16", block_len=16, num_blocks=300, max_batch_len=4096, max_prefill_chunk_len=4096,
        max_requests=4, decode_lookahead=lookahead), eos_token_ids=())
    generated = engine.generate([prompt], 14)[0]
    assert len(engine.runner._graphs) == 1 and engine.runner.graph_replays >= 10
    logits = plain_impl.forward(config, tensors, prompt + generated[:-1], rounding="bfloat16")
    for i, token in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        best = torch.topk(row, 2)
        if token != int(best.indices[0]):
            assert float(row[best.indices[0]] - row[token]) < 2e-2, (i, token)


@pytest.mark.parametrize("lookahead", [1, 4])
def test_decode_graphs_are_kept_apart_by_how_the_keys_are_cut(folder, lookahead):
    """One request decodes from 8,188 to 8,204 tokens: behind 8,192 the decode attention takes
    several clusters per token, which a graph captured before must not pin.  With graphs (one for
    each way of cutting the keys) the same tokens as without any."""
    from einf_b200 import ops
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    before = ops.decode_plan(1, 14, 2, 64, 16, 8192)
    after = ops.decode_plan(1, 14, 2, 64, 16, 8193)
    assert before != after and after[2] > 1
    prompt = random_tokens(151936, 8188, 78)
    outputs = []
    for graphs in (True, False):
        engine = Engine.from_folder(folder, EngineConfig(
            dtype="bfloat16", block_len=16, num_blocks=600, max_batch_len=4096, max_prefill_chunk_len=4096,
            max_requests=4, decode_lookahead=lookahead, use_cuda_graphs=graphs), eos_token_ids=())
        outputs.append(engine.generate([prompt], 16)[0])
        if graphs:
            keys = set(engine.runner._graphs)
            assert {(1, (before,)), (1, (after,))} <= keys and engine.runner.graph_replays >= 10
    assert outputs[0] == outputs[1]
