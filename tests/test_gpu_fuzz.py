"""Seeded random configurations and engine options against the plain model.

The fixed tiny configurations pin every option once; here sizes and options are drawn at random
(odd widths, every head size from 16 to 256, any number of heads and groups, prime vocabularies,
windows, page sizes, token budgets, policies, lookahead, pools so small that requests are
preempted), which is how a page-count fault in the admission test of windowed groups was found.
"""
import random
import tempfile
from pathlib import Path

import pytest

import plain_impl
import trace_tools
from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", range(8))
def test_random_configuration_in_all_replay_modes(case):
    from einf_b200.config import config_from_dict
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.weights import write_random_model

    rng = random.Random(1000 + case)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 192, 256])
    kv_heads = rng.choice([1, 2, 3, 4, 5])
    heads = kv_heads * rng.choice([1, 2, 3, 4, 7, 8])
    vocab = rng.choice([97, 257, 1000, 1031, 4099])
    window = rng.choice([None, None, 7, 19, 40])
    config = dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=vocab, hidden_size=rng.choice([40, 64, 72, 100, 136, 200, 264, 330, 75, 101]),
        intermediate_size=rng.choice([48, 100, 125, 160, 256, 333]), num_hidden_layers=rng.choice([1, 2, 3, 5]),
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
        rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]), hidden_act="silu", rope_theta=rng.choice([1e4, 5e5, 1e6]),
        max_position_embeddings=4096, tie_word_embeddings=rng.random() < 0.5, bos_token_id=0, eos_token_id=1,
        use_sliding_window=window is not None, sliding_window=window, max_window_layers=rng.choice([0, 1]) if window else None,
    )
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(Path(tmp) / "model", config_from_dict(config), seed=case)
        requests = {f"r{i}": random_tokens(vocab, rng.randrange(1, 90), case * 10 + i) for i in range(5)}
        mixed, most = trace_tools.mixed(requests, seed=case, page_round=64)
        traces = {"whole": (trace_tools.whole(requests), 128), "tail": (trace_tools.last_one_by_one(requests, 32), 128),
                  "portions": (trace_tools.in_portions(requests), 128), "mixed": (mixed, most)}
        for dtype, tolerance in (("float32", dict(rtol=1e-4, atol=2e-5)), ("bfloat16", dict(rtol=2e-2, atol=2e-2))):
            expected = trace_tools.expected_rows(plain_impl, folder, requests, rounding="bfloat16" if dtype == "bfloat16" else None)
            for mode, (steps, max_tokens) in traces.items():
                rows = trace_tools.run_steps(TraceReplayer(folder, dtype, max_tokens), steps)
                try:
                    trace_tools.compare(rows, expected, **tolerance)
                except AssertionError as error:
                    raise AssertionError(f"{config} {dtype} {mode}: {error}") from None


def test_random_engine_options_generate_the_plain_model_tokens(tiny_folders):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    plain = {name: plain_impl.read_folder(tiny_folders[name]) for name in TINY}
    preempted = 0
    for case in range(40):
        rng = random.Random(2000 + case)
        name = rng.choice("ABC")
        vocab = TINY[name]["vocab_size"]
        page = rng.choice([4, 8, 16, 32])
        prompts = [random_tokens(vocab, rng.randrange(1, 40), case * 20 + i) for i in range(rng.randrange(1, 9))]
        new = rng.randrange(1, 14)
        need = sum(-(-(len(p) + new) // page) for p in prompts)
        longest = max(-(-(len(p) + new) // page) for p in prompts)
        pages = rng.choice([need + 4, max(longest + 1, need // 2), max(longest, need // 3)])
        options = dict(dtype="float32", block_len=page, num_blocks=pages, max_batch_len=rng.choice([4, 8, 16, 64]),
                       max_prefill_chunk_len=rng.choice([2, 3, 5, 16, 64]), max_requests=rng.choice([2, 3, 4, 8]),
                       policy=rng.choice(["fcfs", "decode_first"]), decode_lookahead=rng.choice([1, 1, 2, 4, 5]),
                       report_every_step=rng.random() < 0.6, use_cuda_graphs=rng.random() < 0.7)
        engine = Engine.from_folder(tiny_folders[name], EngineConfig(**options), eos_token_ids=())
        want = [plain_impl.greedy_generate(*plain[name], prompt, new) for prompt in prompts]
        assert engine.generate(prompts, new) == want, (case, name, options)
        assert engine.scheduler.free_pages() == pages and engine.scheduler.idle, (case, options)
        engine.scheduler.check_invariants()
        assert engine.generate(prompts[::-1], new) == want[::-1], (case, name, options)
        preempted += engine.scheduler.stats.preemptions
    assert preempted > 0      # some of the pools were small enough
