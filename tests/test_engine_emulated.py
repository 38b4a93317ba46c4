"""The engine's host logic on a machine without a GPU.

The kernels are replaced by their plain PyTorch statements
(``kernel_references.emulate_kernels``), so what is under test is everything
around them: batch packing, block tables and slots, the cache manager, page
reuse, the replay program's loop, scheduler + executor + sampler glue.  The
same traces run on the real kernels in the ``-m gpu`` tests.
"""
import io
import json

import numpy as np
import pytest
import torch

import plain_impl
import trace_tools
from conftest import TINY, TINY_PAGE, random_tokens
from kernel_references import emulate_kernels


def make_requests(name, lengths, seed=0):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed * 100 + i) for i, n in enumerate(lengths)}


@pytest.fixture()
def emulated():
    with emulate_kernels():
        yield


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_modes_match_the_plain_implementation(name, tiny_folders, emulated):
    from einf_b200.engine.replay import TraceReplayer

    requests = make_requests(name, [5, 9, 13, 37, 50])
    expected = trace_tools.expected_rows(plain_impl, tiny_folders[name], requests)
    page = TINY_PAGE[name]
    mixed_steps, most = trace_tools.mixed(requests, seed=3, page_round=page)
    traces = {
        "whole": (trace_tools.whole(requests), 64),
        "tail": (trace_tools.last_one_by_one(requests, tail=8), 64),
        "portions": (trace_tools.in_portions(requests), 64),
        "mixed": (mixed_steps, most),
    }
    for mode, (steps, max_tokens) in traces.items():
        replayer = TraceReplayer(tiny_folders[name], "float32", max_tokens, block_len=page, device="cpu")
        rows = trace_tools.run_steps(replayer, steps)
        trace_tools.compare(rows, expected, rtol=1e-4, atol=2e-5)
        assert replayer.manager.free_pages(0) == replayer.manager.group(0).num_pages, mode
        replayer.manager.check_invariants()


def test_mixed_trace_uses_pages_again(tiny_folders, emulated):
    from einf_b200.engine.replay import TraceReplayer

    requests = make_requests("A", [20, 30, 17, 25, 40, 12, 33], seed=2)
    steps, most = trace_tools.mixed(requests, seed=5, page_round=4)
    replayer = TraceReplayer(tiny_folders["A"], "float32", most, block_len=4, device="cpu")
    seen, reused = set(), False
    position = {}
    for record in steps:
        replayer.run_step({**record, "end": []})
        for entry in record["entries"]:
            table = replayer.manager.block_table(entry["id"], 0)
            first = position.get(entry["id"], 0) // 4
            position[entry["id"]] = position.get(entry["id"], 0) + len(entry["tokens"])
            for page in table[first:]:
                if (entry["id"], page) not in seen and any(p == page for _, p in seen):
                    reused = True
                seen.add((entry["id"], page))
        replayer.run_step({"step": -1, "entries": [], "end": record["end"]})
    assert reused
    assert sum(len(t) for t in requests.values()) > most  # the pool is smaller than the trace


def test_replay_refuses_a_trace_larger_than_its_pool(tiny_folders, emulated):
    from einf_b200.engine.replay import ReplayError, TraceReplayer

    replayer = TraceReplayer(tiny_folders["A"], "float32", 8, block_len=4, device="cpu")
    with pytest.raises(ReplayError, match="max-tokens"):
        replayer.run_step({"step": 0, "entries": [{"id": "a", "tokens": list(range(9)), "want": []}], "end": []})


def test_trace_run_program_loop(tiny_folders, emulated, tmp_path):
    from einf_b200.engine.replay import TraceReplayer, replay

    requests = make_requests("B", [11, 6])
    steps = trace_tools.in_portions(requests, sizes=(4, 2))
    steps.append({"step": len(steps), "entries": [{"id": "x", "tokens": [1, 2, 3], "want": []}], "end": ["x"]})
    lines = [json.dumps(s) + "\n" for s in steps]
    log = io.StringIO()
    replayer = TraceReplayer(tiny_folders["B"], "float32", 64, block_len=8, device="cpu")
    replay(lines, replayer, tmp_path / "out", log)
    assert log.getvalue().splitlines() == [f"done {s['step']}" for s in steps]
    assert not (tmp_path / "out" / f"{steps[-1]['step']}.f32").exists()  # nothing wanted, nothing written
    first = np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(-1, 384)
    expected = trace_tools.expected_rows(plain_impl, tiny_folders["B"], requests)
    np.testing.assert_allclose(first[0], expected[("r0", 0)], rtol=1e-4, atol=2e-5)
    assert first.shape[0] == len(steps[0]["entries"][0]["want"])


def test_step_refuses_bad_batches(tiny_folders, emulated):
    from types import SimpleNamespace

    from einf_b200.config import EngineConfig
    from einf_b200.engine import BatchError, ModelRunner

    runner = ModelRunner.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=8, max_batch_len=16,
                                        max_requests=4, device="cpu"))

    def request(tokens, start=0, table=(0, 1, 2, 3)):
        return SimpleNamespace(input_token_ids=tokens, start_position=start, block_tables=[list(table)],
                               state_slot=-1, need_sample=True)

    with pytest.raises(BatchError, match="at least one request"):
        runner.step([])
    with pytest.raises(BatchError, match="at least one token"):
        runner.step([request([])])
    with pytest.raises(BatchError, match="vocabulary"):
        runner.step([request([256])])
    with pytest.raises(BatchError, match="pages"):
        runner.step([request([1, 2, 3, 4, 5], table=(0,))])
    with pytest.raises(BatchError, match="outside the pool"):
        runner.step([request([1], table=(8,))])
    with pytest.raises(BatchError, match="built for"):
        runner.step([request(list(range(17)), table=(0, 1, 2, 3, 4))])
    with pytest.raises(BatchError, match="wanted place"):
        runner.step([request([1, 2])], want=[[2]])
    out = runner.step([request([1, 2, 3]), request([4], start=0, table=(5,))], want=[[0, 2], []])
    assert out.logits.shape == (2, 256) and out.rows_of_request == [(0, 2), (2, 0)]


def test_generation_through_the_entry_point(tiny_folders, emulated):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine
    from einf_b200.sampling import SamplingParams

    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    prompts = [random_tokens(256, n, 40 + n) for n in (5, 9, 13)]
    engine = Engine.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=24, max_batch_len=8,
                                        max_prefill_chunk_len=6, max_requests=4, device="cpu"),
        eos_token_ids=())
    outputs = engine.generate(prompts, 8)
    for prompt, generated in zip(prompts, outputs):
        assert generated == plain_impl.greedy_generate(config, tensors, prompt, 8)
    assert engine.scheduler.free_pages() == 24
    # temperature: same seed, same tokens, whatever else is in the batch
    params = SamplingParams(temperature=0.8, seed=11)
    alone = engine.generate([prompts[1]], 6, params)[0]
    together = engine.generate(prompts, 6, params)[1]
    assert alone == together
    with pytest.raises(ValueError, match="at most"):
        engine.submit(list(range(90)), 10)


def test_bfloat16_generation_on_the_plain_statements(tiny_folders, emulated):
    """The bfloat16 road of the host code (what is rounded where, partial sums handed from a product
    to its consumer) on the plain statements of the kernels: token for token like the plain model
    with bfloat16 rounding, except where its two best logits are closer than bfloat16 can tell."""
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    for name in ("A", "C"):
        config, tensors = plain_impl.read_folder(tiny_folders[name])
        vocab = TINY[name]["vocab_size"]
        prompts = [random_tokens(vocab, n, 90 + n) for n in (5, 9, 40)]
        engine = Engine.from_folder(
            tiny_folders[name], EngineConfig(dtype="bfloat16", block_len=TINY_PAGE[name], num_blocks=64,
                                             max_batch_len=64, max_prefill_chunk_len=48, max_requests=4, device="cpu"),
            eos_token_ids=())
        outputs = engine.generate(prompts, 6)
        for prompt, generated in zip(prompts, outputs):
            context = list(prompt)
            for token in generated:
                logits = plain_impl.forward(config, tensors, context, rounding="bfloat16")[-1]
                best = int(torch.argmax(logits))
                assert token == best or float(logits[best] - logits[token]) < 2e-2, (name, context, token)
                context.append(token)


def test_a_sequence_limit_narrows_the_block_tables(tiny_folders, emulated):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    engine = Engine.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=64, max_batch_len=16,
                                        max_prefill_chunk_len=16, max_requests=4, device="cpu", max_sequence_len=22),
        eos_token_ids=())
    assert engine.runner.max_sequence_len == 22 and engine.runner.table_width == 6
    with pytest.raises(ValueError, match="at most 22"):
        engine.submit(list(range(20)), 3)
    prompt = random_tokens(256, 15, 77)
    assert engine.generate([prompt], 7)[0] == plain_impl.greedy_generate(config, tensors, prompt, 7)
    wide = Engine.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=64, max_batch_len=16,
                                        max_prefill_chunk_len=16, max_requests=4, device="cpu"), eos_token_ids=())
    assert wide.runner.table_width == 64        # the pool's 256 tokens (the model allows 1,024)


def test_more_prompts_than_request_rows_all_finish(tiny_folders, emulated):
    """The token budget and the pages would admit every prompt at once; the step buffer has
    max_requests rows.  The scheduler stops admitting there and every request is served."""
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    prompts = [random_tokens(256, 2 + n % 3, 300 + n) for n in range(11)]
    engine = Engine.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=64, max_batch_len=64,
                                        max_prefill_chunk_len=16, max_requests=4, device="cpu"),
        eos_token_ids=())
    outputs = engine.generate(prompts, 3)
    for prompt, generated in zip(prompts, outputs):
        assert generated == plain_impl.greedy_generate(config, tensors, prompt, 3)
    assert engine.scheduler.free_pages() == 64


def test_generate_forgets_every_request_before_it_raises(tiny_folders, emulated):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    engine = Engine.from_folder(
        tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=16, max_batch_len=4,
                                        max_prefill_chunk_len=4, max_requests=4, device="cpu"),
        eos_token_ids=())
    # the executor raises on the first batch (which holds the first prompt alone: budget 4): that
    # request fails, the two others are served
    real, calls = engine.executor.execute, []

    def execute(batch):
        calls.append(batch)
        if len(calls) == 1:
            raise RuntimeError("made-up fault")
        return real(batch)

    engine.executor.execute = execute
    prompts = [[1, 2, 3, 4], [5, 6, 7], [8, 9]]
    with pytest.raises(RuntimeError, match="request-0 failed.*made-up fault"):
        engine.generate(prompts, 2)
    for index in range(3):
        assert not engine.scheduler.has_request(f"request-{index}")
    assert engine.scheduler.free_pages() == 16 and engine.scheduler.idle
    # the ids are free again
    engine.submit([1, 2], 1, request_id="request-1")
    engine.run_until_idle()
    assert engine.request("request-1").state == "finished"


# ---------------------------------------------------------------------------
# The command line (scripts/run_qwen.py of the reference)
def _cli_lines(capsys):
    out = capsys.readouterr().out
    return dict(line.split(": ", 1) for line in out.splitlines() if ": " in line), out


def test_command_line_defaults_follow_the_reference():
    """Option names and defaults of scripts/run_qwen.py:33-74 that this engine keeps."""
    from einf_b200.cli.run_qwen import parse_args

    args = parse_args([])
    assert args.prompt == "The capital of France is"
    assert (args.max_new_len, args.dtype, args.block_len, args.num_blocks) == (8, "bfloat16", 16, 256)
    assert (args.max_batch_len, args.max_prefill_chunk_len) == (128, 128)
    assert str(args.model_dir).endswith("Qwen2.5-0.5B")
    # added here, each off by default
    assert (args.policy, args.temperature, args.top_k, args.top_p, args.min_p) == ("fcfs", 0.0, None, 1.0, 0.0)
    assert not args.random_weights and not args.compare_reference and args.decode_lookahead == 1
    with pytest.raises(SystemExit):
        parse_args(["--dtype", "float16"])


def test_command_line_generates_what_the_plain_model_does(tiny_folders, emulated, capsys, tmp_path):
    from einf_b200.cli.run_qwen import main

    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    prompt = [5, 17, 3, 99, 4]
    code = main(["--model-dir", str(tiny_folders["A"]), "--prompt-ids", "5,17,3,99,4", "--dtype", "float32",
                 "--max-new-len", "6", "--max-prefill-chunk-len", "3", "--block-len", "4", "--ignore-eos",
                 "--device", "cpu", "--compare-reference"])
    fields, out = _cli_lines(capsys)
    assert code == 0, out
    expected = plain_impl.greedy_generate(config, tensors, prompt, 6)
    assert json.loads(fields["generated_ids"]) == expected and json.loads(fields["prompt_ids"]) == prompt
    assert fields["completion_reason"] == "length"
    assert json.loads(fields["reference_generated_ids"]) == expected and fields["tokens_equal"] == "True"
    assert "tokens_per_gen_s=" in out

    # random weights from a bare config.json: the folder it writes is the one write_random_model makes
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(conftest_tiny("B")))
    code = main(["--random-weights", "--config", str(config_path), "--seed", "1", "--prompt-ids", "7,8,9",
                 "--dtype", "float32", "--max-new-len", "4", "--block-len", "8", "--ignore-eos", "--device", "cpu"])
    fields, out = _cli_lines(capsys)
    assert code == 0, out
    config_b, tensors_b = plain_impl.read_folder(tiny_folders["B"])   # seed 1 is tiny B's own
    assert json.loads(fields["generated_ids"]) == plain_impl.greedy_generate(config_b, tensors_b, [7, 8, 9], 4)


def test_command_line_without_tokenizer_or_with_bad_options(tiny_folders, emulated, capsys):
    from einf_b200.cli.run_qwen import main

    assert main(["--model-dir", str(tiny_folders["A"]), "--device", "cpu"]) == 2
    assert "--prompt-ids" in capsys.readouterr().err
    assert main(["--model-dir", str(tiny_folders["A"]), "--prompt-ids", "1", "--temperature", "0.5",
                 "--compare-reference", "--device", "cpu"]) == 2
    # an end-of-sequence token ends generation unless --ignore-eos is given
    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    free = plain_impl.greedy_generate(config, tensors, [5, 17, 3], 8)
    eos = config["eos_token_id"]
    code = main(["--model-dir", str(tiny_folders["A"]), "--prompt-ids", "5,17,3", "--dtype", "float32",
                 "--block-len", "4", "--device", "cpu"])
    fields, out = _cli_lines(capsys)
    assert code == 0
    generated = json.loads(fields["generated_ids"])
    if eos in free:
        assert generated == free[: free.index(eos) + 1] and fields["completion_reason"] == "eos"
    else:
        assert generated == free and fields["completion_reason"] == "length"


def conftest_tiny(name):
    return dict(TINY[name])


def test_decode_lookahead_generates_the_same_tokens(tiny_folders, emulated):
    """Several decode steps per report (inputs moved on by advance_decode): the same tokens as
    with one, greedy and sampled, also when an end-of-sequence token comes on the way."""
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine
    from einf_b200.sampling import SamplingParams

    prompts = [random_tokens(256, n, 60 + n) for n in (5, 9, 13)]
    outputs = {}
    # 1: every step reports; 4: plans of four steps, each step reported as it ends while the later
    # ones run; (4, False): plans of four steps, one report per plan
    for lookahead, every_step in ((1, True), (4, True), (4, False)):
        engine = Engine.from_folder(
            tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=40, max_batch_len=8,
                                            max_prefill_chunk_len=6, max_requests=4, device="cpu",
                                            decode_lookahead=lookahead, report_every_step=every_step),
            eos_token_ids=())
        greedy = engine.generate(prompts, 11)
        sampled = engine.generate(prompts, 9, SamplingParams(temperature=0.9, seed=5))
        assert engine.scheduler.free_pages() == 40
        outputs[lookahead, every_step] = (greedy, sampled, engine.scheduler.stats.steps)
        assert (engine.executor.ahead_batches > 0) == (lookahead > 1)
    assert outputs[1, True] == outputs[4, True] == outputs[4, False]
    outputs = {1: outputs[1, True]}
    # with a token of the greedy output as end of sequence, both stop at it
    eos = outputs[1][0][0][4]
    stopped = []
    for lookahead, every_step in ((1, True), (4, True), (4, False)):
        engine = Engine.from_folder(
            tiny_folders["A"], EngineConfig(dtype="float32", block_len=4, num_blocks=40, max_batch_len=8,
                                            max_prefill_chunk_len=6, max_requests=4, device="cpu",
                                            decode_lookahead=lookahead, report_every_step=every_step),
            eos_token_ids=(eos,))
        stopped.append(engine.generate(prompts, 11))
        assert engine.scheduler.free_pages() == 40
        engine.scheduler.check_invariants()
    assert stopped[0] == stopped[1] == stopped[2] and stopped[0][0][-1] == eos and len(stopped[0][0]) <= 5


def test_runner_refuses_the_cpu(tiny_folders):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import ModelRunner

    with pytest.raises(RuntimeError, match="no CPU path"):
        ModelRunner.from_folder(tiny_folders["A"], EngineConfig(device="cpu"))
