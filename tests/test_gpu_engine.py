"""Generation through the entry point, parts alone, and parts defined outside the framework."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_impl
import trace_tools
from conftest import TINY, TINY_PAGE, random_tokens

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype, page, pages=64, **kwargs):
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine

    options = dict(dtype=dtype, block_len=page, num_blocks=pages, max_batch_len=16, max_prefill_chunk_len=6, max_requests=4)
    options.update(kwargs)
    return Engine.from_folder(folder, EngineConfig(**options), eos_token_ids=())


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32(name, tiny_folders):
    config, tensors = plain_impl.read_folder(tiny_folders[name])
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(vocab, n, 70 + n) for n in (5, 9, 13, 30)]
    engine = engine_for(tiny_folders[name], "float32", TINY_PAGE[name])
    outputs = engine.generate(prompts, 8)
    for prompt, generated in zip(prompts, outputs):
        assert generated == plain_impl.greedy_generate(config, tensors, prompt, 8)
    assert engine.scheduler.free_pages() == 64


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_bfloat16(name, tiny_folders):
    """Token for token like the plain model, except where its two best logits are closer
    than bfloat16 can tell apart: then either may be taken, and the comparison restarts
    from the engine's choice."""
    config, tensors = plain_impl.read_folder(tiny_folders[name])
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(vocab, n, 90 + n) for n in (5, 9, 13, 30)]
    engine = engine_for(tiny_folders[name], "bfloat16", TINY_PAGE[name])
    outputs = engine.generate(prompts, 8)
    for prompt, generated in zip(prompts, outputs):
        context = list(prompt)
        for token in generated:
            logits = plain_impl.forward(config, tensors, context, rounding="bfloat16")[-1]
            best = torch.topk(logits, 2)
            if token != int(best.indices[0]):
                assert float(logits[best.indices[0]] - logits[token]) < 2e-2, (context, token)
            context.append(token)


def test_cuda_graph_steps_equal_eager_steps(tiny_folders):
    prompts = [random_tokens(331, n, 30 + n) for n in (5, 9, 13)]
    for dtype in ("float32", "bfloat16"):
        with_graphs = engine_for(tiny_folders["C"], dtype, 16, use_cuda_graphs=True)
        without = engine_for(tiny_folders["C"], dtype, 16, use_cuda_graphs=False)
        assert with_graphs.runner.graphs_enabled and not without.runner.graphs_enabled
        assert with_graphs.generate(prompts, 20) == without.generate(prompts, 20)
        assert with_graphs.runner.graph_replays >= 15 and without.runner.graph_replays == 0
        # a second batch of another size uses another bucket
        assert with_graphs.generate(prompts[:1], 5) == without.generate(prompts[:1], 5)
        assert len(with_graphs.runner._graphs) >= 2


def test_prompt_portions_of_one_shape_replay_a_graph(tiny_folders):
    """Long prompts cut into portions of one size: the steps repeat a shape, the second such
    step captures a graph and the later ones replay it, with the same tokens as eager steps."""
    prompts = [random_tokens(331, n, 300 + n) for n in (150, 97, 64)]
    for dtype in ("float32", "bfloat16"):
        options = dict(pages=96, max_batch_len=24, max_prefill_chunk_len=16)
        with_graphs = engine_for(tiny_folders["C"], dtype, 16, use_cuda_graphs=True, **options)
        without = engine_for(tiny_folders["C"], dtype, 16, use_cuda_graphs=False, **options)
        assert with_graphs.generate(prompts, 6) == without.generate(prompts, 6)
        runner = with_graphs.runner
        assert len(runner._shape_graphs) >= 1 and len(runner._shape_graphs) <= runner.MAX_SHAPE_GRAPHS
        assert runner.graph_replays > without.runner.graph_replays == 0
        # and again, now that the graphs exist from the first step on
        assert with_graphs.generate(prompts, 6) == without.generate(prompts, 6)
        assert with_graphs.scheduler.free_pages() == 96


@pytest.mark.parametrize("name", ["A", "C"])
def test_decode_lookahead_equals_single_steps(name, tiny_folders):
    """Several decode steps per host round trip (graph replays with the inputs moved on by a kernel):
    the same tokens as one step at a time, greedy and sampled, with and without CUDA graphs, and
    with an end-of-sequence token on the way."""
    from einf_b200.sampling import SamplingParams

    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(vocab, n, 200 + n) for n in (5, 9, 13, 21)]
    for dtype in ("float32", "bfloat16"):
        single = engine_for(tiny_folders[name], dtype, TINY_PAGE[name], pages=96)
        greedy = single.generate(prompts, 19)
        sampled = single.generate(prompts, 12, SamplingParams(temperature=0.8, seed=9))
        for graphs, every_step in ((True, True), (False, True), (True, False)):
            ahead = engine_for(tiny_folders[name], dtype, TINY_PAGE[name], pages=96, decode_lookahead=4,
                               use_cuda_graphs=graphs, report_every_step=every_step)
            assert ahead.generate(prompts, 19) == greedy
            assert ahead.generate(prompts, 12, SamplingParams(temperature=0.8, seed=9)) == sampled
            assert ahead.executor.ahead_batches > 0
            assert ahead.scheduler.free_pages() == 96
        eos = greedy[1][6]
        stop_single = engine_for(tiny_folders[name], dtype, TINY_PAGE[name], pages=96)
        stop_single.executor.eos_token_ids = frozenset([eos])
        stop_ahead = engine_for(tiny_folders[name], dtype, TINY_PAGE[name], pages=96, decode_lookahead=5)
        stop_ahead.executor.eos_token_ids = frozenset([eos])
        assert stop_ahead.generate(prompts, 19) == stop_single.generate(prompts, 19)
        assert stop_ahead.scheduler.free_pages() == 96


def test_temperature_stream_does_not_depend_on_the_batch(tiny_folders):
    from einf_b200.sampling import SamplingParams

    prompts = [random_tokens(384, n, 50 + n) for n in (3, 7, 17, 30)]
    engine = engine_for(tiny_folders["B"], "float32", 8)
    params = SamplingParams(temperature=0.8, seed=21)
    together = engine.generate(prompts, 6, params)
    for prompt, want in zip(prompts, together):
        assert engine.generate([prompt], 6, params)[0] == want
    other = engine.generate(prompts, 6, SamplingParams(temperature=0.8, seed=22))
    assert other != together
    # the first sampled token of each request is the plain inverse CDF of the plain logits
    config, tensors = plain_impl.read_folder(tiny_folders["B"])
    for prompt, generated in zip(prompts, together):
        logits = plain_impl.forward(config, tensors, prompt)[-1]
        probabilities = torch.softmax(logits.double() / 0.8, -1)
        cumulative = probabilities.cumsum(0)
        u = plain_impl.uniform_from_key(21, 0)
        token = generated[0]
        assert float(cumulative[token] - probabilities[token]) - 1e-4 <= u <= float(cumulative[token]) + 1e-4


def test_sampling_filters_through_the_entry_point(tiny_folders):
    """Top-k, top-p and min-p through ``Engine.generate``: every generated token is one that the
    filters keep on the plain model's logits for the sequence so far, the stream of a request does
    not depend on the batch, and another seed gives another stream."""
    import kernel_references as ref
    from einf_b200.sampling import SamplingParams

    prompts = [random_tokens(384, n, 60 + n) for n in (4, 9, 21)]
    engine = engine_for(tiny_folders["B"], "float32", 8)
    cases = [dict(temperature=0.9, top_k=5, seed=3), dict(temperature=1.1, top_p=0.7, seed=4),
             dict(temperature=0.8, top_k=12, top_p=0.9, min_p=0.05, seed=5)]
    config, tensors = plain_impl.read_folder(tiny_folders["B"])
    for case in cases:
        params = SamplingParams(**case)
        together = engine.generate(prompts, 8, params)
        assert engine.generate([prompts[1]], 8, params)[0] == together[1]
        assert engine.generate(prompts, 8, SamplingParams(**dict(case, seed=case["seed"] + 100))) != together
        for prompt, generated in zip(prompts, together):
            logits = plain_impl.forward(config, tensors, prompt + generated[:-1])[len(prompt) - 1:]
            for step, token in enumerate(generated):
                kept = ref.kept_weights(logits[step], params.temperature, params.top_k or 0, params.top_p, params.min_p)
                assert kept[token] > 0, (params, step, token)


def test_preemption_under_cache_pressure_keeps_the_tokens(tiny_folders):
    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    prompts = [random_tokens(256, n, 20 + n) for n in (9, 11, 10)]
    roomy = engine_for(tiny_folders["A"], "float32", 4, pages=64)
    want = roomy.generate(prompts, 12)
    tight = engine_for(tiny_folders["A"], "float32", 4, pages=13)   # 52 tokens for 3 x ~22
    got = tight.generate(prompts, 12)
    assert got == want
    assert tight.scheduler.stats.preemptions >= 1 and tight.scheduler.free_pages() == 13
    for prompt, generated in zip(prompts, got):
        assert generated == plain_impl.greedy_generate(config, tensors, prompt, 12)


def test_a_status_bit_fails_the_batch_frees_its_pages_and_the_engine_goes_on(tiny_folders):
    """The road from the device status word to the caller: a bit in it -> ``StepError`` in the
    executor -> ``LLMServer`` fails the batch -> every request of it is failed, its pages come back
    -> the next request is served.  The bit is made on the host side here (a torch operation on
    the status word after the step's own kernels); nothing is made to fault or to wait."""
    from einf_b200 import ops
    from einf_b200.config import EngineConfig
    from einf_b200.engine import Engine, ModelRunner

    class RunnerWithAFault(ModelRunner):
        fault_at_step = None

        def step(self, requests, want=None):
            output = super().step(requests, want)
            if self.fault_at_step is not None and self.steps >= self.fault_at_step:
                with torch.inference_mode():
                    output.context.status.bitwise_or_(ops.STATUS_WAIT_EXPIRED)
            return output

    config, tensors = plain_impl.read_folder(tiny_folders["A"])
    # eager and graph steps; single-step plans and plans of four steps reported step by step (the
    # fault then shows in the report of the plan's first step and fails the whole plan)
    for graphs, lookahead in ((False, 1), (True, 1), (True, 4)):
        runner = RunnerWithAFault.from_folder(tiny_folders["A"], EngineConfig(
            dtype="float32", block_len=4, num_blocks=32, max_batch_len=16, max_prefill_chunk_len=6, max_requests=4,
            use_cuda_graphs=graphs, decode_lookahead=lookahead))
        engine = Engine(runner, eos_token_ids=())
        prompts = [random_tokens(256, n, 700 + n) for n in (5, 9)]
        ids = [engine.submit(p, 8) for p in prompts]
        runner.fault_at_step = 5          # a decode step of both requests (the prompts take two steps)
        engine.run_until_idle()
        for request_id in ids:
            view = engine.request(request_id)
            assert view.state == "failed" and "StepError" in view.error and "bounded wait" in view.error
            assert 0 < len(view.generated_token_ids) < 8
        assert engine.scheduler.free_pages() == 32 and engine.scheduler.idle
        engine.scheduler.check_invariants()
        assert engine.scheduler.stats.failures == 2
        # the engine lives: the same prompts now run to their end, on the pages the failed ones held
        runner.fault_at_step = None
        outputs = engine.generate(prompts, 8)
        for prompt, generated in zip(prompts, outputs):
            assert generated == plain_impl.greedy_generate(config, tensors, prompt, 8)
        assert engine.scheduler.free_pages() == 32


# --- parts alone -------------------------------------------------------------
def _runtime(dtype):
    from einf_b200.parts import Runtime

    return Runtime(dtype, torch.device("cuda:0"))


def _context(tokens_per_request, starts, page, tables, vocab_tokens=None):
    from types import SimpleNamespace

    from einf_b200.engine.batch import StepInputBuilder

    pages = max(max(t) for t in tables) + 1
    builder = StepInputBuilder(torch.device("cuda:0"), page, [pages], [None], 1 << 20, 64, 512, 8)
    requests = [
        SimpleNamespace(input_token_ids=list(range(n)) if vocab_tokens is None else vocab_tokens[i],
                        start_position=s, block_tables=[t], state_slot=-1, need_sample=True)
        for i, (n, s, t) in enumerate(zip(tokens_per_request, starts, tables))
    ]
    return builder.build(requests)[0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from einf_b200.config import PartSpec
    from einf_b200.parts import build_part

    weight = torch.rand(72) + 0.5
    part = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 1e-4}, "n."), {"n.weight": weight.bfloat16()}, _runtime(dtype))
    residual = torch.randn(5, 72, device="cuda")
    pending = torch.randn(5, 72, device="cuda").to(dtype)
    want = plain_impl.rms_norm((residual + pending.float()).cpu(), weight.bfloat16().float(), 1e-4)
    out = part.forward(pending, residual)
    tolerance = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float().cpu(), want, **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from einf_b200.config import PartSpec
    from einf_b200.parts import build_part

    torch.manual_seed(1)
    g, u, d = (torch.randn(56, 40) * 0.2).bfloat16(), (torch.randn(56, 40) * 0.2).bfloat16(), (torch.randn(40, 56) * 0.2).bfloat16()
    spec = PartSpec("gated_mlp", {"hidden_size": 40, "intermediate_size": 56, "activation": "silu"}, "m.")
    part = build_part("feed_forward", spec, {"m.gate_proj.weight": g, "m.up_proj.weight": u, "m.down_proj.weight": d}, _runtime(dtype))
    x = torch.randn(9, 40, device="cuda").to(dtype)
    round_ = plain_impl._rounder("bfloat16" if dtype == torch.bfloat16 else None)
    want = plain_impl.swiglu(x.float().cpu(), g.float(), u.float(), d.float(), round_)
    from types import SimpleNamespace
    out = part.forward(x, SimpleNamespace(status=torch.zeros(1, dtype=torch.int32, device="cuda")))
    if out.dim() == 3:
        out = out.sum(0)     # split-K partial sums: the next norm would add them up
    tolerance = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float().cpu(), want, **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window, position_kind, out_bias", [(None, "rope", False), (5, "rope", True), (None, "none", False)])
def test_attention_part(dtype, window, position_kind, out_bias):
    """The mixer alone, a whole sequence in two portions over shuffled pages, against the
    plain functions; also with an output bias and without position encoding."""
    from einf_b200.config import PartSpec
    from einf_b200.parts import CacheView, build_part

    torch.manual_seed(2)
    hidden, heads, kv_heads, size, page = 40, 5, 1, 32, 4
    tensors = {
        "a.q_proj.weight": torch.randn(heads * size, hidden) * 0.2, "a.k_proj.weight": torch.randn(kv_heads * size, hidden) * 0.2,
        "a.v_proj.weight": torch.randn(kv_heads * size, hidden) * 0.2, "a.o_proj.weight": torch.randn(hidden, heads * size) * 0.2,
        "a.q_proj.bias": torch.randn(heads * size) * 0.2, "a.k_proj.bias": torch.randn(kv_heads * size) * 0.2,
        "a.v_proj.bias": torch.randn(kv_heads * size) * 0.2, "a.o_proj.bias": torch.randn(hidden) * 0.2,
    }
    tensors = {k: v.bfloat16() for k, v in tensors.items()}
    position = PartSpec(position_kind, {"rotary_dim": size, "theta": 10000.0} if position_kind == "rope" else {})
    spec = PartSpec("attention", dict(hidden_size=hidden, num_heads=heads, num_kv_heads=kv_heads, head_size=size,
                                      qkv_bias=True, out_bias=out_bias, scale=size ** -0.5, window=window,
                                      position=position), "a.")
    part = build_part("mixer", spec, tensors, _runtime(dtype))
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_size, need.window) == (kv_heads, size, window)
    tokens = 11
    x = torch.randn(tokens, hidden, device="cuda").to(dtype)
    kv = torch.zeros(2, 8, kv_heads, page, size, device="cuda", dtype=dtype)
    cache = CacheView(group=0, k=kv[0], v=kv[1], writes=True, page_size=page)
    table = [6, 1, 4]
    first = part.forward(x[:7], _context([7], [0], page, [table]), cache)
    second = part.forward(x[7:], _context([4], [7], page, [table]), cache)
    first, second = (t.sum(0) if t.dim() == 3 else t for t in (first, second))   # split-K partial sums
    out = torch.cat([first.float(), second.float()]).cpu()
    # plain
    round_ = plain_impl._rounder("bfloat16" if dtype == torch.bfloat16 else None)
    f = {k: v.float() for k, v in tensors.items()}
    xs = x.float().cpu()
    q, k, v = plain_impl.qkv_projection(xs, {k.replace("a.", ""): t for k, t in f.items()}, "", heads, kv_heads, size, round_)
    v = round_(v)
    if position_kind == "rope":
        cos, sin = plain_impl.rope_cos_sin(list(range(tokens)), size, 10000.0)
        q, k = plain_impl.apply_rope(q, cos, sin), plain_impl.apply_rope(k, cos, sin)
    q, k = round_(q), round_(k)
    mixed = round_(plain_impl.causal_attention(q, k, v, size ** -0.5, window)).reshape(tokens, -1)
    want = round_(mixed @ f["a.o_proj.weight"].T)
    if out_bias:
        want = round_(want + f["a.o_proj.bias"])
    tolerance = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(out, want, **tolerance)


def test_embedding_and_head_parts():
    from einf_b200.config import PartSpec
    from einf_b200.parts import build_part

    table = torch.randn(50, 24).bfloat16()
    for dtype in (torch.float32, torch.bfloat16):
        embedding = build_part("embedding", PartSpec("embedding", {"vocab_size": 50, "hidden_size": 24}, "e."), {"e.weight": table}, _runtime(dtype))
        ctx = _context([3], [0], 4, [[0]], vocab_tokens=[[49, 0, 7]])
        torch.testing.assert_close(embedding.forward(ctx).cpu(), table.float()[[49, 0, 7]], rtol=0, atol=0)
        head = build_part("head", PartSpec("linear_head", {"vocab_size": 50, "hidden_size": 24, "tied_to": None}, "h."), {"h.weight": table}, _runtime(dtype))
        x = torch.randn(4, 24, device="cuda").to(dtype)
        logits = head.forward(x, torch.zeros(1, dtype=torch.int32, device="cuda"))
        assert logits.dtype == torch.float32
        torch.testing.assert_close(logits.cpu(), x.float().cpu() @ table.float().T, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)


# --- the order of layers is data ---------------------------------------------
def test_a_layer_named_twice_and_a_shared_cache(tiny_folders, tmp_path):
    """A configuration defined here: four runs over two layers' weights, the last one reading
    the keys and values of the first run of its layer."""
    from einf_b200.config import Qwen2Config, register_architecture
    from einf_b200.config.specs import ModelSpec, ScheduleEntry
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.weights import write_random_model

    order = ((0, None), (1, None), (0, None), (1, 1))

    @dataclasses.dataclass(frozen=True)
    class LoopedConfig(Qwen2Config):
        architecture = "LoopedQwen2ForTests"

        def model_spec(self):
            spec = super().model_spec()
            return dataclasses.replace(spec, schedule=tuple(ScheduleEntry(l, c) for l, c in order))

    register_architecture(LoopedConfig)
    config = LoopedConfig.from_dict({k: v for k, v in TINY["A"].items() if k != "architectures"})
    folder = write_random_model(tmp_path / "looped", config, seed=3)
    requests = {"r0": random_tokens(256, 23, 1), "r1": random_tokens(256, 10, 2)}
    plain_config, tensors = plain_impl.read_folder(folder)
    expected = {}
    for name, tokens in requests.items():
        logits = plain_impl.forward(plain_config, tensors, tokens, schedule=list(order)).numpy()
        expected.update({(name, i): logits[i] for i in range(len(tokens))})
    replayer = TraceReplayer(folder, "float32", 64, block_len=4)
    assert len(replayer.runner.storage._owned) == 3   # three caches for four runs
    rows = trace_tools.run_steps(replayer, trace_tools.in_portions(requests, sizes=(5, 2, 3)))
    trace_tools.compare(rows, expected, rtol=1e-4, atol=2e-5)


# --- a mixer with state of its own, defined here -------------------------------
def test_a_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A mixer that keeps, per request, the running sum of its inputs and returns their
    running mean through a learned matrix.  It is registered, given a configuration, built,
    and stepped in portions beside another request, without touching the framework."""
    from einf_b200.config import ModelConfig, register_architecture
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.parts import Mixer, StateNeed, register_part
    from einf_b200.weights import write_random_model

    @register_part("mixer", "running_mean_for_tests")
    class RunningMean(Mixer):
        graph_safe = False   # forward reads the slots on the host

        @classmethod
        def tensor_specs(cls, spec):
            return {"mix.weight": TensorSpec((spec["hidden_size"], spec["hidden_size"]))}

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.hidden = spec["hidden_size"]
            self.weight = tensors["mix.weight"].to(runtime.device, torch.float32)

        def cache_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)   # sum and count

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            slots = ctx.state_slots.tolist()
            cursor = 0
            for slot, q_len in zip(slots, ctx.q_lens):
                state = cache.state[slot]
                rows = x[cursor:cursor + q_len].float()
                sums = state[: self.hidden] + rows.cumsum(0)
                counts = state[self.hidden] + torch.arange(1, q_len + 1, device=x.device)
                out[cursor:cursor + q_len] = ((sums / counts[:, None]) @ self.weight.T).to(x.dtype)
                state[: self.hidden] = sums[-1]
                state[self.hidden] = counts[-1]
                cursor += q_len
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "RunningMeanForTests"
        vocab_size: int = 50
        hidden_size: int = 24
        layers: int = 2

        def model_spec(self):
            norm = {"size": self.hidden_size, "eps": 1e-5}
            layers = tuple(
                LayerSpec("prenorm", {
                    "mixer": PartSpec("running_mean_for_tests", {"hidden_size": self.hidden_size}, f"l{i}.mixer."),
                    "feed_forward": PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 32, "activation": "silu"}, f"l{i}.mlp."),
                    "mixer_norm": PartSpec("rmsnorm", norm, f"l{i}.norm1."),
                    "feed_forward_norm": PartSpec("rmsnorm", norm, f"l{i}.norm2."),
                }) for i in range(self.layers))
            return ModelSpec(
                self.hidden_size, self.vocab_size,
                PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "embed."),
                layers, tuple(ScheduleEntry(i) for i in range(self.layers)),
                PartSpec("rmsnorm", norm, "final."),
                PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied_to": "embed.weight"}, "head."),
            )

    register_architecture(ToyConfig)
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=1)
    requests = {"r0": random_tokens(50, 19, 3), "r1": random_tokens(50, 8, 4), "r2": random_tokens(50, 12, 5)}
    whole = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), trace_tools.whole(requests))
    steps, _ = trace_tools.mixed(requests, seed=2, max_live=2, page_round=4)
    replayer = TraceReplayer(folder, "float32", 64, block_len=4)
    assert replayer.runner.num_state_slots > 0 and replayer.manager.num_state_slots > 0
    cut = trace_tools.run_steps(replayer, steps)
    trace_tools.compare(cut, whole, rtol=1e-4, atol=1e-5)
    assert replayer.manager.free_state_slots == replayer.manager.num_state_slots
    # and the running mean is what it claims: position 0 of a request sees itself only
    a = whole[("r0", 0)]
    b = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4),
                              trace_tools.whole({"x": requests["r0"][:1]}))[("x", 0)]
    assert abs(a - b).max() < 1e-5


def test_a_toy_state_mixer_that_runs_from_device_memory_keeps_graphs_and_lookahead(tmp_path):
    """The same running mean, written so that nothing of the device is read on the host: the
    request's slot is found with ``ctx.state_slots`` on the device.  Such a mixer keeps the
    engine's CUDA graphs (decode buckets with padding requests, whose slot is -1, and prompt
    portions by shape) and several decode steps per report; the state rows of requests that start
    are cleared by a kernel inside the captured step.  Nothing in the framework names it."""
    from einf_b200.config import EngineConfig, ModelConfig, register_architecture
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.engine import Engine
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.parts import Mixer, StateNeed, register_part
    from einf_b200.weights import write_random_model

    @register_part("mixer", "device_running_mean_for_tests")
    class DeviceRunningMean(Mixer):
        @classmethod
        def tensor_specs(cls, spec):
            return {"mix.weight": TensorSpec((spec["hidden_size"], spec["hidden_size"]))}

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.hidden = spec["hidden_size"]
            self.weight = tensors["mix.weight"].to(runtime.device, torch.float32)

        def cache_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)   # sum and count

        def forward(self, x, ctx, cache):
            state, hidden = cache.state, self.hidden
            device = x.device
            slots, seq = ctx.state_slots.long(), ctx.seq_of_token.long()
            # which slot each request holds, as a 0/1 matrix (a padding request, slot -1, holds none)
            holds = (slots[:, None] == torch.arange(state.shape[0], device=device)[None, :]).float()
            before = holds @ state                                            # [requests, hidden + 1]
            rows = x.float()
            total = rows.cumsum(0)
            first = ctx.q_start[:-1].long()
            base = torch.cat([torch.zeros((1, hidden), device=device), total])[first]
            running = before[seq, :hidden] + total - base[seq]
            counts = before[seq, hidden] + (torch.arange(x.shape[0], device=device) - first[seq] + 1)
            out = ((running / counts[:, None]) @ self.weight.T).to(x.dtype)
            last = ctx.q_start[1:].long() - 1
            after = torch.cat([running[last], counts[last, None]], dim=1)
            held = holds.sum(0) > 0
            state.copy_(torch.where(held[:, None], holds.T @ after, state))
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "DeviceRunningMeanForTests"
        vocab_size: int = 50
        hidden_size: int = 24
        layers: int = 2

        def model_spec(self):
            norm = {"size": self.hidden_size, "eps": 1e-5}
            layers = tuple(
                LayerSpec("prenorm", {
                    "mixer": PartSpec("device_running_mean_for_tests", {"hidden_size": self.hidden_size}, f"l{i}.mixer."),
                    "feed_forward": PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 32, "activation": "silu"}, f"l{i}.mlp."),
                    "mixer_norm": PartSpec("rmsnorm", norm, f"l{i}.norm1."),
                    "feed_forward_norm": PartSpec("rmsnorm", norm, f"l{i}.norm2."),
                }) for i in range(self.layers))
            return ModelSpec(
                self.hidden_size, self.vocab_size,
                PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "embed."),
                layers, tuple(ScheduleEntry(i) for i in range(self.layers)),
                PartSpec("rmsnorm", norm, "final."),
                PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied_to": "embed.weight"}, "head."),
            )

    register_architecture(ToyConfig)
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=1)
    # logits: whole requests against requests cut and mixed (the state carries over portions)
    requests = {"r0": random_tokens(50, 19, 3), "r1": random_tokens(50, 8, 4), "r2": random_tokens(50, 12, 5)}
    whole = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), trace_tools.whole(requests))
    steps, _ = trace_tools.mixed(requests, seed=2, max_live=2, page_round=4)
    cut = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), steps)
    trace_tools.compare(cut, whole, rtol=1e-4, atol=1e-5)
    # tokens: graphs and lookahead against eager single steps, more requests than slots, twice
    # (the second time every slot has been used before and must be cleared again)
    prompts = [random_tokens(50, n, 600 + n) for n in (5, 9, 13, 30, 3, 17)]

    def engine(**options):
        settings = dict(dtype="float32", block_len=4, num_blocks=64, max_batch_len=16, max_prefill_chunk_len=6,
                        max_requests=4)
        settings.update(options)
        return Engine.from_folder(folder, EngineConfig(**settings), eos_token_ids=())

    eager = engine(use_cuda_graphs=False)
    assert eager.runner.num_state_slots == 4
    want = eager.generate(prompts, 14)
    assert eager.generate(prompts, 14) == want and eager.runner.graph_replays == 0
    for lookahead in (1, 4):
        graphs = engine(use_cuda_graphs=True, decode_lookahead=lookahead)
        assert graphs.runner.graphs_enabled and graphs.scheduler.decode_lookahead == lookahead
        assert graphs.generate(prompts, 14) == want
        assert graphs.generate(prompts, 14) == want
        assert graphs.runner.graph_replays > 10
        assert (graphs.executor.ahead_batches > 0) == (lookahead > 1)
        assert graphs.scheduler.free_pages() == 64


def test_a_toy_mixer_whose_launches_depend_on_a_host_side_figure_says_so_in_its_launch_key(tmp_path):
    """A mixer may pick what it launches from host-side figures of the step (the framework's own
    attention cuts a token's keys by the longest context).  A captured graph would pin the pick;
    ``launch_key`` tells the runner what the pick depends on, and steps whose keys differ get
    graphs of their own.  Here the pick changes the result (another matrix once the longest
    context passes 16 tokens), so a pinned pick would show: with graphs, the same tokens as without
    them, from two graphs per batch-size bucket."""
    from einf_b200.config import EngineConfig, ModelConfig, register_architecture
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.engine import Engine
    from einf_b200.parts import Mixer, register_part
    from einf_b200.weights import write_random_model

    @register_part("mixer", "two_regimes_for_tests")
    class TwoRegimes(Mixer):
        @classmethod
        def tensor_specs(cls, spec):
            size = spec["hidden_size"]
            return {"near.weight": TensorSpec((size, size)), "far.weight": TensorSpec((size, size))}

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.near = tensors["near.weight"].to(runtime.device, torch.float32)
            self.far = tensors["far.weight"].to(runtime.device, torch.float32)

        def cache_need(self):
            return None

        def launch_key(self, ctx, page_size):
            return (ctx.max_context_len > 16,)

        def launch_group(self):
            return "two_regimes"

        def forward(self, x, ctx, cache):
            weight = self.far if ctx.max_context_len > 16 else self.near      # a host-side pick
            return (x.float() @ weight.T).to(x.dtype)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "TwoRegimesForTests"
        vocab_size: int = 40
        hidden_size: int = 16

        def model_spec(self):
            norm = {"size": self.hidden_size, "eps": 1e-5}
            layers = tuple(
                LayerSpec("prenorm", {
                    "mixer": PartSpec("two_regimes_for_tests", {"hidden_size": self.hidden_size}, f"l{i}.mixer."),
                    "feed_forward": PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 24, "activation": "silu"}, f"l{i}.mlp."),
                    "mixer_norm": PartSpec("rmsnorm", norm, f"l{i}.norm1."),
                    "feed_forward_norm": PartSpec("rmsnorm", norm, f"l{i}.norm2."),
                }) for i in range(2))
            return ModelSpec(
                self.hidden_size, self.vocab_size,
                PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "embed."),
                layers, (ScheduleEntry(0), ScheduleEntry(1)),
                PartSpec("rmsnorm", norm, "final."),
                PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied_to": "embed.weight"}, "head."),
            )

    register_architecture(ToyConfig)
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=3)
    prompts = [random_tokens(40, n, 800 + n) for n in (5, 7)]

    def engine(graphs):
        return Engine.from_folder(folder, EngineConfig(dtype="float32", block_len=4, num_blocks=32, max_batch_len=16,
                                                       max_prefill_chunk_len=8, max_requests=2, use_cuda_graphs=graphs),
                                  eos_token_ids=())

    eager, captured = engine(False), engine(True)
    want = eager.generate(prompts, 20)
    assert captured.generate(prompts, 20) == want
    keys = set(captured.runner._graphs)
    assert {(2, ((False,),)), (2, ((True,),))} <= keys and captured.runner.graph_replays > 10


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding(tmp_path):
    """Two more parts defined here, not in the framework: a feed-forward that routes each token
    to one of three small experts (router logits and softmax in 32-bit), used in layer 0 only while
    layer 1 keeps the dense one, and a position encoding that adds a position-dependent offset to
    queries and keys before the framework's own paged store.  Registered, configured, built, and
    stepped whole and in mixed portions with the same logits."""
    from einf_b200 import ops
    from einf_b200.config import ModelConfig, register_architecture
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.parts import FeedForward, register_part
    from einf_b200.parts.position import PositionEncoding
    from einf_b200.weights import write_random_model

    chosen_experts = []

    @register_part("feed_forward", "top1_experts_for_tests")
    class TopOneExperts(FeedForward):
        graph_safe = False

        @classmethod
        def tensor_specs(cls, spec):
            hidden, inner, experts = spec["hidden_size"], spec["expert_size"], spec["experts"]
            specs = {"router.weight": TensorSpec((experts, hidden))}
            for e in range(experts):
                specs[f"experts.{e}.up.weight"] = TensorSpec((inner, hidden))
                specs[f"experts.{e}.down.weight"] = TensorSpec((hidden, inner))
            return specs

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.experts = spec["experts"]
            # a router with a clear preference per token (random weights would leave near ties)
            self.router = tensors["router.weight"].to(runtime.device, torch.float32) * 40.0
            self.up = [tensors[f"experts.{e}.up.weight"].to(runtime.device, torch.float32) for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].to(runtime.device, torch.float32) for e in range(self.experts)]

        def forward(self, x, ctx):
            rows = x.float()
            gates = torch.softmax(rows @ self.router.T, dim=-1)          # 32-bit
            weight, expert = gates.max(dim=-1)
            chosen_experts.extend(expert.tolist())
            out = torch.zeros_like(rows)
            for e in range(self.experts):
                mine = expert == e
                if mine.any():
                    hidden = torch.nn.functional.silu(rows[mine] @ self.up[e].T)
                    out[mine] = (hidden @ self.down[e].T) * weight[mine, None]
            return out.to(x.dtype)

    @register_part("position", "offset_for_tests")
    class OffsetPosition(PositionEncoding):
        @classmethod
        def kernel_libraries(cls, spec, runtime):
            return ("pointwise",)

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.rate = float(spec["rate"])
            self.no_rotation = torch.empty(0, dtype=torch.float32, device=runtime.device)

        def encode_and_store(self, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size):
            rows = (qkv.sum(0) if qkv.dim() == 3 else qkv).float()
            if bias is not None:
                rows = rows + bias
            rotated = (num_heads + num_kv_heads) * head_size              # Q and K, not V
            dims = torch.arange(head_size, device=rows.device, dtype=torch.float32).repeat(num_heads + num_kv_heads)
            angle = ctx.positions.float()[:, None] * self.rate / (1.0 + dims[None, :])
            rows[:, :rotated] += 0.5 * torch.sin(angle)
            writes = cache is not None and cache.writes and cache.k is not None
            ops.rope_kv_write(rows.to(q_out.dtype), None, ctx.positions, self.no_rotation,
                              ctx.slots[cache.group] if writes else None, q_out,
                              cache.k if writes else None, cache.v if writes else None,
                              num_heads, num_kv_heads, head_size, ctx.status)

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architecture = "RoutedForTests"
        vocab_size: int = 61
        hidden_size: int = 48
        layers: int = 2

        def model_spec(self):
            norm = {"size": self.hidden_size, "eps": 1e-5}
            attention = lambda i: PartSpec("attention", dict(
                hidden_size=self.hidden_size, num_heads=3, num_kv_heads=1, head_size=16, qkv_bias=False, out_bias=False,
                scale=0.25, window=None, position=PartSpec("offset_for_tests", {"rate": 0.7})), f"l{i}.attn.")
            routed = PartSpec("top1_experts_for_tests", {"hidden_size": self.hidden_size, "expert_size": 20, "experts": 3}, "l0.moe.")
            dense = PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 40, "activation": "silu"}, "l1.mlp.")
            layers = tuple(
                LayerSpec("prenorm", {
                    "mixer": attention(i), "feed_forward": routed if i == 0 else dense,
                    "mixer_norm": PartSpec("rmsnorm", norm, f"l{i}.norm1."),
                    "feed_forward_norm": PartSpec("rmsnorm", norm, f"l{i}.norm2."),
                }) for i in range(self.layers))
            return ModelSpec(
                self.hidden_size, self.vocab_size,
                PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "embed."),
                layers, tuple(ScheduleEntry(i) for i in range(self.layers)),
                PartSpec("rmsnorm", norm, "final."),
                PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "tied_to": "embed.weight"}, "head."),
            )

    register_architecture(RoutedConfig)
    folder = write_random_model(tmp_path / "routed", RoutedConfig(), seed=3)
    requests = {"r0": random_tokens(61, 21, 6), "r1": random_tokens(61, 9, 7), "r2": random_tokens(61, 14, 8)}
    whole = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), trace_tools.whole(requests))
    assert len(set(chosen_experts)) >= 2           # the router does route
    steps, _ = trace_tools.mixed(requests, seed=5, max_live=3, page_round=4)
    cut = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), steps)
    trace_tools.compare(cut, whole, rtol=1e-4, atol=1e-5)
    again = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4),
                                  trace_tools.whole({"x": requests["r0"][:1] + requests["r1"]}))
    assert abs(again[("x", 0)] - whole[("r0", 0)]).max() < 1e-5   # same token, same place, same logits


def test_a_toy_norm_and_a_toy_block(tmp_path):
    """The last two categories defined outside the framework: a norm with a mean and a bias (layer
    norm) and a block that runs mixer and feed-forward side by side from one norm and adds both
    (``h += attention(norm(h)) + mlp(norm(h))``).  Registered, configured, written as a random
    folder, loaded, and stepped whole and in mixed portions; the logits are also recomputed here in
    plain PyTorch from the folder's tensors."""
    from safetensors.torch import load_file

    from einf_b200.config import ModelConfig, register_architecture
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.engine.replay import TraceReplayer
    from einf_b200.parts import Block, Norm, build_part, register_part
    from einf_b200.weights import write_random_model

    def dense(t):
        return t.float().sum(0) if t.dim() == 3 else t.float()

    @register_part("norm", "layernorm_for_tests")
    class LayerNorm(Norm):
        @classmethod
        def tensor_specs(cls, spec):
            return {"weight": TensorSpec((spec["size"],), "scale"), "bias": TensorSpec((spec["size"],), "bias")}

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.eps = float(spec["eps"])
            self.weight, self.bias = runtime.vector(tensors["weight"]), runtime.vector(tensors["bias"])

        def forward(self, pending, residual, rows=None):
            if pending is not None:
                residual.add_(dense(pending))
            x = residual if rows is None else residual[rows.long()]
            centred = x - x.mean(-1, keepdim=True)
            normed = centred * torch.rsqrt(centred.pow(2).mean(-1, keepdim=True) + self.eps)
            return (normed * self.weight + self.bias).to(self.runtime.dtype)

    @register_part("block", "parallel_for_tests")
    class ParallelBlock(Block):
        @classmethod
        def part_categories(cls):
            return {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def __init__(self, layer_spec, tensors, runtime):
            self.runtime, self.spec = runtime, layer_spec
            for role, category in self.part_categories().items():
                setattr(self, role, build_part(category, layer_spec.parts[role], tensors, runtime))

        def forward(self, residual, pending, ctx, cache):
            x = self.norm.forward(pending, residual)
            return dense(self.mixer.forward(x, ctx, cache)) + dense(self.feed_forward.forward(x, ctx))

    @dataclasses.dataclass(frozen=True)
    class ParallelConfig(ModelConfig):
        architecture = "ParallelForTests"
        vocab_size: int = 73
        hidden_size: int = 40
        layers: int = 3

        def model_spec(self):
            norm = {"size": self.hidden_size, "eps": 1e-4}
            layers = tuple(
                LayerSpec("parallel_for_tests", {
                    "norm": PartSpec("layernorm_for_tests", norm, f"l{i}.ln."),
                    "mixer": PartSpec("attention", dict(
                        hidden_size=self.hidden_size, num_heads=2, num_kv_heads=1, head_size=32, qkv_bias=True,
                        out_bias=False, scale=32 ** -0.5, window=None,
                        position=PartSpec("rope", {"rotary_dim": 32, "theta": 10000.0})), f"l{i}.attn."),
                    "feed_forward": PartSpec("gated_mlp", {"hidden_size": self.hidden_size, "intermediate_size": 56,
                                                           "activation": "silu"}, f"l{i}.mlp."),
                }) for i in range(self.layers))
            return ModelSpec(
                self.hidden_size, self.vocab_size,
                PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "embed."),
                layers, tuple(ScheduleEntry(i) for i in range(self.layers)),
                PartSpec("layernorm_for_tests", norm, "final."),
                PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}, "head."),
            )

    register_architecture(ParallelConfig)
    folder = write_random_model(tmp_path / "parallel", ParallelConfig(), seed=3)
    requests = {"r0": random_tokens(73, 21, 3), "r1": random_tokens(73, 9, 4), "r2": random_tokens(73, 14, 5)}
    whole = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), trace_tools.whole(requests))
    steps, _ = trace_tools.mixed(requests, seed=4, max_live=3, page_round=4)
    cut = trace_tools.run_steps(TraceReplayer(folder, "float32", 64, block_len=4), steps)
    trace_tools.compare(cut, whole, rtol=1e-4, atol=1e-5)

    # the same model in plain PyTorch, from the folder's tensors
    tensors = {name: value.float() for name, value in load_file(str(folder / "model.safetensors")).items()}

    def layer_norm(x, prefix):
        centred = x - x.mean(-1, keepdim=True)
        return centred * torch.rsqrt(centred.pow(2).mean(-1, keepdim=True) + 1e-4) * tensors[prefix + "weight"] + tensors[prefix + "bias"]

    for name, tokens in requests.items():
        h = tensors["embed.weight"][tokens]
        positions = torch.arange(len(tokens))
        for i in range(3):
            x = layer_norm(h, f"l{i}.ln.")
            q, k, v = plain_impl.qkv_projection(x, {n.replace(f"l{i}.attn.", "p."): t for n, t in tensors.items()}, "p.", 2, 1, 32, lambda t: t)
            cos, sin = plain_impl.rope_cos_sin(positions, 32, 10000.0)
            attended = plain_impl.causal_attention(plain_impl.apply_rope(q, cos, sin), plain_impl.apply_rope(k, cos, sin), v, 32 ** -0.5, None)
            mixed = attended.reshape(len(tokens), -1) @ tensors[f"l{i}.attn.o_proj.weight"].T
            mlp = plain_impl.swiglu(x, tensors[f"l{i}.mlp.gate_proj.weight"], tensors[f"l{i}.mlp.up_proj.weight"],
                                    tensors[f"l{i}.mlp.down_proj.weight"], lambda t: t)
            h = h + mixed + mlp
        logits = layer_norm(h, "final.") @ tensors["head.weight"].T
        for position in range(len(tokens)):
            assert np.abs(whole[(name, position)] - logits[position].numpy()).max() < 2e-4, (name, position)
