"""Decode and prefill throughput of the engine on one B200, with its roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  The default run has the layer sizes of Qwen2.5-0.5B with
random weights in bfloat16, a batch of 8 requests at a context of 4,096 tokens;
a "step" is one decode step.  ``value`` is decoded tokens a second timed on the
device over exactly K steps; ``e2e`` is the same through the Python entry point
(`Engine.submit` / `Engine.step`), host tokens in and out; ``prefill`` is one
2,048-token prompt; ``roofline`` compares the bytes a decode step has to read
(every weight once and the cache of the live requests) with the measured copy
bandwidth; ``points`` holds decoding at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN25_05B = dict(
    architectures=["Qwen2ForCausalLM"], vocab_size=151936, hidden_size=896, intermediate_size=4864,
    num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2, rms_norm_eps=1e-6,
    hidden_act="silu", rope_theta=1000000.0, max_position_embeddings=32768, tie_word_embeddings=True,
    bos_token_id=151643, eos_token_id=151643,
)
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.lines: list[str] = []
        self.process = None
        self.thread = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return

        def pump() -> None:
            for line in self.process.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(float(fields[0]))
                max_clock = float(fields[1])
            except ValueError:
                continue
            for name, value in zip(names, fields[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def model_numbers(cfg: dict) -> dict:
    """Bytes a decode step reads and flops a prefill does, from the sizes alone."""
    h, i, layers, vocab = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = h // hq
    per_layer = (hq + 2 * hkv) * d * h + (hq + 2 * hkv) * d + hq * d * h + 3 * i * h + 2 * h
    weights = layers * per_layer + vocab * h + h            # the output matrix is read once (tied: it is the table)
    kv_per_token = layers * 2 * hkv * d * 2                 # bytes, bfloat16
    linear_flops_per_token = 2 * layers * ((hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h)
    return dict(weight_bytes=2 * weights, kv_bytes_per_token=kv_per_token,
                linear_flops_per_token=linear_flops_per_token, head_dim=d,
                attention_flops=lambda t: layers * 4 * hq * d * t * (t + 1) // 2,
                head_flops_per_row=2 * vocab * h)


def decode_requests(batch: int, context: int, runner, manager, tag: str):
    """Requests that stand at position `context`: their pages are reserved, their
    cache holds whatever the pool holds (timing does not depend on the values)."""
    import torch

    requests = []
    generator = torch.Generator().manual_seed(batch)
    for index in range(batch):
        name = f"{tag}{index}"
        if not manager.reserve(name, 0, context + 1):
            raise RuntimeError("the pool is too small for the benchmark")
        requests.append(SimpleNamespace(
            request_id=name, input_token_ids=[int(torch.randint(3, 150000, (1,), generator=generator))],
            start_position=context, block_tables=[manager.block_table(name, 0)], state_slot=-1, need_sample=True))
    return requests


def time_decode(runner, sampler, manager, batch: int, context: int, steps: int, warmup: int,
                min_seconds: float = 0.2) -> dict:
    """Decode steps of `batch` requests near `context`, timed with CUDA events: regions of exactly
    `steps` steps each, repeated until about `min_seconds` have been timed; the figure is the
    median region (one region when `steps` steps alone take that long)."""
    import torch

    from einf_b200 import ops
    from einf_b200.sampling import GREEDY

    tag = f"b{batch}_"
    room = min(context // 2, steps + warmup + 8)     # every timed step stands within `room` tokens of `context`
    requests = decode_requests(batch, context - room, runner, manager, tag)
    params, indices = [GREEDY] * batch, [0] * batch
    budget = [room - 1]

    def one_step() -> None:
        if budget[0] <= 0:        # stay below `context`: start over from where the run began
            for request in requests:
                request.start_position = context - room
            budget[0] = room - 1
        budget[0] -= 1
        output = runner.step(requests)
        sampler.sample(output.logits, params, indices)
        for request in requests:
            request.start_position += 1
            if request.start_position % PAGE == 0:
                manager.reserve(request.request_id, request.start_position, request.start_position + 1)
                request.block_tables = [manager.block_table(request.request_id, 0)]

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    regions, launches, timed = [], 0, 0.0
    while not regions or (timed < min_seconds and len(regions) < 64):
        before = ops.launch_count + runner.graph_kernel_launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        launches = ops.launch_count + runner.graph_kernel_launches - before
        regions.append(start.elapsed_time(end) / steps)
        timed += regions[-1] * steps * 1e-3
    ms = statistics.median(regions)
    for request in requests:
        manager.release(request.request_id)
    return {"ms_per_step": ms, "tokens_per_s": batch / ms * 1e3, "launches": launches, "regions": len(regions)}


def time_prefill(runner, sampler, manager, tokens: int, repeats: int = 7) -> dict:
    """One prompt of `tokens` tokens in one step, first token sampled: the median of `repeats` runs."""
    import torch

    from einf_b200.sampling import GREEDY

    generator = torch.Generator().manual_seed(1)
    ids = torch.randint(3, 150000, (tokens,), generator=generator).tolist()
    times = []
    for attempt in range(repeats + 3):
        name = f"prefill{attempt}"
        manager.reserve(name, 0, tokens)
        request = SimpleNamespace(request_id=name, input_token_ids=ids, start_position=0,
                                  block_tables=[manager.block_table(name, 0)], state_slot=-1, need_sample=True)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        output = runner.step([request])
        sampler.sample(output.logits, [GREEDY], [0])
        end.record()
        torch.cuda.synchronize()
        manager.release(name)
        if attempt >= 3:
            times.append(start.elapsed_time(end))
    return {"ms": statistics.median(times), "tokens": tokens, "ms_min": min(times), "repeats": len(times)}


def time_e2e(engine, batch: int, context: int, steps: int, warmup: int) -> dict:
    """The same decode through Engine.submit / Engine.step: prompts from host memory in,
    sampled tokens read back to the host at every report (every step, unless the engine looks ahead)."""
    import torch

    generator = torch.Generator().manual_seed(2)
    prompt_len = context - steps - warmup - 1
    ids = []
    for index in range(batch):
        prompt = torch.randint(3, 150000, (prompt_len,), generator=generator).tolist()
        ids.append(engine.submit(prompt, steps + warmup + 8, request_id=f"e2e{index}"))
    while any(engine.request(i).cached_len < prompt_len for i in ids):   # drain the prefill
        engine.step()

    def generated() -> int:
        return sum(len(engine.request(i).generated_token_ids) for i in ids)

    # With a decode lookahead one call of Engine.step runs several decode steps; tokens and decode
    # steps are counted, not calls.
    while generated() < batch * warmup:
        engine.step()
    h2d_before, d2h_before = engine.runner.inputs.h2d_bytes, engine.executor.d2h_bytes
    tokens_before, steps_before = generated(), engine.scheduler.stats.steps
    torch.cuda.synchronize()
    started = time.perf_counter()
    while generated() < tokens_before + batch * steps:
        engine.step()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    tokens = generated() - tokens_before
    decode_steps = engine.scheduler.stats.steps - steps_before
    h2d = (engine.runner.inputs.h2d_bytes - h2d_before) / decode_steps
    d2h = (engine.executor.d2h_bytes - d2h_before) / decode_steps
    while engine.scheduler.has_outstanding:      # a plan of several steps may still be in flight
        engine.step()
    for i in ids:
        engine.cancel(i)
    return {"value": tokens / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": elapsed / decode_steps * 1e3}


SIZES = {
    "1.5b": dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=151936, hidden_size=1536, intermediate_size=8960,
        num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2, rms_norm_eps=1e-6,
        hidden_act="silu", rope_theta=1000000.0, max_position_embeddings=32768, tie_word_embeddings=True,
        bos_token_id=151643, eos_token_id=151643,
    ),
    "7b": dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=152064, hidden_size=3584, intermediate_size=18944,
        num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rms_norm_eps=1e-6,
        hidden_act="silu", rope_theta=1000000.0, max_position_embeddings=32768, tie_word_embeddings=False,
        bos_token_id=151643, eos_token_id=151643,
    ),
}


def _graph_time_us(fn, launches: int) -> float:
    """Median over five replays of a CUDA graph of ``launches`` calls of ``fn``, per call."""
    import torch

    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            fn()
    times = []
    for _ in range(5):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1000 / launches)
    return sorted(times)[2]


def run_sampling(args) -> dict:
    """The draw alone: ``ops.argmax`` and ``ops.sample`` on rows of 151,936 logits (the vocabulary of
    the benchmark's model) with each filter, 1 / 8 / 64 rows, microseconds per launch."""
    import torch

    from einf_b200 import ops

    device = torch.device("cuda:0")
    vocab = QWEN25_05B["vocab_size"]
    result = {"scenario": "sampling", "vocab": vocab, "unit": "us per launch"}
    cases = (("temperature", 0, 1.0, 0.0), ("top_k50", 50, 1.0, 0.0), ("top_p0.9", 0, 0.9, 0.0), ("min_p0.05", 0, 1.0, 0.05),
             ("top_k50_top_p0.9_min_p0.05", 50, 0.9, 0.05))
    for rows in (1, 8, 64):
        logits = torch.randn(rows, vocab, device=device) * 3
        tokens = torch.zeros(rows, dtype=torch.int32, device=device)
        seed = torch.arange(rows, dtype=torch.int64, device=device)
        index = torch.zeros(rows, dtype=torch.int64, device=device)
        result[f"argmax_rows{rows}"] = round(_graph_time_us(lambda: ops.argmax(logits, tokens), 20), 1)
        for name, k, p, m in cases:
            temperature = torch.full((rows,), 0.8, device=device)
            top_k = torch.full((rows,), k, dtype=torch.int32, device=device)
            top_p, min_p = torch.full((rows,), p, device=device), torch.full((rows,), m, device=device)
            result[f"{name}_rows{rows}"] = round(_graph_time_us(
                lambda: ops.sample(logits, tokens, temperature, top_k, top_p, min_p, seed, index), 20), 1)
    return result


def run_prefill_attention(args) -> dict:
    """The prefill attention kernel alone at the head counts and sizes of the three model sizes: a
    whole prompt, a late portion of a long one, a short portion; microseconds per launch (the
    cluster size is the one the engine would pick) and TFLOP/s."""
    import torch

    from einf_b200 import ops

    device = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=device)
    result = {"scenario": "prefill-attention", "page_size": PAGE, "unit": "us per launch"}
    launches = 8
    for heads, kv_heads, size in ((14, 2, 64), (12, 2, 128), (28, 4, 128)):
        ops.ensure_built(list(ops.attention_libraries(size, PAGE)))
        for tokens, cached in ((2048, 0), (8192, 0), (512, 1536), (512, 8192), (128, 4096), (64, 512), (128, 0)):
            pages = -(-(cached + tokens) // PAGE)
            k = torch.randn(pages * launches + 4, kv_heads, PAGE, size, device=device).bfloat16()
            v = torch.randn_like(k)
            q = torch.randn(tokens, heads, size, device=device).bfloat16()
            out = torch.empty_like(q)
            tables = [torch.arange(i * pages, (i + 1) * pages, dtype=torch.int32, device=device).view(1, -1)
                      for i in range(launches)]
            tiles = torch.tensor([[0, first, min(128, tokens - first), cached + first] for first in range(0, tokens, 128)],
                                 dtype=torch.int32, device=device)
            turn = [0]

            def launch():
                table = tables[turn[0] % launches]   # another request's pages every launch: K and V do not stay in L2
                turn[0] += 1
                ops.paged_prefill_attention(q, k, v, table, tiles, out, size ** -0.5, None, status, cached_before=cached)

            us = _graph_time_us(launch, launches)
            flops = 4 * heads * size * (tokens * cached + tokens * tokens / 2)
            key = f"h{heads}_d{size}_{tokens}after{cached}"
            result[key + "_us"] = round(us, 1)
            result[key + "_tflops"] = round(flops / us / 1e6)
    result["status"] = int(status)
    return result


def run_decode_attention(args) -> dict:
    """The decode attention kernel alone at the head counts and sizes of the three model sizes, for
    1, 8 and 64 requests at contexts from 1,024 to 32,768 tokens: microseconds per launch (kernel
    and cluster size are the ones the engine would pick) and the rate at which the requests' keys
    and values are read, in GB/s.  Every launch of the timed graph reads another layer's pages."""
    import torch

    from einf_b200 import ops

    device = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=device)
    result = {"scenario": "decode-attention", "page_size": PAGE, "unit": "us per launch"}
    for heads, kv_heads, size in ((14, 2, 64), (12, 2, 128), (28, 4, 128)):
        ops.ensure_built(list(ops.attention_libraries(size, PAGE)))
        for batch, context in ((1, 4096), (1, 32768), (8, 1024), (8, 4096), (8, 16384), (8, 32768), (64, 4096)):
            pages = context // PAGE
            layer_bytes = 2 * batch * context * kv_heads * size * 2
            launches = max(4, min(12, int(1.5e9 // layer_bytes)))   # more than the L2 holds, a few GB at most
            k = torch.randn(pages * batch * launches + 2, kv_heads, PAGE, size, device=device).bfloat16()
            v = torch.randn_like(k)
            q = torch.randn(batch, heads, size, device=device).bfloat16()
            out = torch.empty_like(q)
            tables = [torch.arange(i * pages * batch, (i + 1) * pages * batch, dtype=torch.int32, device=device).view(batch, pages)
                      for i in range(launches)]
            seq = torch.arange(batch, dtype=torch.int32, device=device)
            positions = torch.full((batch,), context - 1, dtype=torch.int32, device=device)
            turn = [0]

            def launch():
                table = tables[turn[0] % launches]
                turn[0] += 1
                ops.paged_decode_attention_auto(q, k, v, table, seq, positions, out, size ** -0.5, None, status,
                                                max_context=context)

            us = _graph_time_us(launch, launches)
            kernel, cluster, splits = ops.decode_plan(batch, heads, kv_heads, size, PAGE, context)
            key = f"h{heads}_d{size}_b{batch}_ctx{context}"
            result[key + "_us"] = round(us, 1)
            result[key + "_gbs"] = round(layer_bytes / us / 1e3)
            result[key + "_plan"] = f"{kernel} {cluster}x{splits}"
            del k, v
    result["status"] = int(status)
    return result


def run_prefill_sizes(args) -> dict:
    """A prompt of 2,048 and of 8,192 tokens in one step at the three model sizes (all layers unless
    --layers says otherwise): milliseconds, tokens a second and the fraction of the tensor-core
    peak the step reaches."""
    import torch

    from einf_b200.cache import CacheManager
    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import ModelRunner
    from einf_b200.sampling import Sampler

    peak = peaks()
    result = {"scenario": "prefill-sizes"}
    for name, sizes in (("0.5b", QWEN25_05B), ("1.5b", SIZES["1.5b"]), ("7b", SIZES["7b"])):
        cfg = dict(sizes)
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
            result["layers"] = args.layers
        numbers = model_numbers(cfg)
        runner = ModelRunner.from_random(
            config_from_dict(cfg), 0,
            EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=8192 // PAGE + 64, max_batch_len=8192,
                         max_prefill_chunk_len=8192, max_requests=8))
        manager = CacheManager(runner.group_specs(), 0)
        sampler = Sampler(runner.runtime.device, 8)
        for tokens in (2048, 8192):
            timed = time_prefill(runner, sampler, manager, tokens, repeats=5)
            flops = numbers["linear_flops_per_token"] * tokens + numbers["attention_flops"](tokens) + numbers["head_flops_per_row"]
            result[f"{name}_{tokens}_ms"] = round(timed["ms"], 3)
            result[f"{name}_{tokens}_tokens_per_s"] = round(tokens / (timed["ms"] * 1e-3))
            result[f"{name}_{tokens}_frac"] = round(flops / (timed["ms"] * 1e-3) / (peak["bf16_tflops"] * 1e12), 3)
        del runner, manager, sampler
        torch.cuda.empty_cache()
    return result


def run_mixed_15b(args) -> dict:
    """Qwen2.5-1.5B sizes: every step runs 32 decoding requests at context 2,048 beside one
    512-token portion of a prompt (positions 1,536 to 2,047)."""
    import torch

    from einf_b200.cache import CacheManager
    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import ModelRunner
    from einf_b200.sampling import GREEDY, Sampler

    cfg = SIZES["1.5b"]
    numbers = model_numbers(cfg)
    peak = peaks()
    runner = ModelRunner.from_random(
        config_from_dict(cfg), 0,
        EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=40 * 130, max_batch_len=1024,
                     max_prefill_chunk_len=512, max_requests=64))
    manager = CacheManager(runner.group_specs(), 0)
    sampler = Sampler(runner.runtime.device, 64)
    generator = torch.Generator().manual_seed(3)
    requests = []
    for index in range(32):
        manager.reserve(f"d{index}", 0, 2048)
        requests.append(SimpleNamespace(request_id=f"d{index}", input_token_ids=[int(torch.randint(3, 150000, (1,), generator=generator))],
                                        start_position=2047, block_tables=[manager.block_table(f"d{index}", 0)],
                                        state_slot=-1, need_sample=True))
    manager.reserve("p", 0, 2048)
    requests.append(SimpleNamespace(request_id="p", input_token_ids=torch.randint(3, 150000, (512,), generator=generator).tolist(),
                                    start_position=1536, block_tables=[manager.block_table("p", 0)], state_slot=-1,
                                    need_sample=True))

    def one_step():
        output = runner.step(requests)
        sampler.sample(output.logits, [GREEDY] * 33, [0] * 33)

    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    step_bytes = numbers["weight_bytes"] + 33 * 2048 * numbers["kv_bytes_per_token"]
    chunk_flops = numbers["linear_flops_per_token"] * 544 + 28 * 4 * 12 * 128 * (512 * 1536 + 512 * 513 // 2)
    return {"scenario": "1.5b-mixed", "ms_per_step": round(ms, 4), "tokens_per_step": 544,
            "tokens_per_s": round(544 / ms * 1e3, 1), "decode_tokens_per_s": round(32 / ms * 1e3, 1),
            "hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4),
            "flops_frac": round(chunk_flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4), "steps": args.steps}


def run_decode_sizes(args) -> dict:
    """Decode at the 1.5B and 7B sizes of the family (batch 8 and 64, context 4,096) with the
    fraction of the HBM roofline each step reaches: at these sizes a step's kernels are long
    enough to be bound by bytes, not by the number of dependent kernels."""
    import torch

    from einf_b200.cache import CacheManager
    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import ModelRunner
    from einf_b200.sampling import Sampler

    peak = peaks()
    result = {"scenario": "decode-sizes", "context": CONTEXT, "steps": args.steps}
    for name in ("1.5b", "7b"):
        cfg = dict(SIZES[name])
        if args.layers:
            cfg["num_hidden_layers"] = args.layers     # for profiling a small case
            result["layers"] = args.layers
        numbers = model_numbers(cfg)
        pages = 64 * (CONTEXT // PAGE + 2) + 64
        runner = ModelRunner.from_random(
            config_from_dict(cfg), 0,
            EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=pages, max_batch_len=256,
                         max_prefill_chunk_len=256, max_requests=64))
        manager = CacheManager(runner.group_specs(), 0)
        sampler = Sampler(runner.runtime.device, 64)
        for batch in (1, 8, 64):
            timed = time_decode(runner, sampler, manager, batch, CONTEXT, args.steps, args.warmup)
            step_bytes = numbers["weight_bytes"] + batch * CONTEXT * numbers["kv_bytes_per_token"]
            result[f"{name}_b{batch}_tokens_per_s"] = round(timed["tokens_per_s"], 1)
            result[f"{name}_b{batch}_ms"] = round(timed["ms_per_step"], 3)
            result[f"{name}_b{batch}_hbm_frac"] = round(step_bytes / (timed["ms_per_step"] * 1e-3) / 1e9 / peak["hbm_gbs"], 3)
        del runner, manager, sampler
        torch.cuda.empty_cache()
    return result


def run_decode_contexts(args) -> dict:
    """Decode at contexts from 1,024 to 32,768 tokens (batch 8; 0.5B and 7B sizes) with the fraction
    of the HBM roofline each step reaches: the longer the context, the more of a step is the
    attention's walk over the cache."""
    import torch

    from einf_b200.cache import CacheManager
    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import ModelRunner
    from einf_b200.sampling import Sampler

    peak = peaks()
    batch = args.batch
    contexts = (1024, 4096, 16384, 32768)
    result = {"scenario": "decode-contexts", "batch": batch, "steps": args.steps}
    for name, sizes in (("0.5b", QWEN25_05B), ("7b", SIZES["7b"])):
        cfg = dict(sizes)
        if args.layers:
            cfg["num_hidden_layers"] = args.layers     # for profiling a small case
            result["layers"] = args.layers
        numbers = model_numbers(cfg)
        pages = batch * (contexts[-1] // PAGE + 2) + 64
        runner = ModelRunner.from_random(
            config_from_dict(cfg), 0,
            EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=pages, max_batch_len=256,
                         max_prefill_chunk_len=256, max_requests=64))
        manager = CacheManager(runner.group_specs(), 0)
        sampler = Sampler(runner.runtime.device, 64)
        for context in contexts:
            timed = time_decode(runner, sampler, manager, batch, context, args.steps, args.warmup)
            step_bytes = numbers["weight_bytes"] + batch * context * numbers["kv_bytes_per_token"]
            result[f"{name}_ctx{context}_ms"] = round(timed["ms_per_step"], 3)
            result[f"{name}_ctx{context}_hbm_frac"] = round(step_bytes / (timed["ms_per_step"] * 1e-3) / 1e9 / peak["hbm_gbs"], 3)
        del runner, manager, sampler
        torch.cuda.empty_cache()
    return result


def run_preempt_7b(args) -> dict:
    """Qwen2.5-7B sizes through the entry point: 64 requests with 4,096-token prompts and fewer
    pages than they all need, so the scheduler has to preempt and recompute."""
    import torch

    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import Engine

    cfg = dict(SIZES["7b"])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    new_tokens = 192
    needed = 64 * -(-(4096 + new_tokens) // PAGE)
    pages = int(needed * 0.93)
    engine = Engine.from_random(
        config_from_dict(cfg), 0,
        EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=pages, max_batch_len=4096,
                     max_prefill_chunk_len=2048, max_requests=64, policy="decode_first"),
        eos_token_ids=())
    generator = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, 150000, (4096,), generator=generator).tolist() for _ in range(64)]
    torch.cuda.synchronize()
    started = time.perf_counter()
    outputs = engine.generate(prompts, new_tokens)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    stats = engine.scheduler.stats
    return {"scenario": "7b-preempt", "layers": cfg["num_hidden_layers"], "requests": 64, "prompt_tokens": 4096,
            "new_tokens": new_tokens, "pages": pages, "pages_needed_without_preemption": needed,
            "seconds": round(elapsed, 2), "generated": sum(len(o) for o in outputs),
            "generated_tokens_per_s": round(sum(len(o) for o in outputs) / elapsed, 1),
            "prefill_tokens_run": stats.prefill_tokens, "decode_tokens_run": stats.decode_tokens,
            "preemptions": stats.preemptions, "failures": stats.failures, "steps": stats.steps}


def other_sizes_points(args) -> dict:
    """The baseline's other workloads as flat points of the default line: the mixed step at 1.5B
    sizes, decoding at 1.5B and 7B sizes with the fraction of the HBM roofline each step reaches,
    and 64 requests at 7B sizes with fewer pages than they need (preemptions and tokens a second)."""
    import gc

    import torch

    short = argparse.Namespace(**vars(args))
    short.steps, short.warmup = min(args.steps, 64), max(3, min(args.warmup, 4))
    points = {}
    mixed = run_mixed_15b(short)
    for key in ("ms_per_step", "tokens_per_s", "hbm_frac", "flops_frac"):
        points[f"1.5b_mixed_{key}"] = mixed[key]
    gc.collect()
    torch.cuda.empty_cache()
    sizes = run_decode_sizes(short)
    for key, value in sizes.items():
        if key.startswith(("1.5b_", "7b_")) and not key.endswith("_ms"):
            points[f"decode_{key}"] = value
    gc.collect()
    torch.cuda.empty_cache()
    preempt = run_preempt_7b(short)
    for key in ("generated_tokens_per_s", "preemptions", "failures", "seconds", "pages", "pages_needed_without_preemption"):
        points[f"7b_preempt_{key}"] = preempt[key]
    return points


def run_ours(args) -> dict:
    import torch

    from einf_b200.cache import CacheManager
    from einf_b200.config import EngineConfig, config_from_dict
    from einf_b200.engine import Engine
    from einf_b200.sampling import Sampler

    cfg = dict(QWEN25_05B)
    layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    config = config_from_dict(cfg)
    numbers = model_numbers(cfg)
    peak = peaks()
    pages = 64 * (CONTEXT // PAGE + 2) + PREFILL_TOKENS // PAGE + 64
    engine = Engine.from_random(
        config, seed=0,
        engine_config=EngineConfig(dtype="bfloat16", block_len=PAGE, num_blocks=pages, max_batch_len=PREFILL_TOKENS,
                                   max_prefill_chunk_len=PREFILL_TOKENS, max_requests=64, policy="decode_first",
                                   use_cuda_graphs=not args.no_graphs, max_sequence_len=CONTEXT + 64),
        eos_token_ids=(),
    )
    runner = engine.runner
    manager = CacheManager(runner.group_specs(), 0)   # pages for the device-timed runs, by hand
    sampler = Sampler(runner.runtime.device, 64)
    if args.only == "decode":
        result = time_decode(runner, sampler, manager, args.batch, CONTEXT, args.steps, args.warmup,
                             min_seconds=args.min_seconds)
        return {"only": "decode", "batch": args.batch, **{k: round(v, 4) for k, v in result.items()}}
    if args.only == "prefill":
        return {"only": "prefill", **time_prefill(runner, sampler, manager, PREFILL_TOKENS, repeats=args.steps)}
    clocks = ClockSampler()
    clocks.start()
    headline = time_decode(runner, sampler, manager, args.batch, CONTEXT, args.steps, args.warmup)
    clock_record = clocks.stop()
    points = {}
    for batch in (1, 64):
        points[f"decode_b{batch}"] = round(time_decode(runner, sampler, manager, batch, CONTEXT, args.steps, args.warmup)["tokens_per_s"], 1)
    for batch in (1, 8, 64):
        points[f"decode_b{batch}_ctx1024"] = round(time_decode(runner, sampler, manager, batch, 1024, args.steps, args.warmup)["tokens_per_s"], 1)
    prefill = time_prefill(runner, sampler, manager, PREFILL_TOKENS)
    prefill_flops = (numbers["linear_flops_per_token"] * PREFILL_TOKENS + numbers["attention_flops"](PREFILL_TOKENS)
                     + numbers["head_flops_per_row"])
    # End to end through Engine.submit / Engine.step.  The engine plans `lookahead` decode steps at a
    # time and reports each step's tokens to the host as that step ends, while the later steps of
    # the plan run (EngineConfig.decode_lookahead, report_every_step): tokens reach the caller after
    # every step.  The second figure is the same engine planning one step at a time.
    ahead_engine = Engine(runner, eos_token_ids=(), decode_lookahead=args.lookahead)
    e2e = time_e2e(ahead_engine, args.batch, CONTEXT, args.steps, args.warmup)
    e2e_single = time_e2e(engine, args.batch, CONTEXT, args.steps, args.warmup)
    step_bytes = numbers["weight_bytes"] + args.batch * CONTEXT * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (headline["ms_per_step"] * 1e-3) / 1e9
    return {
        "metric": "decode tokens/s, Qwen2.5-0.5B sizes, batch 8, context 4096 (B200)",
        "value": round(headline["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(headline["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "Qwen2.5-0.5B sizes", "layers": cfg["num_hidden_layers"], "layers_of_model": layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": numbers["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_embeddings": True, "global_batch": args.batch, "seq_len": CONTEXT, "page_size": PAGE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 GPU", "l2": "step reads > L2 (weights 988 MB)",
            "cuda_graphs": bool(getattr(runner, "graphs_enabled", False)),

        },
        "e2e": {"decode_lookahead": args.lookahead, "report_every_step": True,
                **{k: (round(v, 4 if k == "ms_per_step" else 1) if isinstance(v, float) else v) for k, v in e2e.items()}},
        "e2e_single_step_plans": {"decode_lookahead": 1,
                                  **{k: (round(v, 4 if k == "ms_per_step" else 1) if isinstance(v, float) else v)
                                     for k, v in e2e_single.items()}},
        "timed_regions": headline["regions"],
        "gpu_launches": headline["launches"],
        "clocks": clock_record,
        "prefill": {
            "value": round(PREFILL_TOKENS / (prefill["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
            "ms": round(prefill["ms"], 4),
            "frac": round(prefill_flops / (prefill["ms"] * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
        },
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"],
        },
        "points": points,
    }


def run_reference(args) -> dict:
    """The reference arm: mon3stera/einf's own executor, model runner, cache storage and sampler
    (the unmodified Python tree under baseline/_ref) on the same sizes, batch, context and page
    size, each of its attention back ends in a child process of its own (one that crashes or
    cannot be built is recorded and the others still run).  No code of einf_b200 runs here."""
    arm = ROOT / "baseline" / "reference_arm.py"
    cfg = dict(QWEN25_05B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    steps = min(args.steps, 64)     # a reference step takes milliseconds: 64 are a long enough region
    base = [sys.executable, str(arm), "--config", json.dumps(cfg), "--context", str(CONTEXT), "--block-len", str(PAGE),
            "--prefill-tokens", str(PREFILL_TOKENS), "--steps", str(steps), "--warmup", str(args.warmup),
            "--batches", f"{args.batch},1,64"]
    env = dict(os.environ)
    env.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    env.setdefault("MAX_JOBS", str(os.cpu_count() or 8))

    def child(backend: str, limit: int) -> dict:
        try:
            done = subprocess.run(base + ["--backend", backend], env=env, capture_output=True, text=True, timeout=limit)
        except subprocess.TimeoutExpired:
            return {"backend": backend, "unavailable": f"no result within {limit} s"}
        sys.stderr.write(done.stderr[-4000:])
        lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
        if done.returncode != 0 or not lines:
            tail = (done.stderr.strip().splitlines() or ["no output"])[-1][:300]
            return {"backend": backend, "unavailable": f"exit code {done.returncode}: {tail}"}
        return json.loads(lines[-1])

    # its CUDA extension first (compiled by torch at the first call of any of its ops)
    built = child("build-ops", 2400)
    backends = {"build-ops": built}
    for backend in ("flashinfer", "paged", "default"):
        backends[backend] = child(backend, 1500)
    ran = {name: record for name, record in backends.items() if "tokens_per_s_device" in record}
    if not ran:
        reasons = "; ".join(f"{name}: {record.get('unavailable')}" for name, record in backends.items()
                            if "unavailable" in record)
        return {"impl": "reference", "unavailable": f"no back end of the reference ran on this box: {reasons}"[:900]}
    best = max(ran, key=lambda name: ran[name]["tokens_per_s_wall"])
    record = ran[best]
    numbers = model_numbers(cfg)
    peak = peaks()
    step_bytes = numbers["weight_bytes"] + args.batch * CONTEXT * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (record["device_ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s, Qwen2.5-0.5B sizes, batch 8, context 4096 (B200)",
        "value": record["tokens_per_s_device"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": record["device_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "impl": "reference", "same_config": True,
        "config": {
            "model": "Qwen2.5-0.5B sizes", "layers": cfg["num_hidden_layers"], "layers_of_model": QWEN25_05B["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": numbers["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_embeddings": True, "global_batch": args.batch, "seq_len": CONTEXT, "page_size": PAGE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 GPU", "attention_backend": best,
            "scheduler_in_loop": False, "l2": "step reads > L2 (weights 988 MB)",
        },
        "reference_code": "unmodified src/einf of mon3stera/einf: TorchExecutor.execute over QwenModelRunner, "
                          "TorchKVCacheStorage, ModelInputPool, Sampler; its Rust scheduler cannot be built here, "
                          "so its executor is fed hand-made decode plans",
        "e2e": {"value": record["tokens_per_s_wall"], "unit": "tokens/s", "ms_per_step": record["wall_ms_per_step"],
                "h2d_bytes_per_step": record["h2d_bytes_per_step"], "d2h_bytes_per_step": record["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "clocks": record.get("clocks"),
        "prefill": record.get("prefill"),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": record.get("points", {}),
        "backends": {name: ({k: v for k, v in rec.items() if k not in ("clocks",)}) for name, rec in backends.items()},
    }
    prefill = line["prefill"]
    if prefill and "ms" in prefill:
        flops = (numbers["linear_flops_per_token"] * PREFILL_TOKENS + numbers["attention_flops"](PREFILL_TOKENS)
                 + numbers["head_flops_per_row"] * PREFILL_TOKENS)    # the reference's head runs every row
        prefill["frac"] = round(flops / (prefill["ms"] * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)
    return line


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--only", choices=("all", "decode", "prefill"), default="all",
                        help="time one part only (for profiling a small case); the line then lacks the other keys")
    parser.add_argument("--no-graphs", action="store_true", help="run decode steps eagerly")
    parser.add_argument("--leave-out", default="", help="comma-separated kinds of kernel to leave out of every step "
                        "(decode_attention, prefill_attention, norms, rotary, activation): what a kind costs inside "
                        "the step's CUDA graph is the step's time without it; the results are then garbage, the line "
                        "is marked, and it is no benchmark value")
    parser.add_argument("--min-seconds", type=float, default=0.2,
                        help="with --only decode: repeat the region of K steps until this much is timed (0: one region)")
    parser.add_argument("--skip-other-sizes", action="store_true",
                        help="leave the 1.5B and 7B workloads out of `points` (they take about a minute)")
    parser.add_argument("--lookahead", type=int, default=8,
                        help="EngineConfig.decode_lookahead of the end-to-end run: decode steps per report to the host")
    parser.add_argument("--scenario", choices=("default", "1.5b-mixed", "7b-preempt", "decode-sizes", "decode-contexts", "sampling", "prefill-attention", "decode-attention", "prefill-sizes"), default="default",
                        help="other workloads of the baseline: a mixed step at 1.5B sizes, decoding under "
                             "cache pressure at 7B sizes, decode rooflines at 1.5B and 7B sizes; each prints "
                             "its own JSON line")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU engine")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    left_out = [kind for kind in args.leave_out.split(",") if kind]
    if left_out and args.impl == "ours":
        from einf_b200 import ops

        names = {"decode_attention": "paged_decode_attention_auto", "prefill_attention": "paged_prefill_attention",
                 "norms": "add_rmsnorm", "rotary": "rope_kv_write", "activation": "silu_mul"}
        for kind in left_out:
            setattr(ops, names[kind], lambda *a, **k: None)
        print(f"left out of every step: {left_out}; the line below is a diagnosis, not a benchmark value", file=sys.stderr)
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    if args.scenario == "default" and args.only == "all" and not left_out:
        line = run_ours(args)
        if not args.skip_other_sizes:
            import gc

            import torch

            gc.collect()
            torch.cuda.empty_cache()
            line["points"].update(other_sizes_points(args))
            line["config"]["sizes_1.5b"] = "L28 H1536 Hq12 Hkv2 D128 I8960 V151936 tied"
            line["config"]["sizes_7b"] = "L28 H3584 Hq28 Hkv4 D128 I18944 V152064 untied"
        print(json.dumps(line))
        return 0
    scenarios = {"1.5b-mixed": run_mixed_15b, "7b-preempt": run_preempt_7b, "decode-sizes": run_decode_sizes, "decode-contexts": run_decode_contexts, "decode-attention": run_decode_attention, "prefill-sizes": run_prefill_sizes,
                 "sampling": run_sampling, "prefill-attention": run_prefill_attention}
    if args.scenario in scenarios:
        line = scenarios[args.scenario](args)
        if left_out:
            line["left_out"] = left_out
        print(json.dumps(line))
    else:
        line = run_ours(args)
        if left_out:
            line = {"left_out": left_out, **{k: v for k, v in line.items() if k in ("only", "batch", "ms_per_step", "ms", "tokens")},
                    "prefill_ms": (line.get("prefill") or {}).get("ms")}
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
