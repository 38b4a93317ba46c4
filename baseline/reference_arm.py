"""The reference arm of ``bench.py``: mon3stera/einf's own executor on this GPU.

Nothing of ``einf_b200`` is imported here.  The arm runs the unmodified Python
tree of the reference (a copy of its ``pyproject.toml`` and ``src/`` under
``baseline/_ref``): ``TorchExecutor.execute`` (``src/einf/executors/torch/
executor.py:28-117``) over ``QwenModelRunner`` (``qwen.py:595-790``),
``TorchKVCacheStorage`` (``src/einf/cache/storage.py:16-182``), its input pool
and its sampler, timed as ``benchmarks/benchmark_decode_only.py:302-324`` does.

What is not the reference's: its control plane is a Rust extension
(``einf._control``) that cannot be built without a Rust toolchain, so the
plans its executor consumes are made here by hand (plain objects with the
fields ``execution_plan.rs:12-29`` gives them: every request decodes one token
per step, pages are handed out in order), and the result classes are
placeholders.  The scheduler is therefore not in the timed loop; the reference's
own benchmark has it there.  Weights are drawn N(0, 0.02) under the checkpoint's
tensor names and loaded through the reference's ``load_state_dict``.

The reference has three attention back ends for decoding
(``scripts/run_qwen.py:48-57``): its default (keys and values gathered per
request, PyTorch's scaled-dot-product attention), ``--paged-decode-attention``
(its own split-KV kernel) and ``--attn-backend flashinfer`` (with its decode
CUDA graph).  Each is tried; one that cannot run here is recorded with the
exception it raised; the headline is the fastest that ran.
"""
from __future__ import annotations

import statistics
import sys
import time
import types
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent.parent
REFERENCE_TREE = ROOT / "baseline" / "_ref"

#: names ``src/einf/__init__.py:3-17`` imports from the Rust extension
CONTROL_NAMES = (
    "BatchPlan", "CompletionReason", "ExecutionResult", "RequestExecutionResult", "RequestSpec", "RequestState",
    "RequestView", "SamplingParams", "SamplingPlan", "ScheduledBatch", "ScheduledRequest", "Scheduler", "WorkType",
)


class ReferenceUnavailable(RuntimeError):
    pass


def _placeholder(name: str) -> type:
    def __init__(self, *args, **kwargs):
        self.args = args
        self.__dict__.update(kwargs)

    return type(name, (), {"__init__": __init__})


def import_reference(tree: Path = REFERENCE_TREE) -> None:
    """Make ``import einf`` work from the copied tree, with placeholders for the Rust module."""
    if not (tree / "src" / "einf" / "__init__.py").is_file():
        raise ReferenceUnavailable(
            f"no copy of the reference's Python tree at {tree} (copy its pyproject.toml and src/ there)"
        )
    if "einf._control" not in sys.modules:
        stub = types.ModuleType("einf._control")
        for name in CONTROL_NAMES:
            setattr(stub, name, _placeholder(name))
        sys.modules["einf._control"] = stub
    path = str(tree / "src")
    if path not in sys.path:
        sys.path.insert(0, path)
    # The reference's kernels include CUTLASS from a git submodule at third_party/cutlass
    # (ops/loader.py:64-69); the same headers come with a package of this image.
    target = tree / "third_party" / "cutlass" / "include"
    if not (target / "cute" / "tensor.hpp").is_file():
        for entry in sys.path:
            candidate = Path(entry) / "flashinfer" / "data" / "cutlass" / "include"
            if (candidate / "cute" / "tensor.hpp").is_file():
                target.parent.mkdir(parents=True, exist_ok=True)
                if target.is_symlink() or target.exists():
                    target.unlink()
                target.symlink_to(candidate, target_is_directory=True)
                break


def _random_state(config, torch, device, dtype, seed: int) -> dict:
    """Random tensors under the checkpoint's names (``qwen.py:698-735`` loads them)."""
    generator = torch.Generator(device=device).manual_seed(seed)
    h, i, v = config.hidden_size, config.intermediate_size, config.vocab_size
    q, kv = config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim

    def normal(*shape):
        return (torch.randn(shape, generator=generator, device=device, dtype=torch.float32) * 0.02).to(dtype)

    def scale(n):
        return (1 + 0.05 * torch.randn(n, generator=generator, device=device, dtype=torch.float32)).to(dtype)

    state = {"model.embed_tokens.weight": normal(v, h), "model.norm.weight": scale(h)}
    for layer in range(config.num_hidden_layers):
        p = f"model.layers.{layer}."
        state[p + "input_layernorm.weight"] = scale(h)
        state[p + "post_attention_layernorm.weight"] = scale(h)
        for name, rows in (("q", q), ("k", kv), ("v", kv)):
            state[p + f"self_attn.{name}_proj.weight"] = normal(rows, h)
            state[p + f"self_attn.{name}_proj.bias"] = normal(rows)
        state[p + "self_attn.o_proj.weight"] = normal(h, q)
        state[p + "mlp.gate_proj.weight"] = normal(i, h)
        state[p + "mlp.up_proj.weight"] = normal(i, h)
        state[p + "mlp.down_proj.weight"] = normal(h, i)
    state["lm_head.weight"] = state["model.embed_tokens.weight"] if config.tie_word_embeddings else normal(v, h)
    return state


class _Plans:
    """Hand-made decode plans: what the Rust scheduler would hand the executor for ``batch``
    requests that each bring their last token, with pages handed out in order."""

    def __init__(self, batch: int, context: int, block_len: int, vocab: int, seed: int, room: int) -> None:
        """``context``: tokens each request holds before its first step here; ``room``: steps it
        may run (its block table covers that many more tokens)."""
        import random

        rng = random.Random(seed)
        self.block_len = block_len
        self.step_id = 0
        pages_each = -(-(context + room + 1) // block_len)
        params = SimpleNamespace(temperature=0.0, top_k=None, top_p=1.0, min_p=0.0, seed=0, stop_token_ids=())
        self.requests = []
        for index in range(batch):
            self.requests.append(SimpleNamespace(
                request_id=f"request-{index}",
                input_token_ids=[rng.randrange(3, vocab)],
                start_position=context,
                block_table=list(range(index * pages_each, (index + 1) * pages_each)),
                sampling_plan=SimpleNamespace(params=params, sample_index=0),
                need_sample=True,
                work_type="decode",
            ))
        self.num_blocks = batch * pages_each

    def plan(self):
        self.step_id += 1
        return SimpleNamespace(step_id=self.step_id, requests=tuple(self.requests))

    def apply(self, result) -> None:
        for request, outcome in zip(self.requests, result.request_results):
            request.input_token_ids = [int(outcome.generated_token_ids[0])]
            request.start_position += 1
            request.sampling_plan.sample_index += 1


def _build(cfg: dict, backend: str, num_blocks: int, block_len: int, torch, seed: int):
    from einf.cache.storage import KVCacheGeometry, TorchKVCacheStorage
    from einf.executors.torch.executor import TorchExecutor
    from einf.executors.torch.qwen import QwenConfig, QwenModelRunner

    device, dtype = torch.device("cuda:0"), torch.bfloat16
    config = QwenConfig.from_dict(cfg)
    # the page the reference's decode graph keeps for its padding rows is its last (qwen.py:681)
    cache = TorchKVCacheStorage(
        KVCacheGeometry(num_layers=config.num_hidden_layers, num_blocks=num_blocks + 1, block_len=block_len,
                        num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim),
        dtype=dtype, device=device,
    )
    cache.K.zero_()
    cache.V.zero_()
    previous = torch.get_default_dtype()
    torch.set_default_dtype(dtype)       # as scripts/run_qwen.py:84-108 constructs it
    try:
        runner = QwenModelRunner(
            config, cache=cache,
            use_paged_decode_attention=backend == "paged",
            use_flashinfer_attention=backend == "flashinfer",
            dtype=dtype,
        )
    finally:
        torch.set_default_dtype(previous)
    runner = runner.to(device=device, dtype=dtype).eval()
    runner.load_state_dict(_random_state(config, torch, device, dtype, seed), strict=True)
    executor = TorchExecutor(model_runner=runner, block_len=block_len, eos_token_id=-1, device=device)
    return config, runner, executor


def _time_decode(executor, plans: _Plans, steps: int, warmup: int, torch) -> dict:
    """As benchmarks/benchmark_decode_only.py:302-324: every step is execute + synchronize, wall
    clock around K steps; tokens come back to the host inside every step (the executor's own read)."""
    with torch.inference_mode():
        for _ in range(warmup):
            plans.apply(executor.execute(plans.plan()))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall = time.perf_counter()
        start.record()
        for _ in range(steps):
            result = executor.execute(plans.plan())
            torch.cuda.synchronize()
            plans.apply(result)
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
    batch = len(plans.requests)
    return {"device_ms_per_step": start.elapsed_time(end) / steps, "wall_ms_per_step": wall / steps * 1e3,
            "tokens_per_s": batch * steps / wall}


def _time_prefill(executor, cfg: dict, tokens: int, block_len: int, first_block: int, torch, repeats: int = 5) -> dict:
    import random

    rng = random.Random(1)
    ids = [rng.randrange(3, cfg["vocab_size"]) for _ in range(tokens)]
    params = SimpleNamespace(temperature=0.0, top_k=None, top_p=1.0, min_p=0.0, seed=0, stop_token_ids=())
    pages = -(-tokens // block_len)
    times = []
    with torch.inference_mode():
        for attempt in range(repeats + 2):
            request = SimpleNamespace(
                request_id="prefill", input_token_ids=ids, start_position=0,
                block_table=list(range(first_block, first_block + pages)),
                sampling_plan=SimpleNamespace(params=params, sample_index=0), need_sample=True, work_type="prefill")
            torch.cuda.synchronize()
            started = time.perf_counter()
            executor.execute(SimpleNamespace(step_id=10_000 + attempt, requests=(request,)))
            torch.cuda.synchronize()
            if attempt >= 2:
                times.append((time.perf_counter() - started) * 1e3)
    return {"ms": statistics.median(times), "tokens": tokens}


def h2d_bytes_per_decode_step(batch: int, context: int, block_len: int) -> int:
    """What ``ModelInputPool.build`` copies to the device for a step of ``batch`` single tokens
    (``input.py:197-213``): tokens, positions, slots, prefix sums, context lengths and block tables
    as 64-bit integers, the page list as 32-bit."""
    pages = -(-(context + 1) // block_len)
    return 8 * (3 * batch + (batch + 1) + batch + batch * pages) + 4 * batch * pages


def run_backend(cfg: dict, backend: str, batches, context: int, block_len: int, prefill_tokens: int, steps: int,
                warmup: int, clock_sampler=None, log=sys.stderr) -> dict:
    """One attention back end of the reference (``flashinfer``, ``paged`` or ``default``): its decode
    step at each batch size of ``batches`` (the first is the headline) near ``context`` tokens, and one
    prefill of ``prefill_tokens``."""
    import_reference()
    import torch

    if not torch.cuda.is_available():
        raise ReferenceUnavailable("no CUDA device")
    record: dict = {"backend": backend}
    started = time.perf_counter()
    for index, batch in enumerate(batches):
        print(f"[reference] {backend}: batch {batch}", file=log, flush=True)
        plans = _Plans(batch, context - steps - warmup, block_len, cfg["vocab_size"], seed=batch,
                       room=steps + warmup + 4)
        spare = -(-prefill_tokens // block_len) if index == 0 else 0
        _, runner, executor = _build(cfg, backend, plans.num_blocks + spare, block_len, torch, seed=0)
        if index == 0:
            record["setup_s"] = round(time.perf_counter() - started, 1)
            # one untimed pass first: kernels that are compiled at their first call
            with torch.inference_mode():
                for _ in range(2):
                    plans.apply(executor.execute(plans.plan()))
            torch.cuda.synchronize()
            record["first_steps_s"] = round(time.perf_counter() - started - record["setup_s"], 1)
            if clock_sampler is not None:
                clock_sampler.start()
        timed = _time_decode(executor, plans, steps, warmup, torch)
        if index == 0:
            if clock_sampler is not None:
                record["clocks"] = clock_sampler.stop()
            record.update(
                batch=batch,
                tokens_per_s_device=round(batch / timed["device_ms_per_step"] * 1e3, 1),
                tokens_per_s_wall=round(timed["tokens_per_s"], 1),
                device_ms_per_step=round(timed["device_ms_per_step"], 4),
                wall_ms_per_step=round(timed["wall_ms_per_step"], 4),
                h2d_bytes_per_step=h2d_bytes_per_decode_step(batch, context, block_len),
                d2h_bytes_per_step=8 * batch,
            )
            try:
                prefill = _time_prefill(executor, cfg, prefill_tokens, block_len, plans.num_blocks, torch)
                record["prefill"] = {"value": round(prefill_tokens / prefill["ms"] * 1e3, 1), "tokens": prefill_tokens,
                                     "ms": round(prefill["ms"], 3)}
            except Exception as error:  # noqa: BLE001 - recorded; the decode number stands
                record["prefill"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        else:
            record.setdefault("points", {})[f"decode_b{batch}"] = round(timed["tokens_per_s"], 1)
        del executor, runner
        torch.cuda.empty_cache()
    return record


def main(argv=None) -> int:
    """Child process of ``bench.py --impl reference``: one back end, one JSON line.  A back end that
    raises prints its exception as ``unavailable`` and exits 0; one that crashes the interpreter is
    seen by the parent as a non-zero exit."""
    import argparse
    import json

    parser = argparse.ArgumentParser()
    parser.add_argument("--backend", required=True, choices=("flashinfer", "paged", "default", "build-ops"))
    parser.add_argument("--config", required=True, help="the model's config.json keys, as JSON")
    parser.add_argument("--batches", default="8,1,64")
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--block-len", type=int, default=16)
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=4)
    args = parser.parse_args(argv)
    try:
        if args.backend == "build-ops":
            # the reference compiles its CUDA extension at the first call of any of its ops
            import_reference()
            started = time.perf_counter()
            from einf.executors.torch.ops.loader import load_custom_ops

            load_custom_ops()
            print(json.dumps({"backend": "build-ops", "seconds": round(time.perf_counter() - started, 1)}))
            return 0
        sys.path.insert(0, str(ROOT))
        from bench import ClockSampler   # nvidia-smi sampling only; nothing of the engine

        record = run_backend(json.loads(args.config), args.backend, [int(b) for b in args.batches.split(",")],
                             args.context, args.block_len, args.prefill_tokens, args.steps, args.warmup,
                             clock_sampler=ClockSampler())
    except Exception as error:  # noqa: BLE001 - the parent records why this back end did not run
        import traceback

        traceback.print_exc(file=sys.stderr)
        record = {"backend": args.backend, "unavailable": f"{type(error).__name__}: {error}"[:400]}
    print(json.dumps(record), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
