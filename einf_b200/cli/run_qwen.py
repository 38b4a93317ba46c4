"""Command line: run a Qwen2.5 model folder (or random weights) to generated tokens.

Options keep the reference's names and meanings where it has them
(``scripts/run_qwen.py:33-74``): ``--model-dir``, ``--prompt``, ``--max-new-len``,
``--dtype``, ``--block-len``, ``--num-blocks``, ``--max-batch-len``,
``--max-prefill-chunk-len``.  Backend switches of the reference
(``--flash-attention``, ``--attn-backend`` ...) do not exist: there is one backend.
Added here: ``--prompt-ids`` (no tokenizer needed), ``--random-weights`` with
``--config`` and ``--seed``, ``--policy``, and the sampling parameters.
Prints ``completion_reason``, timings, ``prompt_ids``, ``generated_ids`` and, when
a tokenizer is at hand, ``generated_text``, one ``key: value`` a line as the
reference does (``run_qwen.py:144,251-256``).

``--compare-reference`` stands where the reference has ``--compare-hf``
(``run_qwen.py:258-288``): the same prompt is generated greedily a second time
by this engine's true 32-bit path (32-bit weights, cache and products, the whole
prompt in one step, no CUDA graphs), and ``reference_generated_ids`` and
``tokens_equal`` are printed.  Model code of an installed package is not used.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from pathlib import Path

DEFAULT_MODEL_DIR = Path(os.environ.get("EINF_MODEL_DIR", str(Path.home() / "models" / "Qwen2.5-0.5B")))


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="run_qwen", description="Run Qwen2.5 through einf_b200")
    parser.add_argument("--model-dir", type=Path, default=DEFAULT_MODEL_DIR)
    parser.add_argument("--prompt", default="The capital of France is")
    parser.add_argument("--prompt-ids", default=None, help="comma-separated token ids; no tokenizer is needed then")
    parser.add_argument("--max-new-len", type=int, default=8)
    parser.add_argument("--dtype", choices=("float32", "bfloat16"), default="bfloat16")
    parser.add_argument("--block-len", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=256)
    parser.add_argument("--max-batch-len", type=int, default=128)
    parser.add_argument("--max-prefill-chunk-len", type=int, default=128)
    parser.add_argument("--policy", choices=("fcfs", "decode_first"), default="fcfs")
    parser.add_argument("--decode-lookahead", type=int, default=1,
                        help="decode steps per report to the host (not an option of the reference; 1 is its behaviour)")
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=None)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--sampler-seed", type=int, default=0)
    parser.add_argument("--random-weights", action="store_true",
                        help="write a random model folder from --config (or --model-dir/config.json) and run it")
    parser.add_argument("--config", type=Path, default=None, help="a config.json for --random-weights")
    parser.add_argument("--seed", type=int, default=0, help="seed of --random-weights")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--compare-reference", action="store_true",
                        help="generate again on the 32-bit path (whole prompt, no graphs) and print tokens_equal")
    parser.add_argument("--device", default="cuda:0")
    return parser.parse_args(argv)


def _tokenizer(model_dir: Path):
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(str(model_dir), local_files_only=True)
    except Exception:
        return None


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.compare_reference and args.temperature != 0.0:
        print("--compare-reference compares greedy tokens: leave --temperature at 0", file=sys.stderr)
        return 2
    from ..config import EngineConfig, load_config
    from ..engine import Engine
    from ..sampling import SamplingParams
    from ..weights import write_random_model

    scratch = None
    model_dir = args.model_dir
    if args.random_weights:
        config = load_config(args.config if args.config else model_dir)
        scratch = tempfile.TemporaryDirectory(prefix="einf_b200_random_")
        model_dir = write_random_model(Path(scratch.name) / "model", config, args.seed)
    tokenizer = None
    if args.prompt_ids is not None:
        prompt_ids = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    else:
        tokenizer = _tokenizer(args.model_dir)
        if tokenizer is None:
            print("no tokenizer in the model folder: give --prompt-ids", file=sys.stderr)
            return 2
        prompt_ids = list(tokenizer(args.prompt)["input_ids"])
    started = time.perf_counter()
    engine = Engine.from_folder(
        model_dir,
        EngineConfig(
            dtype=args.dtype, block_len=args.block_len, num_blocks=args.num_blocks,
            max_batch_len=args.max_batch_len, max_prefill_chunk_len=args.max_prefill_chunk_len,
            policy=args.policy, device=args.device, decode_lookahead=args.decode_lookahead,
        ),
        eos_token_ids=() if args.ignore_eos else None,
    )
    load_s = time.perf_counter() - started
    sampling = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, seed=args.sampler_seed
    )
    request_id = engine.submit(prompt_ids, args.max_new_len, sampling, request_id="qwen")
    started = time.perf_counter()
    engine.run_until_idle()
    gen_s = time.perf_counter() - started
    view = engine.request(request_id)
    if view.state == "failed":
        print(f"request failed: {view.error}", file=sys.stderr)
        return 1
    generated = list(view.generated_token_ids)
    print(f"completion_reason: {view.completion_reason}")
    print(f"load_s={load_s:.3f} gen_s={gen_s:.3f} tokens_per_gen_s={len(generated) / max(gen_s, 1e-9):.2f}")
    print(f"prompt_ids: {json.dumps(prompt_ids)}")
    print(f"generated_ids: {json.dumps(generated)}")
    if tokenizer is not None:
        print(f"generated_text: {tokenizer.decode(generated)!r}")
    if args.compare_reference:
        del engine
        total = len(prompt_ids) + args.max_new_len
        reference = Engine.from_folder(
            model_dir,
            EngineConfig(
                dtype="float32", block_len=args.block_len, num_blocks=-(-total // args.block_len) + 1,
                max_batch_len=max(total, 8), max_prefill_chunk_len=max(total, 8), policy="fcfs",
                device=args.device, decode_lookahead=1, use_cuda_graphs=False,
            ),
            eos_token_ids=() if args.ignore_eos else None,
        )
        reference_ids = reference.generate([prompt_ids], args.max_new_len)[0]
        print(f"reference_generated_ids: {json.dumps(reference_ids)}")
        print(f"tokens_equal: {generated == reference_ids}")
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
