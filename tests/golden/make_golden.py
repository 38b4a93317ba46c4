"""Make tests/golden/*.safetensors: logits of the reference's own model code.

Runs ``QwenModelRunner`` of mon3stera/einf on the CPU in float32 on the tiny
random models A and B (the reference cannot express C: it derives the head size
and reads no window key).  The reference package needs its compiled control
module only for scheduling, so a stub of ``einf._control`` with the thirteen
names ``einf/__init__.py`` imports stands in; the model code itself is imported
unmodified from ``--reference/src``.  Weights are the engine's random-weights
mode with the tests' seeds, which the test regenerates; the prompt is stored
beside the logits.

Each prompt runs twice: whole, and in portions of 6 over shuffled pages; both
must agree before the file is written.

    python tests/golden/make_golden.py --reference /path/to/einf
"""
from __future__ import annotations

import argparse
import sys
import tempfile
import types
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from conftest import TINY, TINY_PAGE, make_folder, random_tokens  # noqa: E402

STUB_NAMES = (
    "BatchPlan", "CompletionReason", "ExecutionResult", "RequestExecutionResult", "RequestSpec",
    "RequestState", "RequestView", "SamplingParams", "SamplingPlan", "ScheduledBatch",
    "ScheduledRequest", "Scheduler", "WorkType",
)
PROMPT_LEN = {"A": 13, "B": 30}


def reference_logits(name: str, folder: Path, tokens: list[int], portions: list[int], pages: list[int]):
    from einf.cache.storage import KVCacheGeometry, TorchKVCacheStorage
    from einf.executors.torch.input import ModelInput
    from einf.executors.torch.qwen import QwenConfig, QwenModelRunner

    config = QwenConfig.from_json(folder / "config.json")
    page = TINY_PAGE[name]
    cache = TorchKVCacheStorage(
        KVCacheGeometry(config.num_hidden_layers, 16, page, config.num_key_value_heads, config.head_dim),
        dtype=torch.float32, device=torch.device("cpu"), use_custom_ops=False,
    )
    torch.set_default_dtype(torch.float32)
    runner = QwenModelRunner(config, cache=cache).eval()
    runner.load_checkpoint(folder)
    runner = runner.float()
    rows = []
    start = 0
    table = torch.tensor([pages], dtype=torch.int64)
    with torch.inference_mode():
        for length in portions:
            position = torch.arange(start, start + length)
            slot = torch.tensor([pages[p // page] * page + p % page for p in position.tolist()])
            model_input = ModelInput(
                input_token_ids=torch.tensor(tokens[start:start + length]),
                position=position,
                slot_mapping=slot,
                query_start_loc=torch.tensor([0, length]),
                block_tables=table,
                context_lens=torch.tensor([start + length]),
                query_start_loc_host=(0, length),
                context_lens_host=(start + length,),
            )
            rows.append(runner.forward(model_input).logits.float())
            start += length
    return torch.cat(rows)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    args = parser.parse_args()
    stub = types.ModuleType("einf._control")
    for attribute in STUB_NAMES:
        setattr(stub, attribute, type(attribute, (), {}))
    sys.modules["einf._control"] = stub
    sys.path.insert(0, str(args.reference / "src"))
    for name in ("A", "B"):
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_folder(name, Path(tmp) / name)
            vocab = TINY[name]["vocab_size"]
            tokens = random_tokens(vocab, PROMPT_LEN[name], seed=100 + ord(name))
            page = TINY_PAGE[name]
            needed = -(-len(tokens) // page)
            whole = reference_logits(name, folder, tokens, [len(tokens)], list(range(needed)))
            shuffled = [7, 2, 9, 4, 11, 0, 5, 13][:needed]
            portions = [6] * (len(tokens) // 6) + ([len(tokens) % 6] if len(tokens) % 6 else [])
            cut = reference_logits(name, folder, tokens, portions, shuffled)
            difference = float((whole - cut).abs().max())
            assert difference < 1e-5, difference
            save_file(
                {"tokens": torch.tensor(tokens, dtype=torch.int32), "logits": whole.contiguous()},
                str(HERE / f"tiny_{name}.safetensors"),
            )
            print(f"tiny {name}: logits {tuple(whole.shape)}, whole vs portions {difference:.2e}")


if __name__ == "__main__":
    main()
