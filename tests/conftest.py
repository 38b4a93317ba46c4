"""Shared fixtures: tiny configurations, random model folders, trace builders."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Three tiny configurations that differ in every size and option.
TINY = {
    # 2 layers, tied, theta 1e4, page 4
    "A": dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=128,
        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6,
        hidden_act="silu", rope_theta=10000.0, max_position_embeddings=1024, tie_word_embeddings=True,
        bos_token_id=0, eos_token_id=1,
    ),
    # 3 layers, untied, one key/value head, theta 1e6, eps 1e-5, page 8
    "B": dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=160,
        num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, rms_norm_eps=1e-5,
        hidden_act="silu", rope_theta=1000000.0, max_position_embeddings=2048, tie_word_embeddings=False,
        bos_token_id=2, eos_token_id=3,
    ),
    # 4 layers, sizes that are no power of two, head size given (48 != 80 / 6), the last two
    # layers see a window of 11 keys, page 16
    "C": dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=331, hidden_size=80, intermediate_size=112,
        num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
        rms_norm_eps=3e-6, hidden_act="silu", rope_theta=500000.0, max_position_embeddings=4096,
        tie_word_embeddings=True, bos_token_id=5, eos_token_id=7, use_sliding_window=True,
        sliding_window=11, max_window_layers=2, initializer_range=0.03,
    ),
}
TINY_PAGE = {"A": 4, "B": 8, "C": 16}
TINY_SEED = {"A": 0, "B": 1, "C": 2}


def make_folder(name: str, folder: Path, seed: int | None = None) -> Path:
    from einf_b200.config import config_from_dict
    from einf_b200.weights import write_random_model

    config = config_from_dict(TINY[name])
    return write_random_model(folder, config, TINY_SEED[name] if seed is None else seed)


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """One random model folder per tiny configuration, in a temporary place."""
    base = tmp_path_factory.mktemp("models")
    return {name: make_folder(name, base / name) for name in TINY}


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


# Two layers each at the layer sizes of the family's models: what the tensor-core kernels are tuned
# for.  0.5B: head size 64 and the real vocabulary (no power of two); 1.5B: head size 128; 7B: seven
# query heads per key/value head at head size 128, the widest products, an output matrix of its own.
# The two larger ones have a small vocabulary (no power of two) to keep the plain model cheap.
_QWEN25 = dict(
    architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, rms_norm_eps=1e-6, hidden_act="silu",
    rope_theta=1000000.0, max_position_embeddings=32768,
)
SIZED = {
    "0.5b": dict(_QWEN25, vocab_size=151936, hidden_size=896, intermediate_size=4864, num_attention_heads=14,
                 num_key_value_heads=2, tie_word_embeddings=True, bos_token_id=151643, eos_token_id=151643),
    "1.5b": dict(_QWEN25, vocab_size=3001, hidden_size=1536, intermediate_size=8960, num_attention_heads=12,
                 num_key_value_heads=2, tie_word_embeddings=True, bos_token_id=1, eos_token_id=2),
    "7b": dict(_QWEN25, vocab_size=2003, hidden_size=3584, intermediate_size=18944, num_attention_heads=28,
               num_key_value_heads=4, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2),
}
SIZED_SEED = {"0.5b": 4, "1.5b": 5, "7b": 6}


@pytest.fixture(scope="session")
def sized_folders(tmp_path_factory):
    """``folder(name)``: a random two-layer model folder at the layer sizes of ``SIZED[name]``, written
    once per session into a temporary place when a test first asks for it."""
    base = tmp_path_factory.mktemp("sized_models")
    made: dict[str, Path] = {}

    def folder(name: str) -> Path:
        if name not in made:
            from einf_b200.config import config_from_dict
            from einf_b200.weights import write_random_model

            made[name] = write_random_model(base / name, config_from_dict(SIZED[name]), SIZED_SEED[name])
        return made[name]

    return folder
