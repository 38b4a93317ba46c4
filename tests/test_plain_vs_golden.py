"""The plain implementation against the reference's own model code, and against itself (no GPU)."""
from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file

import plain_impl
from conftest import TINY

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model(name, tiny_folders):
    golden = load_file(str(GOLDEN / f"tiny_{name}.safetensors"))
    config, tensors = plain_impl.read_folder(tiny_folders[name])
    logits = plain_impl.forward(config, tensors, golden["tokens"].tolist())
    torch.testing.assert_close(logits, golden["logits"], rtol=1e-5, atol=1e-5)


def test_parts_one_by_one():
    torch.manual_seed(0)
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    normed = plain_impl.rms_norm(x, w, 1e-5)
    expected = w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    torch.testing.assert_close(normed, expected)
    # rotation keeps lengths and turns pairs (i, i + D/2) by position * theta^(-2i/D)
    cos, sin = plain_impl.rope_cos_sin([0, 3], 8, 100.0)
    v = torch.randn(2, 1, 8)
    r = plain_impl.apply_rope(v, cos, sin)
    torch.testing.assert_close(r[0], v[0])
    torch.testing.assert_close(r.norm(dim=-1), v.norm(dim=-1))
    angle = 3 * 100.0 ** (-2 / 8)
    torch.testing.assert_close(
        r[1, 0, 1], v[1, 0, 1] * torch.cos(torch.tensor(angle)) - v[1, 0, 5] * torch.sin(torch.tensor(angle))
    )
    # causal: the first query sees only itself; a window of 2 drops older keys
    q, k, v = torch.randn(4, 2, 8), torch.randn(4, 1, 8), torch.randn(4, 1, 8)
    out = plain_impl.causal_attention(q, k, v, 0.3)
    torch.testing.assert_close(out[0], v[0].expand(2, 8))
    windowed = plain_impl.causal_attention(q, k, v, 0.3, window=2)
    two = plain_impl.causal_attention(q[2:4], k[2:4], v[2:4], 0.3)
    torch.testing.assert_close(windowed[3], two[1])
    # swiglu
    g, u, d = torch.randn(6, 12), torch.randn(6, 12), torch.randn(12, 6)
    torch.testing.assert_close(
        plain_impl.swiglu(x, g, u, d), (torch.nn.functional.silu(x @ g.T) * (x @ u.T)) @ d.T
    )


def test_later_tokens_do_not_change_earlier_logits(tiny_folders):
    config, tensors = plain_impl.read_folder(tiny_folders["C"])
    tokens = list(range(3, 40))
    full = plain_impl.forward(config, tensors, tokens)
    part = plain_impl.forward(config, tensors, tokens[:20])
    torch.testing.assert_close(full[:20], part, rtol=1e-5, atol=1e-6)


def test_window_changes_only_windowed_layers(tiny_folders):
    config, tensors = plain_impl.read_folder(tiny_folders["C"])
    tokens = list(range(5, 35))
    windowed = plain_impl.forward(config, tensors, tokens)
    unwindowed = plain_impl.forward({**config, "use_sliding_window": False}, tensors, tokens)
    # up to the window's length the two agree; beyond it they differ
    torch.testing.assert_close(windowed[:11], unwindowed[:11], rtol=1e-5, atol=1e-6)
    assert (windowed[20:] - unwindowed[20:]).abs().max() > 1e-4


def test_sampling_reference():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0, 0.5])
    assert plain_impl.sample_token(logits, 0.0) == 1  # first of the ties
    probabilities = plain_impl.filtered_probabilities(logits, 1.0, top_k=2)
    assert probabilities.nonzero().flatten().tolist() == [1, 2]
    probabilities = plain_impl.filtered_probabilities(torch.tensor([3.0, 2.0, 1.0, 0.0]), 1.0, top_p=0.7)
    assert probabilities.nonzero().flatten().tolist() == [0, 1]  # 0.64 < 0.7: the crossing token stays
    probabilities = plain_impl.filtered_probabilities(torch.tensor([3.0, 2.0, 1.0, 0.0]), 1.0, min_p=0.2)
    assert probabilities.nonzero().flatten().tolist() == [0, 1]
    u = [plain_impl.uniform_from_key(7, i) for i in range(2000)]
    assert 0.45 < sum(u) / len(u) < 0.55 and min(u) >= 0 and max(u) < 1
    assert plain_impl.uniform_from_key(7, 3) == plain_impl.uniform_from_key(7, 3)
    draws = [plain_impl.sample_token(logits, 0.8, seed=1, sample_index=i) for i in range(3000)]
    share = draws.count(1) / len(draws)
    expected = float(torch.softmax(logits / 0.8, -1)[1])
    assert abs(share - expected) < 0.03
