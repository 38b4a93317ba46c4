"""Weights by name, the error that lists every fault, and the random mode (no GPU)."""
import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY, make_folder
from einf_b200.config import config_from_dict
from einf_b200.parts import expected_tensors
from einf_b200.weights import WeightsError, kept_dtype, load_tensors, random_tensors


def _expected(name):
    return expected_tensors(config_from_dict(TINY[name]).model_spec())


def test_random_folder_round_trip(tmp_path):
    folder = make_folder("B", tmp_path / "b")
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 96
    expected, optional = _expected("B")
    tensors = load_tensors(folder, expected, optional=optional)
    assert set(tensors) == set(expected)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert tensors["lm_head.weight"].shape == (384, 96)
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05
    matrix = tensors["model.layers.1.mlp.down_proj.weight"].float()
    assert 0.015 < float(matrix.std()) < 0.025


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = load_file(str(make_folder("A", tmp_path / "a1", seed=5) / "model.safetensors"))
    b = load_file(str(make_folder("A", tmp_path / "a2", seed=5) / "model.safetensors"))
    c = load_file(str(make_folder("A", tmp_path / "a3", seed=6) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert "lm_head.weight" not in a  # tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder("B", tmp_path / "b")
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    del tensors["lm_head.weight"]
    del tensors["model.layers.2.self_attn.k_proj.bias"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.norm.weight"] = torch.zeros(95, dtype=torch.bfloat16)
    tensors["model.layers.1.mlp.up_proj.weight"] = torch.zeros((96, 160), dtype=torch.bfloat16)
    save_file(tensors, str(path))
    expected, optional = _expected("B")
    with pytest.raises(WeightsError) as info:
        load_tensors(folder, expected, optional=optional)
    error = info.value
    assert set(error.missing) == {"lm_head.weight", "model.layers.2.self_attn.k_proj.bias"}
    assert error.unexpected == ("model.layers.0.extra.weight",)
    assert {name for name, _, _ in error.wrong_shape} == {"model.norm.weight", "model.layers.1.mlp.up_proj.weight"}
    text = str(error)
    for needle in ("missing (2)", "unexpected (1)", "model.norm.weight is [95], expected [96]", "[96, 160], expected [160, 96]"):
        assert needle in text


def test_tied_folder_may_store_the_output_matrix(tmp_path):
    folder = make_folder("A", tmp_path / "a")
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(path))
    expected, optional = _expected("A")
    assert "lm_head.weight" in optional and "lm_head.weight" not in expected
    load_tensors(folder, expected, optional=optional)


def test_storage_policy(tmp_path):
    assert kept_dtype(torch.float32) == torch.float32
    assert kept_dtype(torch.float16) == torch.bfloat16
    assert kept_dtype(torch.bfloat16) == torch.bfloat16
    assert kept_dtype(torch.int64) == torch.int32
    folder = make_folder("A", tmp_path / "a")
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4  # not representable in bfloat16
    save_file(tensors, str(path))
    expected, optional = _expected("A")
    loaded = load_tensors(folder, expected, optional=optional)
    assert loaded["model.norm.weight"].dtype == torch.float32
    assert torch.equal(loaded["model.norm.weight"], tensors["model.norm.weight"])
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_integer_tensor_where_a_float_is_expected(tmp_path):
    folder = make_folder("A", tmp_path / "a")
    path = folder / "model.safetensors"
    tensors = load_file(str(path))
    tensors["model.norm.weight"] = torch.ones(64, dtype=torch.int64)
    save_file(tensors, str(path))
    expected, optional = _expected("A")
    with pytest.raises(WeightsError, match="wrong kind: model.norm.weight"):
        load_tensors(folder, expected, optional=optional)


def test_missing_folder_and_sharded_folder(tmp_path):
    expected, optional = _expected("A")
    with pytest.raises(FileNotFoundError):
        load_tensors(tmp_path, expected)
    folder = make_folder("A", tmp_path / "a")
    tensors = load_file(str(folder / "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    weight_map = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, k in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    loaded = load_tensors(folder, expected, optional=optional)
    assert all(torch.equal(loaded[k], tensors[k]) for k in names)


def test_random_tensors_follow_roles():
    expected, _ = _expected("C")
    tensors = random_tensors(expected, seed=3, std=0.03)
    assert tensors["model.layers.3.self_attn.q_proj.bias"].shape == (288,)
    assert abs(float(tensors["model.embed_tokens.weight"].float().std()) - 0.03) < 0.003
