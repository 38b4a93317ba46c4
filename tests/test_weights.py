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


def test_parts_nested_in_any_category_have_their_tensors_expected_and_built():
    """A feed-forward that nests a norm of its own (with a weight), and that norm's name is not a
    category: its tensors are expected and loaded like any others, and it is built from them."""
    from einf_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
    from einf_b200.parts import FeedForward, Runtime, build_nested, build_part, register_part
    from einf_b200.parts.base import walk_part_specs

    @register_part("feed_forward", "sandwich_for_tests")
    class Sandwich(FeedForward):
        @classmethod
        def tensor_specs(cls, spec):
            return {"up.weight": TensorSpec((spec["inner"], spec["hidden_size"]))}

        @classmethod
        def nested_parts(cls, spec):
            return {"inner_norm": "norm"}

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec, tensors, runtime)
            self.inner_norm = build_nested("norm", spec["inner_norm"], tensors, runtime)

    inner = PartSpec("rmsnorm", {"size": 6, "eps": 1e-5}, "l0.mlp.inner_norm.")
    sandwich = PartSpec("sandwich_for_tests", {"hidden_size": 8, "inner": 6, "inner_norm": inner}, "l0.mlp.")
    assert [(c, s.kind) for c, s in walk_part_specs("feed_forward", sandwich)] == [
        ("feed_forward", "sandwich_for_tests"), ("norm", "rmsnorm")]
    norm = {"size": 8, "eps": 1e-5}
    attention = PartSpec("attention", {"hidden_size": 8, "num_heads": 1, "num_kv_heads": 1, "head_size": 16,
                                       "scale": 0.25, "position": PartSpec("none", {})}, "l0.attn.")
    spec = ModelSpec(
        8, 11, PartSpec("embedding", {"vocab_size": 11, "hidden_size": 8}, "embed."),
        (LayerSpec("prenorm", {"mixer": attention, "feed_forward": sandwich,
                               "mixer_norm": PartSpec("rmsnorm", norm, "l0.n1."),
                               "feed_forward_norm": PartSpec("rmsnorm", norm, "l0.n2.")}),),
        (ScheduleEntry(0),), PartSpec("rmsnorm", norm, "final."),
        PartSpec("linear_head", {"vocab_size": 11, "hidden_size": 8, "tied_to": "embed.weight"}, "head."))
    expected, _ = expected_tensors(spec)
    assert expected["l0.mlp.inner_norm.weight"].shape == (6,) and "l0.mlp.up.weight" in expected
    tensors = random_tensors(expected, 3, 0.02, 0.05, torch.bfloat16, "cpu")
    part = build_part("feed_forward", sandwich, tensors, Runtime(torch.float32, torch.device("cpu")))
    assert torch.equal(part.inner_norm.weight, tensors["l0.mlp.inner_norm.weight"].float())
    # a nested spec under a name that is no category, and no nested_parts() to say which it is
    @register_part("feed_forward", "unnamed_nesting_for_tests")
    class Unnamed(FeedForward):
        pass

    with pytest.raises(ValueError, match="no category"):
        list(walk_part_specs("feed_forward", PartSpec("unnamed_nesting_for_tests", {"inner_norm": inner})))
