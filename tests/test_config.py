"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY
from einf_b200.config import (
    ConfigError, EngineConfig, ModelConfig, Qwen2Config, config_from_dict, known_architectures,
    load_config, register_architecture,
)
from einf_b200.config.specs import ModelSpec, PartSpec, ScheduleEntry


def test_qwen2_reads_its_own_keys():
    config = config_from_dict(TINY["A"])
    assert isinstance(config, Qwen2Config)
    assert config.head_size == 16 and config.eos_token_ids == (1,)
    spec = config.model_spec()
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    attention = spec.layers[0].parts["mixer"]
    assert attention.kind == "attention" and attention["num_kv_heads"] == 2
    assert attention["scale"] == pytest.approx(16 ** -0.5)
    assert attention["position"]["theta"] == 10000.0 and attention["window"] is None
    assert spec.head["tied_to"] == "model.embed_tokens.weight"
    assert spec.layers[1].parts["mixer_norm"]["eps"] == 1e-6


def test_every_size_comes_from_the_config():
    c = config_from_dict(TINY["C"])
    spec = c.model_spec()
    assert c.head_size == 48  # given, not hidden // heads
    assert [l.parts["mixer"]["window"] for l in spec.layers] == [None, None, 11, 11]
    assert spec.layers[0].parts["feed_forward"]["intermediate_size"] == 112
    assert c.init_std == 0.03
    b = config_from_dict(TINY["B"]).model_spec()
    assert b.head["tied_to"] is None and b.layers[2].parts["mixer"]["num_kv_heads"] == 1


def test_missing_keys_are_named():
    data = dict(TINY["A"])
    del data["rope_theta"], data["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps, rope_theta|rope_theta.*rms_norm_eps|rms_norm_eps.*rope_theta"):
        config_from_dict(data)


@pytest.mark.parametrize(
    "change, message",
    [
        (dict(num_key_value_heads=3), "not a multiple"),
        (dict(hidden_act="gelu"), "hidden_act"),
        (dict(hidden_size=66), "not a multiple"),
        (dict(use_sliding_window=True), "sliding_window"),
        (dict(vocab_size=0), "vocab_size"),
        (dict(head_dim=15), "even"),
    ],
)
def test_bad_values_are_refused(change, message):
    with pytest.raises(ConfigError, match=message):
        config_from_dict({**TINY["A"], **change})


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict({**TINY["A"], "architectures": ["NoSuchModel"]})
    assert "Qwen2ForCausalLM" in known_architectures()


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    config = load_config(tmp_path)
    assert config.vocab_size == 384
    assert config.to_dict()["architectures"] == ["Qwen2ForCausalLM"]
    assert config_from_dict(config.to_dict()) == config
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nothing")


def test_schedule_is_checked():
    part = PartSpec("rmsnorm", {"size": 4, "eps": 1e-6})
    with pytest.raises(ValueError, match="names layer 1"):
        ModelSpec(4, 8, part, (), (ScheduleEntry(1),), part, part)
    from einf_b200.config.specs import LayerSpec
    layer = LayerSpec("prenorm", {})
    with pytest.raises(ValueError, match="does not run before"):
        ModelSpec(4, 8, part, (layer,), (ScheduleEntry(0, cache_from=0),), part, part)
    with pytest.raises(ValueError, match="owns no cache"):
        ModelSpec(4, 8, part, (layer,), (ScheduleEntry(0), ScheduleEntry(0, 0), ScheduleEntry(0, 1)), part, part)
    ModelSpec(4, 8, part, (layer,), (ScheduleEntry(0), ScheduleEntry(0), ScheduleEntry(0, 0)), part, part)


def test_registering_an_architecture():
    import dataclasses

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture = "ToyForTests"
        width: int = 4

    register_architecture(ToyConfig)
    assert config_from_dict({"architectures": ["ToyForTests"], "width": 6}).width == 6
    with pytest.raises(ValueError, match="already registered"):
        @dataclasses.dataclass(frozen=True)
        class Other(ModelConfig):
            architecture = "ToyForTests"
        register_architecture(Other)


def test_engine_config_checks():
    assert EngineConfig().block_len == 16
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(policy="lifo")
    with pytest.raises(ValueError):
        EngineConfig(block_len=0)


def test_keys_that_are_not_computed_are_refused_by_name():
    """The reference reads neither key and would run plain rotary angles (qwen.py:93-117); a folder
    that sets one to anything but null / 1 would give wrong logits without a word."""
    base = dict(TINY["A"])
    for harmless in ({"rope_scaling": None}, {"partial_rotary_factor": 1.0}, {"some_other_key": {"a": 1}}):
        assert config_from_dict({**base, **harmless}).hidden_size == 64
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict({**base, "rope_scaling": {"type": "yarn", "factor": 4.0,
                                                    "original_max_position_embeddings": 32768}})
    with pytest.raises(ConfigError, match="partial_rotary_factor"):
        config_from_dict({**base, "partial_rotary_factor": 0.5})


def test_engine_config_sequence_limit():
    assert EngineConfig().max_sequence_len is None and EngineConfig(max_sequence_len=4096).max_sequence_len == 4096
    with pytest.raises(ValueError):
        EngineConfig(max_sequence_len=0)
