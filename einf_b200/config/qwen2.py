"""Typed configuration of the Qwen2 / Qwen2.5 dense decoder.

Keys and their use follow ``QwenConfig`` of the reference
(``src/einf/executors/torch/qwen.py:60-122``): thirteen required keys, the
head size derived as ``hidden_size // num_attention_heads`` (``qwen.py:85-87``)
unless ``head_dim`` is given, ``hidden_act`` must be ``silu`` (``qwen.py:138-139``),
query heads a multiple of key/value heads (``qwen.py:335-338``), Q/K/V
projections with bias and O without (``qwen.py:353-360``).

The reference never reads ``use_sliding_window``, ``sliding_window`` or
``max_window_layers`` (``qwen.py:93-117``): with ``use_sliding_window`` false,
the value every Qwen2.5 folder carries, this class describes exactly what the
reference computes.  With it true, layers from ``max_window_layers`` on attend
to the last ``sliding_window`` keys only, as the keys say.

``rope_scaling`` (YaRN, NTK, linear ...) and ``partial_rotary_factor`` are not
computed here; the reference ignores them without a word (``qwen.py:93-117``,
``model_runner.py:42-78``: plain rotary angles over the whole head), this class
refuses any value but null / 1.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import ConfigError, ModelConfig
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclasses.dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    architecture: ClassVar[str] = "Qwen2ForCausalLM"
    refused_keys: ClassVar[dict[str, tuple]] = {
        "rope_scaling": (None,),
        "partial_rotary_factor": (None, 1, 1.0),
    }

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    rms_norm_eps: float
    hidden_act: str
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: int
    eos_token_id: int
    head_dim: int | None = None
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    initializer_range: float = 0.02

    def validate(self) -> None:
        def positive(name: str) -> None:
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")

        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "max_position_embeddings",
        ):
            positive(name)
        if self.head_dim is None and self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size {self.hidden_size} is not a multiple of "
                f"num_attention_heads {self.num_attention_heads} and no head_dim is given"
            )
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_size % 2:
            raise ConfigError(f"head size {self.head_size} must be even for rotary encoding")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported; Qwen2 uses 'silu'")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if self.use_sliding_window:
            if not isinstance(self.sliding_window, int) or self.sliding_window <= 0:
                raise ConfigError(
                    "use_sliding_window is true but sliding_window is "
                    f"{self.sliding_window!r}; it must be a positive integer"
                )

    # Derived sizes -----------------------------------------------------
    @property
    def head_size(self) -> int:
        if self.head_dim is not None:
            return self.head_dim
        return self.hidden_size // self.num_attention_heads

    @property
    def eos_token_ids(self) -> tuple[int, ...]:
        return (self.eos_token_id,)

    @property
    def init_std(self) -> float:
        return self.initializer_range

    def window_of_layer(self, layer: int) -> int | None:
        """Number of keys layer ``layer`` may see, or None for all of them."""
        if not self.use_sliding_window:
            return None
        first_windowed = self.max_window_layers if self.max_window_layers is not None else 0
        return self.sliding_window if layer >= first_windowed else None

    # The part-by-part description --------------------------------------
    def model_spec(self) -> ModelSpec:
        norm = {"size": self.hidden_size, "eps": self.rms_norm_eps}
        layers = []
        for index in range(self.num_hidden_layers):
            prefix = f"model.layers.{index}."
            attention = PartSpec(
                "attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_size": self.head_size,
                    "qkv_bias": True,
                    "out_bias": False,
                    "scale": self.head_size ** -0.5,
                    "window": self.window_of_layer(index),
                    "position": PartSpec(
                        "rope",
                        {
                            "rotary_dim": self.head_size,
                            "theta": self.rope_theta,
                            "max_position": self.max_position_embeddings,
                        },
                    ),
                },
                prefix + "self_attn.",
            )
            mlp = PartSpec(
                "gated_mlp",
                {
                    "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size,
                    "activation": self.hidden_act,
                },
                prefix + "mlp.",
            )
            layers.append(
                LayerSpec(
                    "prenorm",
                    {
                        "mixer": attention,
                        "feed_forward": mlp,
                        "mixer_norm": PartSpec("rmsnorm", norm, prefix + "input_layernorm."),
                        "feed_forward_norm": PartSpec(
                            "rmsnorm", norm, prefix + "post_attention_layernorm."
                        ),
                    },
                )
            )
        return ModelSpec(
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            embedding=PartSpec(
                "embedding",
                {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
                "model.embed_tokens.",
            ),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", norm, "model.norm."),
            head=PartSpec(
                "linear_head",
                {
                    "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size,
                    "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None,
                },
                "lm_head.",
            ),
        )
