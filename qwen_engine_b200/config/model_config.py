"""Typed model configurations read from a model folder's ``config.json``.

Every size and constant of a model comes from the keys of its own
``config.json``; nothing in the code stands in for them.  The only defaults
are the ones the reference's ``Qwen3Config`` has
(src/models/qwen3/config.py:6-19) and its ``from_hf_config``
(src/models/qwen3/config.py:22-38), which apply when a key is absent.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
from dataclasses import dataclass
from typing import Any, ClassVar, Optional


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses are dataclasses whose field names are the ``config.json`` keys.
    ``architecture`` names the registry entry that builds the model.
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        out = dataclasses.asdict(self)
        out["architectures"] = [self.architecture]
        return out

    def validate(self) -> None:
        raise NotImplementedError


def _require_int(name: str, value: Any, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: {name} must be >= {minimum}, got {value}")
    return value


@dataclass
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (reference src/models/qwen3/config.py:6-19).

    ``head_dim`` is independent of ``hidden_size / num_attention_heads``
    (16 x 128 = 2048 != 1024 in Qwen3-0.6B); when the key is absent it falls
    back to that quotient as the reference's model constructor does
    (src/models/qwen3/model.py:320).
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"

    num_hidden_layers: int = 28
    hidden_size: int = 1024
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    vocab_size: int = 151936
    rope_theta: float = 1_000_000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    max_position_embeddings: int = 40960
    attention_bias: bool = False
    hidden_act: str = "silu"
    eos_token_id: Optional[int] = None

    # -- derived, as src/models/qwen3/config.py:40-56 derives them -----------------
    @property
    def attention_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen3Config":
        rope_parameters = raw.get("rope_parameters") or {}
        rope_scaling = raw.get("rope_scaling")
        if rope_scaling not in (None, {}):
            kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
            if kind not in (None, "default"):
                raise ConfigError(
                    f"config.json: rope_scaling of type {kind!r} is not supported "
                    "(only plain rotary position encoding)")
        rope_type = rope_parameters.get("rope_type", "default")
        if rope_type not in (None, "default"):
            raise ConfigError(
                f"config.json: rope_parameters.rope_type {rope_type!r} is not supported")
        if raw.get("use_sliding_window"):
            raise ConfigError(
                "config.json: use_sliding_window=true is not supported for "
                "Qwen3ForCausalLM (every layer attends to all earlier tokens)")
        defaults = cls()
        hidden = raw.get("hidden_size", defaults.hidden_size)
        heads = raw.get("num_attention_heads", defaults.num_attention_heads)
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if not isinstance(hidden, int) or not isinstance(heads, int) or heads <= 0 \
                    or hidden % heads:
                raise ConfigError(
                    "config.json: head_dim is absent and hidden_size is not a "
                    "multiple of num_attention_heads")
            head_dim = hidden // heads
        eos = raw.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            num_hidden_layers=raw.get("num_hidden_layers", defaults.num_hidden_layers),
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=raw.get("num_key_value_heads", defaults.num_key_value_heads),
            head_dim=head_dim,
            intermediate_size=raw.get("intermediate_size", defaults.intermediate_size),
            vocab_size=raw.get("vocab_size", defaults.vocab_size),
            rope_theta=float(rope_parameters.get(
                "rope_theta", raw.get("rope_theta", defaults.rope_theta))),
            rms_norm_eps=float(raw.get("rms_norm_eps", defaults.rms_norm_eps)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings",
                                             defaults.tie_word_embeddings)),
            max_position_embeddings=raw.get("max_position_embeddings",
                                            defaults.max_position_embeddings),
            attention_bias=bool(raw.get("attention_bias", False)),
            hidden_act=raw.get("hidden_act", "silu"),
            eos_token_id=eos,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size",
                     "vocab_size", "max_position_embeddings"):
            _require_int(name, getattr(self, name))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a "
                f"multiple of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(
                f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if self.attention_bias:
            # The reference adds q/k/v biases and drops the per-head norms in this
            # case (src/models/qwen3/model.py:173-175, 204-206); no Qwen3 checkpoint
            # uses it and it is not built here.
            raise ConfigError("config.json: attention_bias=true is not supported")
        if self.hidden_act != "silu":
            raise ConfigError(
                f"config.json: hidden_act {self.hidden_act!r} is not supported (silu only)")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not (self.rope_theta > 0.0):
            raise ConfigError("config.json: rope_theta must be positive")


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def write_config_json(config: ModelConfig, model_dir: str) -> str:
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2, sort_keys=True)
        f.write("\n")
    return path
