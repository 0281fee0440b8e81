"""The configuration of the Qwen3 dense decoder, read from its ``config.json`` keys.

The defaults are those of the reference's ``Qwen3Config`` (src/models/qwen3/config.py:6-19) and of its
``from_hf_config`` (src/models/qwen3/config.py:22-38); they apply when a key is absent.  The generic base
class, the error type and the reading and writing of ``config.json`` are in ``model_config.py``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, ClassVar, Optional

from .model_config import ConfigError, ModelConfig, _require_int


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
    eos_token_id: Optional[int] = None          # the first (or only) end-of-sequence id of config.json
    eos_token_ids: tuple = ()                   # every one of them (config.json may give a list)

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        ids = out.pop("eos_token_ids")
        if len(ids) > 1:
            out["eos_token_id"] = list(ids)          # config.json's own form for several ids
        return out

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
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        eos = eos_all[0] if eos_all else None
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
            eos_token_ids=eos_all,
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
