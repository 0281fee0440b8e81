"""Named configurations: each is the content of a ``config.json``.

The sizes are data here, not constants of the code: a preset is turned into a
model folder (config.json + model.safetensors) by the random-weights writer
and read back like any other model.  ``init`` gives the spread of the random
weights and the page size the configuration is usually run with.
"""
from __future__ import annotations

from typing import Any

_QWEN3_COMMON = dict(
    architectures=["Qwen3ForCausalLM"], hidden_act="silu", attention_bias=False,
    head_dim=128, vocab_size=151936, rope_theta=1_000_000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=40960,
)

PRESETS: dict[str, dict[str, Any]] = {
    "tiny-a": dict(
        config=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                    rms_norm_eps=1e-6, tie_word_embeddings=True,
                    max_position_embeddings=512),
        init=dict(seed=0, std=0.02, norm_std=0.1, block_size=4)),
    "tiny-b": dict(
        config=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=80,
                    num_attention_heads=4, num_key_value_heads=1, head_dim=32,
                    intermediate_size=224, vocab_size=389, rope_theta=1_000_000.0,
                    rms_norm_eps=1e-5, tie_word_embeddings=False,
                    max_position_embeddings=512),
        init=dict(seed=1, std=0.05, norm_std=0.2, block_size=8)),
    "qwen3-0.6b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=28, hidden_size=1024,
                    num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072),
        init=dict(seed=2, std=0.02, norm_std=0.1, block_size=16)),
    "qwen3-1.7b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=28, hidden_size=2048,
                    num_attention_heads=16, num_key_value_heads=8, intermediate_size=6144),
        init=dict(seed=3, std=0.02, norm_std=0.1, block_size=16)),
    "qwen3-4b": dict(
        config=dict(_QWEN3_COMMON, num_hidden_layers=36, hidden_size=2560,
                    num_attention_heads=32, num_key_value_heads=8, intermediate_size=9728),
        init=dict(seed=4, std=0.02, norm_std=0.1, block_size=16)),
}


def preset_config_dict(name: str) -> dict[str, Any]:
    try:
        return dict(PRESETS[name]["config"])
    except KeyError:
        raise ValueError(f"unknown preset {name!r}; known: {sorted(PRESETS)}") from None


def preset_init(name: str) -> dict[str, Any]:
    preset_config_dict(name)
    return dict(PRESETS[name]["init"])
