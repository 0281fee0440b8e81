"""Qwen3 dense decoder as a layout of parts (reference src/models/qwen3/model.py).

Every layer is the same here: a pre-norm block of RMS norm, grouped-query
attention with per-head q/k norms and rotary positions, and a SwiGLU
feed-forward (model.py:240-298).  Tensor names are the checkpoint's own
(model.layers.{i}.self_attn.q_proj.weight and so on), which are the
reference's parameter names.
"""
from __future__ import annotations

from ..config import Qwen3Config
from ..parts.base import PartSpec
from .decoder import LayerSpec, ModelLayout, PlanEntry


def qwen3_layout(cfg: Qwen3Config) -> ModelLayout:
    norm = PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps))
    rope = PartSpec("rope_neox", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))
    mixer = PartSpec("gqa_attention", dict(
        hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
        num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
        scale=cfg.attention_scale, qk_norm_eps=cfg.rms_norm_eps, position_encoding=rope))
    ffn = PartSpec("swiglu", dict(hidden_size=cfg.hidden_size,
                                  intermediate_size=cfg.intermediate_size))
    block = PartSpec("pre_norm", dict(hidden_size=cfg.hidden_size, mixer=mixer,
                                      feed_forward=ffn, norm=norm))
    n = cfg.num_hidden_layers
    return ModelLayout(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        layers=tuple(LayerSpec(block, f"model.layers.{i}.") for i in range(n)),
        plan=tuple(PlanEntry(i, i, True) for i in range(n)),
        final_norm=norm, tie_head=cfg.tie_word_embeddings,
        max_positions=cfg.max_position_embeddings)
