"""A plain, slow Qwen3 dense decoder: whole sequences, no cache, float32, CPU.

It is the oracle of the tests.  It shares no code with the engine: it reads the
model folder itself and computes every part with one small function written
from the formulas of kzw3933/Qwen-Engine; each function cites the file and line
of the reference it restates.  tests/golden/ holds logits of the reference's own
model code (its ``mode="torch"`` path run on the CPU) for a tiny random model;
tests/test_plain.py checks this file against them.
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


def read_model_folder(model_dir: str) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict, and every tensor of model.safetensors as float32.

    The reference copies checkpoint tensors into float32 parameters on the CPU
    (src/models/qwen3/utils.py:84-91, main.py:26)."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    tensors: dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt",
                   device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(torch.float32)
    return cfg, tensors


def cfg_numbers(cfg: dict) -> dict:
    """The numbers the formulas need, from the config.json keys with the
    reference's fall-backs (src/models/qwen3/config.py:22-38, 40-56)."""
    rope_parameters = cfg.get("rope_parameters") or {}
    hidden = cfg["hidden_size"]
    heads = cfg["num_attention_heads"]
    head_dim = cfg.get("head_dim", hidden // heads)
    return dict(
        layers=cfg["num_hidden_layers"], hidden=hidden, heads=heads,
        kv_heads=cfg.get("num_key_value_heads", heads), head_dim=head_dim,
        inter=cfg["intermediate_size"], vocab=cfg["vocab_size"],
        theta=float(rope_parameters.get("rope_theta", cfg.get("rope_theta", 1_000_000))),
        eps=float(cfg.get("rms_norm_eps", 1e-6)),
        tied=bool(cfg.get("tie_word_embeddings", True)),
        scale=1.0 / math.sqrt(head_dim),          # config.py:46
    )


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :]  (src/layers/ops/embedding.py:28-44, 136-137)."""
    return table[ids]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis
    (src/layers/ops/layernorm.py:50-88; commented formula at :200-207)."""
    x = x.to(torch.float32)
    mean_square = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(mean_square + eps) * weight.to(torch.float32)


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T with W stored [out, in], no bias
    (src/layers/ops/linear.py:101-122, 173-185)."""
    return x @ weight.t()


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq[j] = theta^(-2j/D); angle = pos * inv_freq; cos and sin of it in
    float32 (src/models/qwen3/model.py:75-84)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    return torch.cos(freqs), torch.sin(freqs)


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split ("neox") rotation of x [T, heads, D]:
    out = [cos*x1 - sin*x2 , sin*x1 + cos*x2] with x1, x2 the two halves
    (src/layers/ops/rope.py:256-272)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([c * x1 - s * x2, s * x1 + c * x2], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None) -> torch.Tensor:
    """Whole-sequence attention of one request.  q [T, Hq, D]; k, v [T, Hkv, D].

    Query head h uses key/value head h // (Hq / Hkv) (src/layers/fused_ops/attn.py:181-182);
    key j is allowed for query i iff j <= i (attn.py:195, 239: q_abs_pos >= key_pos);
    scores are scaled dot products, softmax over the allowed keys, then the
    weighted sum of values (attn.py:236-267; torch twin :767-780).
    ``window`` (not a Qwen3 option) further restricts to j > i - window."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    out = torch.empty_like(q)
    idx = torch.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window is not None:
        allowed &= idx[None, :] > idx[:, None] - window
    for h in range(Hq):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        scores = (q[:, h, :] @ kh.t()) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ vh
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g))
    (src/layers/fused_ops/silumul.py:50-53, 156-157)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_part(x: torch.Tensor, positions: torch.Tensor, w: dict[str, torch.Tensor],
                   prefix: str, n: dict) -> torch.Tensor:
    """q/k/v projections, per-head norms of q and k, rotation, attention, output
    projection (src/models/qwen3/model.py:200-213)."""
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"]).view(T, n["heads"], n["head_dim"])
    k = linear(x, w[prefix + "k_proj.weight"]).view(T, n["kv_heads"], n["head_dim"])
    v = linear(x, w[prefix + "v_proj.weight"]).view(T, n["kv_heads"], n["head_dim"])
    q = rmsnorm(q, w[prefix + "q_norm.weight"], n["eps"])      # model.py:204-206
    k = rmsnorm(k, w[prefix + "k_norm.weight"], n["eps"])
    cos, sin = rope_angles(positions, n["head_dim"], n["theta"])
    q = rope_rotate(q, cos, sin)                                # model.py:208
    k = rope_rotate(k, cos, sin)
    o = causal_attention(q, k, v, n["scale"])                   # model.py:210
    return linear(o.reshape(T, n["heads"] * n["head_dim"]), w[prefix + "o_proj.weight"])


def mlp_part(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x))  (src/models/qwen3/model.py:232-237)."""
    gate = linear(x, w[prefix + "gate_proj.weight"])
    up = linear(x, w[prefix + "up_proj.weight"])
    return linear(silu_mul(gate, up), w[prefix + "down_proj.weight"])


def decoder_layer(x: torch.Tensor, positions: torch.Tensor, w: dict[str, torch.Tensor],
                  i: int, n: dict) -> torch.Tensor:
    """Pre-norm residual block (src/models/qwen3/model.py:278-298)."""
    p = f"model.layers.{i}."
    h = rmsnorm(x, w[p + "input_layernorm.weight"], n["eps"])
    x = x + attention_part(h, positions, w, p + "self_attn.", n)
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], n["eps"])
    return x + mlp_part(h, w, p + "mlp.")


def forward_logits(cfg: dict, w: dict[str, torch.Tensor], token_ids) -> torch.Tensor:
    """Logits [T, vocab] of one whole request (positions 0..T-1)
    (src/models/qwen3/model.py:347-360, 420-422; tied head :417-418)."""
    n = cfg_numbers(cfg)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    x = embedding(ids, w["model.embed_tokens.weight"])
    for i in range(n["layers"]):
        x = decoder_layer(x, positions, w, i, n)
    x = rmsnorm(x, w["model.norm.weight"], n["eps"])
    head = w["model.embed_tokens.weight"] if n["tied"] else w["lm_head.weight"]
    return linear(x, head)


# ---- sampling, restated for the tests of the engine's sampler ---------------------------

def greedy_token(logits_row: torch.Tensor) -> int:
    """argmax over the vocabulary (src/engine/executor.py:51-54); the lowest
    index wins a tie."""
    return int(torch.argmax(logits_row.to(torch.float32)).item())


def greedy_generate(cfg: dict, w: dict[str, torch.Tensor], prompt, steps: int) -> list[int]:
    """Greedy decoding by recomputing the whole sequence at every step: the stop
    rule is the reference's count of new tokens (src/engine/llm_engine.py:36-42)."""
    tokens = list(prompt)
    out: list[int] = []
    for _ in range(steps):
        nxt = greedy_token(forward_logits(cfg, w, tokens)[-1])
        out.append(nxt)
        tokens.append(nxt)
    return out
