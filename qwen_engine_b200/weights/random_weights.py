"""Seeded random weights, and a writer of whole model folders.

The reference initialises in its constructors, unseeded (embedding and head
N(0, 0.02), linears kaiming-uniform, norms one: src/models/qwen3/model.py:22,
34, 58, 367).  Here every tensor has a generator of its own, seeded by
(seed, tensor name), so a tensor's values do not depend on the order of
creation, on the device or on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import os
from typing import Iterable

import torch
from safetensors.torch import save_file

from ..config import ModelConfig, write_config_json
from .spec import MATRIX, NORM, WeightSpec


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.blake2b(f"{seed}:{name}".encode("utf-8"), digest_size=8).digest()
    return int.from_bytes(digest, "little") & 0x7FFF_FFFF_FFFF_FFFF


class RandomSource:
    """A TensorSource that makes each tensor when asked.

    Matrices are N(0, std); norm scales are 1 + N(0, norm_std).  Values are drawn
    in float32 on the CPU and rounded to ``store_dtype``."""

    def __init__(self, manifest: Iterable[WeightSpec], seed: int, std: float = 0.02,
                 norm_std: float = 0.1, store_dtype: torch.dtype = torch.bfloat16):
        self._specs = {s.name: s for s in manifest if not s.optional}
        self.seed, self.std, self.norm_std = seed, std, norm_std
        self.store_dtype = store_dtype

    def names(self):
        return self._specs.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._specs[name].shape)

    def get(self, name: str) -> torch.Tensor:
        spec = self._specs[name]
        gen = torch.Generator(device="cpu").manual_seed(_tensor_seed(self.seed, name))
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if spec.kind == NORM:
            t = 1.0 + self.norm_std * t
        elif spec.kind == MATRIX:
            t = self.std * t
        else:
            raise ValueError(f"unknown weight kind {spec.kind!r} for {name}")
        return t.to(self.store_dtype)


def write_model_folder(config: ModelConfig, model_dir: str, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` of a random model."""
    from ..registry import weight_manifest_for
    source = RandomSource(weight_manifest_for(config), seed, std, norm_std, store_dtype)
    os.makedirs(model_dir, exist_ok=True)
    write_config_json(config, model_dir)
    tensors = {name: source.get(name).contiguous() for name in source.names()}
    save_file(tensors, os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})
    return model_dir
