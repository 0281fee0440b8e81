"""Safetensors reading by tensor name, with one strict check.

The reference reads every ``*.safetensors`` of the folder into a CPU dict and
copies by parameter name, recording but never raising on unknown names or
shape mismatches, and never noticing a parameter that no file holds
(src/models/qwen3/utils.py:66-95).  Here the same names are read, but a
checkpoint that does not fit is refused with one error listing every missing
tensor, every unexpected tensor and every wrong shape.
"""
from __future__ import annotations

import json
import os
from typing import Iterable

import torch
from safetensors import safe_open

from .spec import WeightError, WeightSpec


class SafetensorsSource:
    """All tensors of a model folder's safetensors files, opened lazily."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                files = sorted(set(json.load(f)["weight_map"].values()))
        else:
            files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors")) \
                if os.path.isdir(model_dir) else []
        if not files:
            raise WeightError(f"no .safetensors file in model folder {model_dir!r}")
        self._file_of: dict[str, str] = {}
        self._shapes: dict[str, tuple[int, ...]] = {}
        self._handles: dict[str, object] = {}
        for fname in files:
            path = os.path.join(model_dir, fname)
            if not os.path.isfile(path):
                raise WeightError(f"{path}: named by the index but not in the folder")
            handle = safe_open(path, framework="pt", device="cpu")
            self._handles[fname] = handle
            for name in handle.keys():
                self._file_of[name] = fname
                self._shapes[name] = tuple(handle.get_slice(name).get_shape())

    def names(self) -> Iterable[str]:
        return self._file_of.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return self._shapes[name]

    def get(self, name: str) -> torch.Tensor:
        return self._handles[self._file_of[name]].get_tensor(name)


def check_against_manifest(source, manifest: Iterable[WeightSpec], where: str = "checkpoint") -> None:
    """Raise one WeightError naming every fault, or return silently."""
    specs = {s.name: s for s in manifest}
    have = set(source.names())
    missing = sorted(n for n, s in specs.items() if n not in have and not s.optional)
    unexpected = sorted(n for n in have if n not in specs)
    wrong = []
    for n in sorted(have & set(specs)):
        got, want = tuple(source.shape(n)), tuple(specs[n].shape)
        if got != want and not specs[n].optional:
            wrong.append(f"{n}: stored {list(got)}, model needs {list(want)}")
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where} does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
    raise WeightError("\n".join(lines))
