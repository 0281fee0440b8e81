"""What a model says about the tensors it needs, and where tensors come from."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Protocol

import torch

# kinds decide the random initialisation and the dtype a tensor is kept in
MATRIX = "matrix"        # [out, in] projection or embedding table: compute dtype
NORM = "norm"            # scale vector of a norm: always float32 on the device


@dataclass(frozen=True)
class WeightSpec:
    """One tensor of a checkpoint: its name there, its shape, and its kind.

    ``optional`` tensors may be absent (and are ignored when present), e.g.
    ``lm_head.weight`` of a model whose output head is tied to the embedding.
    """

    name: str
    shape: tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False


class TensorSource(Protocol):
    """Tensors by checkpoint name, on the CPU, in the dtype they are stored in."""

    def names(self) -> Iterable[str]: ...

    def shape(self, name: str) -> tuple[int, ...]: ...

    def get(self, name: str) -> torch.Tensor: ...


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every fault."""
