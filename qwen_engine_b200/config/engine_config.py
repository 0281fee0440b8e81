"""Engine-side knobs: the constants the reference keeps at the top of its
``main.py`` (main.py:17-27: max_num_seqs, max_model_len, block_size,
num_blocks, dtype) plus the ones its README lists as not covered (token
budget and prompt portions, README.md:30-35)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {name!r}") from None


@dataclass
class EngineConfig:
    """How the engine runs a model; none of it changes a model's numbers."""

    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda:0"
    block_size: int = 16                  # tokens in a page (main.py:22)
    num_blocks: Optional[int] = None      # pages per cache group; None: from gpu_memory_fraction, else max_num_seqs*max_model_len
    gpu_memory_fraction: Optional[float] = None   # with num_blocks None: the cache takes what is left of this share of the device's memory
    max_model_len: int = 256              # most tokens one request may hold (main.py:21)
    max_num_seqs: int = 4                 # most live requests (main.py:20)
    max_num_batched_tokens: int = 2048    # token budget of one step
    prefill_chunk_size: Optional[int] = None  # largest prompt portion; None: the budget
    enable_prefix_cache: bool = True
    use_cuda_graphs: bool = True
    run_ahead: bool = True                # launch the next decode step before the host has read this one's tokens
    seed: int = 0
    profile: bool = False                 # time every step on the device (CUDA events) and keep sums per kind of step

    def __post_init__(self) -> None:
        self.dtype = parse_dtype(self.dtype)
        if self.block_size < 1:
            raise ValueError("block_size must be >= 1")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_model_len < 2:
            raise ValueError("max_model_len must be >= 2")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.prefill_chunk_size is not None and self.prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be >= 1")
        if self.gpu_memory_fraction is not None and not (0.0 < self.gpu_memory_fraction <= 1.0):
            raise ValueError("gpu_memory_fraction must be in (0, 1]")

    @property
    def blocks_per_seq(self) -> int:
        return -(-self.max_model_len // self.block_size)

    def resolved_num_blocks(self) -> Optional[int]:
        """The number of pages per cache group: ``num_blocks`` if given; None if the loader is to size the cache
        from ``gpu_memory_fraction``; else main.py:23: ``max_num_seqs * ceil(max_model_len / block_size)``."""
        if self.num_blocks is not None:
            return self.num_blocks
        if self.gpu_memory_fraction is not None:
            return None
        return self.max_num_seqs * self.blocks_per_seq
