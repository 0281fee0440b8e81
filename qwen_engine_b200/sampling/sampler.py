"""Greedy and temperature / top-k sampling on the device, with the uniform
numbers made on the host by a counter-based generator: the number for
(seed, request, output position) is a pure function of the three, so a
request's tokens do not depend on which other requests share its steps, and a
plain implementation on the CPU can reproduce them."""
from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from .params import SamplingParams

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, request_index: int, position: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32)."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ (request_index & _MASK))
    h = _splitmix64(h ^ (position & _MASK))
    return (h >> 40) / float(1 << 24)


class SampledTokens:
    """The tokens of one sampling call: on the device at once (``device``, int32 [N]), on the host
    when ``read()`` is called (their copy to pinned memory is queued right behind the sampling)."""

    def __init__(self, device_tokens: torch.Tensor):
        self.device = device_tokens
        self._host = None
        self._event = None
        if device_tokens.is_cuda:
            self._host = torch.empty(device_tokens.shape, dtype=device_tokens.dtype, pin_memory=True)
            self._host.copy_(device_tokens, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()

    def read(self) -> list[int]:
        if self._host is None:
            return self.device.tolist()
        self._event.synchronize()
        return self._host.tolist()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               uniforms: Sequence[float]) -> list[int]:
        """One token per row of float32 logits [N, V]; returns host ints."""
        return self.sample_async(logits, params, uniforms).read()

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     uniforms: Sequence[float]) -> SampledTokens:
        """The same without waiting for the device."""
        N = logits.shape[0]
        assert N == len(params) == len(uniforms)
        out = torch.empty(N, dtype=torch.int32, device=self.device)
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
        else:
            meta = torch.tensor([[p.temperature for p in params], list(uniforms)], dtype=torch.float32)
            topk = torch.tensor([p.top_k for p in params], dtype=torch.int32)
            if self.device.type == "cuda":
                meta = meta.pin_memory().to(self.device, non_blocking=True)
                topk = topk.pin_memory().to(self.device, non_blocking=True)
            ops.sample(logits, meta[0].contiguous(), topk, meta[1].contiguous(), out)
        return SampledTokens(out)
