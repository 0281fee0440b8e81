"""How a request's next tokens are chosen and when it stops.

The reference samples with argmax only and stops on the count of new tokens
(src/engine/executor.py:51-54, src/engine/llm_engine.py:36-42;
``max_new_tokens`` defaults to 16 in ``submit``, llm_engine.py:75).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0          # 0: greedy (argmax, the lowest index wins a tie)
    top_k: int = 0                    # 0: the whole vocabulary
    seed: Optional[int] = None        # None: the engine's seed
    ignore_eos: bool = False
    stop_token_ids: Sequence[int] = ()

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
