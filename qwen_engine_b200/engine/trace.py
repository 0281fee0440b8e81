"""Trace replay: given token ids are fed through the model step by step and the
logits at the wanted places are written out.  Nothing is sampled.

The replayer drives the engine's own model, step function, cache manager and
kernels, the ones generation uses; it only stands where the scheduler stands.
A step is a JSON object

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted; all entries of a step run as one batch.  ``end``: requests
that are finished after the step; what they hold goes back to the pool.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Optional

import numpy as np
import torch

from ..cache.manager import RequestCache
from .loading import LoadedModel, load_model
from .runner import StepEntry

ROUND_TOKENS = 64      # a request's tokens are counted rounded up to this (or to a larger page)


class TraceError(ValueError):
    pass


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: torch.dtype, max_tokens: int, device="cuda:0",
                 page_size: int = 16, max_live: int = 64, enable_prefix_cache: bool = True,
                 loaded: Optional[LoadedModel] = None):
        if max_tokens < 1:
            raise TraceError("--max-tokens must be positive")
        unit = max(ROUND_TOKENS, page_size)
        unit = -(-unit // page_size) * page_size
        num_pages = -(-max_tokens // unit) * (unit // page_size)
        self.loaded = loaded or load_model(model_dir, dtype, device, page_size, num_pages, max_live,
                                           enable_prefix_cache=enable_prefix_cache)
        self.cache = self.loaded.cache
        self.runner = self.loaded.runner
        self.live: dict[str, RequestCache] = {}

    def run_step(self, step: dict) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [wanted, vocab] on the device, or None."""
        entries = step.get("entries", [])
        if not isinstance(entries, list):
            raise TraceError("'entries' must be a list")
        batch: list[StepEntry] = []
        seen = set()
        for e in entries:
            rid = e["id"]
            if rid in seen:
                raise TraceError(f"request {rid!r} appears twice in step {step.get('step')}")
            seen.add(rid)
            tokens = [int(t) for t in e["tokens"]]
            want = [int(w) for w in e.get("want", [])]
            for w in want:
                if not (0 <= w < len(tokens)):
                    raise TraceError(f"request {rid!r}: wanted place {w} is outside its {len(tokens)} tokens")
            skip = 0
            rc = self.live.get(rid)
            if rc is None:
                # a new request: pages of an equal prefix may be shared, but never past a place
                # whose logits are wanted, and one token is always left to run
                limit = min(want) if want else max(len(tokens) - 1, 0)
                rc = self.cache.open(rid, known_tokens=tokens, max_shared_tokens=min(limit, max(len(tokens) - 1, 0)))
                self.live[rid] = rc
                skip = rc.num_tokens
            batch.append(StepEntry(rc, tokens[skip:], [w - skip for w in want]))
        logits = self.runner.step(batch)
        for rid in step.get("end", []):
            rc = self.live.pop(rid, None)
            if rc is None:
                raise TraceError(f"'end' names request {rid!r}, which is not live")
            self.cache.close(rc)
        return logits

    def close_all(self) -> None:
        for rc in self.live.values():
            self.cache.close(rc)
        self.live.clear()


def replay_stream(replayer: TraceReplayer, lines, out_dir: str, log=sys.stdout) -> int:
    """Read steps (one JSON object a line), write ``<out_dir>/<step>.f32`` for the steps in
    which something is wanted, print ``done <step>`` after each."""
    os.makedirs(out_dir, exist_ok=True)
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        try:
            step = json.loads(line)
        except json.JSONDecodeError as e:
            raise TraceError(f"step {n}: not a JSON object: {e}") from None
        sid = step.get("step", n)
        logits = replayer.run_step(step)
        if logits is not None and logits.shape[0] > 0:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            with open(os.path.join(out_dir, f"{sid}.f32"), "wb") as f:
                f.write(arr.tobytes())
        print(f"done {sid}", file=log, flush=True)
        n += 1
    return n


def read_logits_file(path: str, vocab: int) -> np.ndarray:
    return np.fromfile(path, dtype="<f4").reshape(-1, vocab)
