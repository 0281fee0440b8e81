"""A decode step's kernels on one time axis, without a profiler.

    python -m qwen_engine_b200.engine.timeline [--model qwen3-0.6b] [--batch 8] [--context 1024] [--layer 14]

builds (at its first call) and loads the timeline build of the CUDA library, in which thread 0 of every
CTA notes the GPU's global timer when it lets its dependents start (about when the CTA started), when its
wait for the kernel before it returns (that kernel has completed), and at marks inside some kernels;
replays one decode step of random weights from its CUDA graph and prints, for the kernels between two
attention launches (one layer), when their CTAs started and when their waits returned, in microseconds.
The reference has no such tool (its only timing is Triton's do_bench in the op files, e.g.
src/layers/ops/linear.py:241).  The probes cost a few hundred nanoseconds each, so the step is some
10-20 % slower than in the plain build: read the shares and the gaps, not the absolutes.
"""
from __future__ import annotations

import argparse
import collections
import os
import random
import sys


def record_decode_step(model: str, batch: int, context: int):
    """Events (see ``ops.timeline_events``) of one replayed decode step."""
    os.environ["QE_TIMELINE"] = "1"            # before the library is built and loaded
    import torch
    from .. import ops
    from ..config import preset_config_dict
    from ..registry import config_from_dict
    from .loading import load_model
    from .runner import StepEntry
    cfg = config_from_dict(preset_config_dict(model))
    page = 16
    pages = batch * (-(-(context + 64) // page)) + 16
    loaded = load_model(None, torch.bfloat16, "cuda:0", page, pages, batch + 2, enable_prefix_cache=False,
                        config=cfg, random_seed=2)
    runner, cache = loaded.runner, loaded.cache
    rng = random.Random(0)
    reqs = [cache.open(i) for i in range(batch)]
    for i in range(0, batch, 4):
        runner.step([StepEntry(rc, [rng.randrange(cfg.vocab_size) for _ in range(context)], []) for rc in reqs[i:i + 4]])

    def one():
        runner.step([StepEntry(rc, [rng.randrange(cfg.vocab_size)], [0]) for rc in reqs])
    for _ in range(6):                          # the step's graph is captured and warm
        one()
    torch.cuda.synchronize()
    ops.timeline_begin(1 << 18)
    one()
    torch.cuda.synchronize()
    return ops.timeline_events()


def layer_table(events, layer: int) -> str:
    """The events between the ``layer``-th and the next launch of the attention kernel, grouped by probe."""
    att = [e for e in events if e[0].startswith("attention_decode") and e[2] == 0]
    if not att:
        return "no attention launches among the events"
    grid = att[0][4]
    n_launches = len(att) // grid
    layer = max(0, min(layer, n_launches - 2))
    t0, t1 = att[layer * grid][5], att[(layer + 1) * grid][5]
    kinds = {0: "CTA started", 1: "wait returned", 2: "mark 2", 3: "mark 3"}
    rows = collections.defaultdict(list)
    for f, line, kind, cta, total, t, sm in events:
        if t0 <= t < t1:
            rows[(f, line, kind, total)].append((t - t0) / 1000.0)
    out = [f"one layer of the step: {(t1 - t0) / 1000.0:.2f} us from attention launch {layer} to the next "
           f"({n_launches} launches of {grid} CTAs in the step)",
           f"{'probe (file:line)':34s} {'what':14s} {'grid':>5s} {'n':>5s} {'first':>8s} {'median':>8s} {'last':>8s}   us"]
    for (f, line, kind, total), ts in sorted(rows.items(), key=lambda kv: kv[1][0]):
        ts.sort()
        out.append(f"{f + ':' + str(line):34s} {kinds[kind]:14s} {total:5d} {len(ts):5d} {ts[0]:8.2f} {ts[len(ts) // 2]:8.2f} {ts[-1]:8.2f}")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen3-0.6b", help="a preset's name")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layer", type=int, default=14, help="which layer's kernels to print")
    args = ap.parse_args(argv)
    events = record_decode_step(args.model, args.batch, args.context)
    print(f"{len(events)} events")
    print(layer_table(events, args.layer))
    return 0


if __name__ == "__main__":
    sys.exit(main())
