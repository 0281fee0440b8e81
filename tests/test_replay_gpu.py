"""The engine against the plain implementation through trace replay: the same requests whole,
with the last 32 tokens decoded one by one, in portions of changing size, and mixed with other
requests over so few pages that they are used again; in float32 and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from helpers import (assert_close_logits, plain_logits, random_tokens, make_replayer as _replayer,
                     run_steps as _run, check_requests as _check, mixed_steps as _mixed_steps)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
NAMES = list(helpers.TINY)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(model_folders, name, dtype):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    reqs = {"a": random_tokens(V, 5, 1), "b": random_tokens(V, 77, 2), "c": random_tokens(V, 200, 3)}
    rep = _replayer(folder, name, dtype, 256)
    steps = [{"entries": [{"id": rid, "tokens": t, "want": list(range(len(t)))}], "end": [rid]}
             for rid, t in reqs.items()]
    _check(_run(rep, steps), folder, reqs, dtype, "whole")
    assert rep.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_decoded(model_folders, name, dtype):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    toks = random_tokens(V, 150, 4)
    rep = _replayer(folder, name, dtype, 192)
    head = len(toks) - 32
    steps = [{"entries": [{"id": "r", "tokens": toks[:head], "want": [0, head - 1]}]}]
    steps += [{"entries": [{"id": "r", "tokens": [toks[i]], "want": [0]}]} for i in range(head, len(toks))]
    steps[-1]["end"] = ["r"]
    got = _run(rep, steps)
    assert sorted(got["r"]) == [0, head - 1] + list(range(head, len(toks)))
    _check(got, folder, {"r": toks}, dtype, "last32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_changing_portions(model_folders, name, dtype):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    toks = random_tokens(V, 131, 5)
    rep = _replayer(folder, name, dtype, 192)
    sizes = [7, 3, 2, 11, 2, 5, 33, 2, 17, 16, 2, 31]
    assert sum(sizes) == len(toks)
    steps, p = [], 0
    for n in sizes:
        steps.append({"entries": [{"id": "r", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    got = _run(rep, steps)
    _check(got, folder, {"r": toks}, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("poison", [False, True])
def test_mixed_with_few_pages(model_folders, name, dtype, poison):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    lens = helpers.MIXED_LENS
    reqs = {f"r{i}": random_tokens(V, n, 10 + i) for i, n in enumerate(lens)}
    # four live requests of at most 128 tokens: exactly as many pages as they can hold at once
    rep = _replayer(folder, name, dtype, 4 * 128, poison=poison)
    total_pages = rep.cache.paged_groups[0].pool.num_pages
    steps = _mixed_steps(reqs, seed=99)
    got = _run(rep, steps)
    pages_needed = sum(-(-n // rep.cache.page_size) for n in lens)
    assert pages_needed > total_pages, "the trace must reuse pages"
    _check(got, folder, reqs, dtype, "mixed")
    assert rep.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_shared_prefix_and_its_absence_agree(model_folders, dtype):
    """Two requests that share their first tokens: with page sharing on, the second reuses the
    first one's pages; the logits equal the plain implementation's either way."""
    name = "tiny-b"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    page = helpers.TINY[name]["page"]
    common = random_tokens(V, 2 * page, 50)
    reqs = {"a": common + random_tokens(V, 9, 51), "b": common + random_tokens(V, 14, 52)}
    for share in (True, False):
        rep = _replayer(folder, name, dtype, 256, prefix_cache=share)
        steps = [{"entries": [{"id": "a", "tokens": reqs["a"], "want": [len(reqs["a"]) - 1]}]},
                 {"entries": [{"id": "b", "tokens": reqs["b"], "want": list(range(2 * page, len(reqs["b"])))}]}]
        got = _run(rep, steps)
        shared = rep.live["b"].shared_tokens
        assert shared == (2 * page if share else 0)
        _check(got, folder, reqs, dtype, f"prefix share={share}")


def test_trace_run_program(model_folders, tmp_path):
    """bin/trace_run as a user runs it: steps on standard input, files out, 'done' lines."""
    name = "tiny-a"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    a, b = random_tokens(V, 21, 60), random_tokens(V, 9, 61)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[10:12], "want": []}, {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[12:], "want": [8]}], "end": ["a"]},
    ]
    for dtype_name, dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        out = tmp_path / dtype_name
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype_name,
             "--out", str(out), "--max-tokens", "128", "--block-size", "4"],
            input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32"]
        wa, wb = plain_logits(folder, a), plain_logits(folder, b)
        l0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
        l1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
        l2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V))
        assert_close_logits(l0, wa[[0, 9]], dtype, "trace_run step 0")
        assert_close_logits(l1, wb[[8]], dtype, "trace_run step 1")
        assert_close_logits(l2, wa[[20]], dtype, "trace_run step 2")
