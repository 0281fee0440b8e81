"""The host side of the engine (cache manager, step function, replay) against the plain
implementation on the CPU, with the plain PyTorch operations in the place of the CUDA kernels.
The same traces run on the GPU, with the kernels, in tests/test_replay_gpu.py."""
import pytest
import torch

import helpers
from helpers import (check_requests, make_replayer, mixed_steps, random_tokens, run_steps)

F32 = torch.float32


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_portions_and_decode_on_host(model_folders, cpu_ops, name):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    toks = random_tokens(V, 70, 5)
    rep = make_replayer(folder, name, F32, 128, device="cpu")
    sizes = [7, 3, 2, 11, 2, 5, 20] + [1] * 20
    steps, p = [], 0
    for n in sizes:
        steps.append({"entries": [{"id": "r", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    check_requests(run_steps(rep, steps), folder, {"r": toks}, F32, "host portions")


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
@pytest.mark.parametrize("prefix_cache", [True, False])
def test_mixed_with_few_pages_on_host(model_folders, cpu_ops, name, prefix_cache):
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    reqs = {f"r{i}": random_tokens(V, n, 10 + i) for i, n in enumerate(helpers.MIXED_LENS)}
    rep = make_replayer(folder, name, F32, 4 * 128, prefix_cache=prefix_cache, poison=True, device="cpu")
    got = run_steps(rep, mixed_steps(reqs, seed=99))
    check_requests(got, folder, reqs, F32, "host mixed")
    assert rep.cache.pages_in_use() == 0
