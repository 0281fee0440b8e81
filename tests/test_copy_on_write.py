"""A prompt that is found whole in shared pages, and preemption while pages are shared.

When every page of a prompt (its length a multiple of the page size) is found in the prefix table, its
last token still has to run, because its logits are needed; its key and value would land in a shared
page, so the request first gets a private copy of that page (the reference writes into the shared
block, src/engine/executor.py:114-119, 139-140).  The copy runs on the device (``ops.copy_pages``)
before the step's first write.  The cache starts out poisoned: a copy that did not run, or went to the
wrong page, shows in the logits.

The host-side tests run with the plain operations in the place of the kernels; the ``gpu`` ones with
the kernels, in 32-bit and in bfloat16."""
import pytest
import torch

import helpers
import plain_qwen3
from helpers import check_requests, make_engine, make_replayer, random_tokens, run_steps
from qwen_engine_b200.sampling import SamplingParams

F32, BF16 = torch.float32, torch.bfloat16


def _plain_greedy(folder, prompt, steps):
    cfg, w = plain_qwen3.read_model_folder(folder)
    return plain_qwen3.greedy_generate(cfg, w, prompt, steps)


def _count_copies(monkeypatch):
    from qwen_engine_b200 import ops
    calls = []
    real = ops.copy_pages
    monkeypatch.setattr(ops, "copy_pages", lambda cache, pairs: (calls.append(pairs.tolist()), real(cache, pairs))[1])
    return calls


# ---- through the engine: scheduler, step function, sampler ---------------------------------------------
def _whole_prompt_found_through_the_engine(folder, name, device, monkeypatch):
    page = helpers.TINY[name]["page"]
    V = helpers.vocab_of(name)
    prompt = random_tokens(V, 2 * page, 201)
    want = _plain_greedy(folder, prompt, 12)
    copies = _count_copies(monkeypatch)
    eng = make_engine(folder, name, F32, device=device, max_model_len=96, poison_cache=True)
    a = eng.add_request(prompt, SamplingParams(max_new_tokens=12, ignore_eos=True))
    done = []
    while len(eng.scheduler.running) == 0 or eng.scheduler.running[0].output_len < 3:
        done += eng.step()
    assert not copies
    b = eng.add_request(prompt, SamplingParams(max_new_tokens=12, ignore_eos=True))     # while a is live
    while eng.has_work():
        done += eng.step()
    c = eng.add_request(prompt, SamplingParams(max_new_tokens=5, ignore_eos=True))      # after both ended: freed, findable pages
    while eng.has_work():
        done += eng.step()
    outs = {s.seq_id: s for s in done}
    assert outs[a].shared_prefix_len == 0
    assert outs[b].shared_prefix_len == 2 * page - 1 and outs[c].shared_prefix_len == 2 * page - 1
    assert len(copies) == 2 and all(len(p) == 2 and p[0] != p[1] for p in copies), copies
    assert outs[a].output_token_ids == want, "the first request's tokens changed"
    assert outs[b].output_token_ids == want and outs[c].output_token_ids == want[:5]
    assert eng.cache.pages_in_use() == 0
    eng.cache.check_invariants()


def test_whole_prompt_found_on_host(model_folders, cpu_ops, monkeypatch):
    _whole_prompt_found_through_the_engine(model_folders["tiny-a"], "tiny-a", "cpu", monkeypatch)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_whole_prompt_found_on_the_gpu(model_folders, monkeypatch, name):
    _whole_prompt_found_through_the_engine(model_folders[name], name, "cuda:0", monkeypatch)


# ---- through replay: logits, also in bfloat16 -------------------------------------------------------------
def _whole_prompt_found_in_replay(folder, name, dtype, device, monkeypatch, poison=True):
    page = helpers.TINY[name]["page"]
    V = helpers.vocab_of(name)
    common = random_tokens(V, 2 * page, 211)
    reqs = {"a": common + random_tokens(V, 5, 212), "b": common + random_tokens(V, 7, 213),
            "c": common + random_tokens(V, page + 3, 214), "d": common[:page] + random_tokens(V, page, 215)}
    n = 2 * page
    copies = _count_copies(monkeypatch)
    rep = make_replayer(folder, name, dtype, 8 * 64, poison=poison, device=device)
    steps = [
        {"entries": [{"id": "a", "tokens": reqs["a"][:n], "want": [n - 1]}]},
        {"entries": [{"id": "a", "tokens": reqs["a"][n:n + 2], "want": [0, 1]}]},
        # b brings exactly the shared prompt and wants its last place only: every page is found
        {"entries": [{"id": "a", "tokens": reqs["a"][n + 2:n + 3], "want": [0]},
                     {"id": "b", "tokens": reqs["b"][:n], "want": [n - 1]}]},
        {"entries": [{"id": "a", "tokens": reqs["a"][n + 3:], "want": [0, 1]},
                     {"id": "b", "tokens": reqs["b"][n:], "want": list(range(7))}], "end": ["a"]},
        # c after a ended (b still holds the pages), whole prompt found again, then a portion across a page's edge;
        # d shares one page only and diverges inside the second
        {"entries": [{"id": "c", "tokens": reqs["c"][:n], "want": [n - 1]},
                     {"id": "d", "tokens": reqs["d"], "want": list(range(page, 2 * page))}], "end": ["b", "d"]},
        {"entries": [{"id": "c", "tokens": reqs["c"][n:], "want": list(range(page + 3))}], "end": ["c"]},
    ]
    shared = {}
    real_open = rep.cache.open

    def open_and_note(rid, **kw):
        rc = real_open(rid, **kw)
        shared[rid] = rc.shared_tokens
        return rc
    rep.cache.open = open_and_note
    got = run_steps(rep, steps)
    assert shared["a"] == 0 and shared["b"] == n - 1 and shared["c"] == n - 1, shared
    assert len(copies) == 2, copies          # b and c
    check_requests(got, folder, reqs, dtype, f"whole prompt found {name}")
    assert rep.cache.pages_in_use() == 0


def test_whole_prompt_found_in_replay_on_host(model_folders, cpu_ops, monkeypatch):
    _whole_prompt_found_in_replay(model_folders["tiny-b"], "tiny-b", F32, "cpu", monkeypatch)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c", "tiny-d"])
def test_whole_prompt_found_in_replay_on_the_gpu(model_folders, monkeypatch, name, dtype):
    poison = 3.0e4 if (name == "tiny-d" and dtype == BF16) else True
    _whole_prompt_found_in_replay(model_folders[name], name, dtype, "cuda:0", monkeypatch, poison=poison)


# ---- preemption while pages are shared ----------------------------------------------------------------------
def _preemption_with_sharing(folder, name, device):
    """Three requests over too few pages with the prefix table on: the request preempted last is admitted
    again over its prompt and the tokens it made, finds the pages it gave back (they stay findable until
    they are handed out again) and recomputes the rest; tokens equal the plain implementation's.  Run at
    several prompt lengths so that the victim's length at preemption is a multiple of the page size too."""
    V = helpers.vocab_of(name)
    page = helpers.TINY[name]["page"]
    lengths_at_preemption = set()
    hits = 0
    cases = [(plens, ahead) for ahead in (False, True)
             for plens in ((10, 10, 10), (9, 11, 12), (12, 10, 11), (11, 9, 8), (10, 12, 9))]
    for plens, ahead in cases:
        # step by step, the newest request is preempted when an older one needs a page, at any length; with steps
        # launched ahead (which never preempt) requests sit out until none can go on, so that the victim is one
        # token into a page
        prompts = [random_tokens(V, n, 90 + i) for i, n in enumerate(plens)]
        eng = make_engine(folder, name, F32, device=device, num_blocks=12, max_model_len=32, enable_prefix_cache=True,
                          run_ahead=ahead)
        real = eng.scheduler._preempt_newest

        def spy(out, reserved, real=real, eng=eng):
            victim = real(out, reserved)
            lengths_at_preemption.add(victim.total_len % page)
            return victim
        eng.scheduler._preempt_newest = spy
        ids = eng.submit(prompts, max_new_tokens=14)
        outs = {o.request_id: o for o in eng.serving()}
        assert eng.stats.preemptions >= 1
        for i, p in zip(ids, prompts):
            assert outs[i].output_token_ids == _plain_greedy(folder, p, 14), f"prompt lengths {plens}, ahead {ahead}, request {i}"
        hits += sum(o.shared_prefix_len > 0 for o in outs.values() if o.num_preemptions)
        assert eng.cache.pages_in_use() == 0
        eng.cache.check_invariants()
    assert 0 in lengths_at_preemption, lengths_at_preemption
    assert hits >= 1, "no preempted request found its own pages again"


def test_preemption_with_sharing_on_host(model_folders, cpu_ops):
    _preemption_with_sharing(model_folders["tiny-a"], "tiny-a", "cpu")


@pytest.mark.gpu
def test_preemption_with_sharing_on_the_gpu(model_folders):
    _preemption_with_sharing(model_folders["tiny-a"], "tiny-a", "cuda:0")


# ---- the copy kernel alone ------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(3, 9, 2, 2, 4, 16), (1, 5, 2, 1, 8, 32), (28, 40, 2, 8, 16, 128), (2, 7, 2, 3, 1, 5)])
def test_copy_pages_kernel(dtype, shape):
    import ref_ops
    from qwen_engine_b200 import ops
    g = torch.Generator().manual_seed(3)
    cache = torch.randn(shape, generator=g).to(dtype)
    n_pages = shape[1]
    pairs = [0, n_pages - 1, 2, 1, 3, 3, n_pages, 0, -1, 2]       # the last three: same page, outside the group (passed over)
    want = cache.clone()
    ref_ops.copy_pages(want, torch.tensor(pairs[:4], dtype=torch.int32))
    dev = cache.to("cuda:0")
    ops.copy_pages(dev, torch.tensor(pairs, dtype=torch.int32, device="cuda:0"))
    assert torch.equal(dev.cpu(), want)
