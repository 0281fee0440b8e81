"""Generation through the Python entry point on the GPU against the plain implementation:
greedy and sampled workloads of the two tiny configurations, long decoding, the first tokens of
a sequence, preemption, and the command line."""
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_qwen3
from helpers import assert_close_logits, make_engine, plain_logits, plain_sampled_generate, random_tokens
from qwen_engine_b200.sampling import SamplingParams

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plain_greedy(folder, prompt, steps):
    cfg, w = plain_qwen3.read_model_folder(folder)
    return plain_qwen3.greedy_generate(cfg, w, prompt, steps)


def _margin_ok(folder, prompt, out, min_margin):
    """Whether every greedy choice of the plain implementation was clear by min_margin (else a
    bfloat16 run may rightly pick the runner-up)."""
    toks = list(prompt)
    for t in out:
        top2 = torch.topk(plain_logits(folder, toks)[-1], 2).values
        if float(top2[0] - top2[1]) < min_margin:
            return False
        toks.append(t)
    return True


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_greedy_generation_float32(model_folders, name):
    from qwen_engine_b200 import LLM
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, n, 70 + n) for n in (5, 9, 13)]
    llm = LLM(folder, dtype="float32", block_size=helpers.TINY[name]["page"], max_model_len=64)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=8))
    for o, p in zip(outs, prompts):
        assert o.prompt_token_ids == p and o.finish_reason == "length"
        assert o.output_token_ids == _plain_greedy(folder, p, 8)


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_greedy_generation_bfloat16(model_folders, name):
    """In bfloat16 the tokens are compared where the plain choice is clear; prompts whose plain
    run has a near tie are skipped, not excused."""
    from qwen_engine_b200 import LLM
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    llm = LLM(folder, dtype="bfloat16", block_size=helpers.TINY[name]["page"], max_model_len=64)
    checked = 0
    for seed in range(40):
        p = random_tokens(V, 6 + seed, 300 + seed)
        want = _plain_greedy(folder, p, 8)
        if not _margin_ok(folder, p, want, 2 * helpers.TOL[torch.bfloat16] * max(1.0, float(plain_logits(folder, p).abs().max()))):
            continue
        got = llm.generate([p], SamplingParams(max_new_tokens=8))[0].output_token_ids
        assert got == want
        checked += 1
    assert checked >= 2


def test_sampled_workload_of_tiny_b(model_folders):
    name = "tiny-b"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    common = random_tokens(V, 16, 80)
    prompts = [random_tokens(V, 3, 81), common + random_tokens(V, 1, 82), common + random_tokens(V, 8, 83),
               random_tokens(V, 31, 84)]
    eng = make_engine(folder, name, torch.float32, prefill_chunk_size=7, max_num_batched_tokens=16, seed=5,
                      max_num_seqs=2)   # the third request is admitted once the second has filled its pages
    sp = SamplingParams(max_new_tokens=6, temperature=0.8, top_k=20, seed=5)
    ids = [eng.add_request(p, sp) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for i, p in zip(ids, prompts):
        assert outs[i].output_token_ids == plain_sampled_generate(folder, p, 6, 0.8, 20, 5, i)
    assert eng.stats.prefix_hit_tokens >= 16


def test_preemption_on_the_gpu(model_folders):
    name = "tiny-a"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, 10, 90 + i) for i in range(3)]
    eng = make_engine(folder, name, torch.float32, num_blocks=12, max_model_len=32, enable_prefix_cache=False)
    ids = eng.submit(prompts, max_new_tokens=14)
    outs = {o.request_id: o for o in eng.serving()}
    assert eng.stats.preemptions >= 1
    for i, p in zip(ids, prompts):
        assert outs[i].output_token_ids == _plain_greedy(folder, p, 14)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_steps_launched_ahead_change_nothing_on_the_gpu(model_folders, dtype):
    """run_ahead (a decode step launched before the host has read the tokens of the step before it,
    which it takes from the device) against the step-by-step engine: the same tokens and finish
    reasons for requests that end by a count and by a stop token, replayed decode steps included."""
    from qwen_engine_b200.sampling import SamplingParams as SP
    name = "tiny-b"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, n, 130 + n) for n in (6, 19, 4, 33)]
    lengths = [7, 30, 12, 24]
    first = {}
    results = {}
    for ahead in (False, True):
        eng = helpers.make_engine(folder, name, dtype, run_ahead=ahead, max_model_len=96)
        for i, (p, n) in enumerate(zip(prompts, lengths)):
            stops = (first[i][5],) if (ahead and i in (1, 3)) else ()
            eng.add_request(p, SP(max_new_tokens=n, stop_token_ids=stops, ignore_eos=True,
                                  temperature=0.7 if i == 2 else 0.0, top_k=8 if i == 2 else 0, seed=3))
        launched_ahead = 0
        done = []
        while eng.has_work():
            done.extend(eng.step())
            launched_ahead += eng._flight is not None
        assert (launched_ahead > 0) == ahead
        assert eng.cache.pages_in_use() == 0
        eng.cache.check_invariants()
        results[ahead] = {s.seq_id: (list(s.output_token_ids), s.finish_reason) for s in done}
        if not ahead:
            first = {i: results[False][i][0] for i in range(len(prompts))}
    for i, n in enumerate(lengths):
        want, reason = results[False][i]
        assert reason == "length" and len(want) == n
        got, got_reason = results[True][i]
        if i in (1, 3):
            cut = want.index(want[5]) + 1
            assert got == want[:cut] and got_reason == "stop"
        else:
            assert got == want and got_reason == "length"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding(model_folders, dtype):
    """400 tokens decoded one by one after a short prompt (teacher-forced, so that both dtypes
    walk the same path); logits compared every 25 steps and at the end."""
    name = "tiny-b"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    toks = random_tokens(V, 420, 123)
    rep = helpers.make_replayer(folder, name, dtype, 448)
    steps = [{"entries": [{"id": "r", "tokens": toks[:20], "want": [19]}]}]
    for i in range(20, 420):
        steps.append({"entries": [{"id": "r", "tokens": [toks[i]], "want": [0] if (i % 25 == 0 or i == 419) else []}]})
    got = helpers.run_steps(rep, steps)
    helpers.check_requests(got, folder, {"r": toks}, dtype, "long decode")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny-a", "tiny-b", "tiny-c"])
def test_first_tokens_of_a_sequence(model_folders, name, dtype):
    """Positions 0, 1, 2: a single token as a whole request, then one by one."""
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    toks = random_tokens(V, 3, 77)
    rep = helpers.make_replayer(folder, name, dtype, 128)
    got = helpers.run_steps(rep, [{"entries": [{"id": "r", "tokens": [t], "want": [0]}]} for t in toks])
    helpers.check_requests(got, folder, {"r": toks}, dtype, "first tokens")
    got = helpers.run_steps(rep, [{"entries": [{"id": "s", "tokens": toks[:1], "want": [0]}], "end": ["s"]}])
    assert_close_logits(got["s"][0][None], plain_logits(folder, toks[:1]), dtype, "one token")


def test_command_line(model_folders):
    name = "tiny-a"
    folder = model_folders[name]
    prompt = random_tokens(helpers.vocab_of(name), 7, 5)
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "main.py"), "--model-name-or-path", folder, "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5", "--block-size", "4", "--stats", "--profile"],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = " ".join(str(t) for t in _plain_greedy(folder, prompt, 5))
    assert want in proc.stdout
    # --profile: one prompt portion of 7 tokens, then 4 steps of one decoded token, each with its device time
    rows = {l.split()[0]: l.split() for l in proc.stdout.splitlines() if l.split() and l.split()[0] in ("prefill", "decode", "mixed")}
    assert rows["prefill"][1:3] == ["1", "7"] and rows["decode"][1:3] == ["4", "4"], proc.stdout[-1500:]
    assert float(rows["prefill"][3]) > 0 and float(rows["decode"][3]) > 0


@pytest.mark.parametrize("fused", [True, False])
def test_norm_and_rotation_with_head_size_128(tmp_path, monkeypatch, fused):
    """Prompt portions of many rows with head size 128 in bfloat16 take their rotation angles from a table that
    the first layer makes for the step and every layer reads (it must outlive the layers' own scratch, also in
    steps whose scratch no longer grows: portions of a size that came before); and with ``fused`` the per-head
    norm, the rotation and the cache write happen in the epilogue of the QKV product (ops.linear_qkv_rope).
    A prompt run whole, in portions of changing and of repeated sizes (some too small for table and
    epilogue: the separate kernel with its own angles), then decoded tokens that read the cache all of these
    left behind, against the plain implementation; and the ways of cutting against each other."""
    from qwen_engine_b200 import ops
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.runner import StepEntry
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.weights import write_model_folder
    raw = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=200, num_attention_heads=6,
               num_key_value_heads=3, head_dim=128, intermediate_size=272, vocab_size=611, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
    folder = write_model_folder(config_from_dict(raw), str(tmp_path / "m"), seed=9, std=0.05, norm_std=0.1)
    tokens = random_tokens(611, 700, 77)
    want = helpers.plain_logits(folder, tokens)
    monkeypatch.setattr(ops, "QKV_ROPE_MIN_TILES", 1 if fused else 10 ** 9)
    used = []
    real = ops.linear_qkv_rope
    monkeypatch.setattr(ops, "linear_qkv_rope", lambda *a, **k: (used.append(a[0].shape[0]), real(*a, **k))[1])
    got = []
    for cut in ([660], [100, 37, 200, 2, 321], [100, 100, 100, 100, 100, 100, 64]):
        loaded = load_model(folder, torch.bfloat16, "cuda:0", 16, 64, 4, enable_prefix_cache=False)
        runner, rc = loaded.runner, loaded.cache.open(0)
        rows, at = [], 0
        for n in cut:
            rows.append(runner.step([StepEntry(rc, tokens[at:at + n], list(range(n)))]).float().cpu().clone())
            at += n
        for t in tokens[at:]:
            rows.append(runner.step([StepEntry(rc, [t], [0])]).float().cpu().clone())
        got.append(torch.cat(rows))
        helpers.assert_close_logits(got[-1], want, torch.bfloat16, f"cut {cut}")
    if fused:
        assert 660 in used and 321 in used and 100 in used and 64 not in used and 37 not in used and 2 not in used, used
    else:
        assert not used
    assert ops.tcgen05_status() == 0
    scale = max(1.0, float(want.abs().max()))
    for other in got[1:]:
        assert float((got[0] - other).abs().max()) <= 2e-2 * scale


def test_cache_sized_from_a_share_of_the_devices_memory(model_folders):
    """``gpu_memory_fraction`` instead of ``num_blocks``: the cache takes what that share of the device's memory
    leaves after the weights and a reserve; generation is what it is with any other cache size."""
    from qwen_engine_b200 import LLM
    name = "tiny-a"
    folder = model_folders[name]
    prompt = random_tokens(helpers.vocab_of(name), 9, 75)
    free, total = torch.cuda.mem_get_info()
    llm = LLM(folder, dtype="float32", block_size=helpers.TINY[name]["page"], max_model_len=64, gpu_memory_fraction=0.05)
    group = llm.engine.cache.paged_groups[0]
    page_bytes = group.tensor[:, 0].numel() * group.tensor.element_size()
    assert 0.01 * total < group.pool.num_pages * page_bytes <= 0.05 * total
    out = llm.generate([prompt], SamplingParams(max_new_tokens=6))[0]
    assert out.output_token_ids == _plain_greedy(folder, prompt, 6)
    del llm
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny-b", "tiny-d"])
def test_prompt_portions_and_admissions_in_steps_launched_ahead_on_the_gpu(model_folders, name, dtype):
    """Arrivals while others decode, prompts in small portions, few slots: steps launched ahead carry prompt
    portions, admissions and decoded tokens together and change no token (against the step-by-step engine; in
    32-bit against the plain implementation too)."""
    from test_generate_host import _arrivals_with_portions, _plain_greedy
    folder = model_folders[name]
    plain_of = (lambda p, n: _plain_greedy(folder, p, n)) if dtype == torch.float32 else None
    _arrivals_with_portions(folder, name, dtype, "cuda:0", plain_of)
