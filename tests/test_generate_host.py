"""Generation through the engine on the CPU (plain operations in the place of the kernels): the
scheduler, the step function, the cache and the sampler's host side against the plain
implementation.  The same workloads run on the GPU in tests/test_generate_gpu.py."""
import pytest
import torch

import helpers
import plain_qwen3
from helpers import make_engine, plain_sampled_generate, random_tokens
from qwen_engine_b200.sampling import SamplingParams, uniform_for

F32 = torch.float32


def _plain_greedy(folder, prompt, steps):
    cfg, w = plain_qwen3.read_model_folder(folder)
    return plain_qwen3.greedy_generate(cfg, w, prompt, steps)


def test_greedy_workload_of_tiny_a(model_folders, cpu_ops):
    """Three prompts of 5, 9 and 13 tokens, 8 greedy steps each."""
    folder = model_folders["tiny-a"]
    V = helpers.vocab_of("tiny-a")
    prompts = [random_tokens(V, n, 70 + n) for n in (5, 9, 13)]
    eng = make_engine(folder, "tiny-a", F32, device="cpu")
    ids = eng.submit(prompts, max_new_tokens=8)
    outs = {o.request_id: o for o in eng.serving()}
    for i, p in zip(ids, prompts):
        assert outs[i].output_token_ids == _plain_greedy(folder, p, 8)
        assert outs[i].finish_reason == "length"
    assert eng.cache.pages_in_use() == 0


def test_sampled_workload_of_tiny_b(model_folders, cpu_ops):
    """Four prompts of 3, 17, 24 and 31 tokens, two sharing 16 tokens; portions of 7 mixed with
    decoded tokens; 6 steps at temperature 0.8 with a fixed seed."""
    name = "tiny-b"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    common = random_tokens(V, 16, 80)
    prompts = [random_tokens(V, 3, 81), common + random_tokens(V, 1, 82), common + random_tokens(V, 8, 83),
               random_tokens(V, 31, 84)]
    eng = make_engine(folder, name, F32, device="cpu", prefill_chunk_size=7, max_num_batched_tokens=16, seed=5,
                      max_num_seqs=2)   # the third request is admitted once the second has filled its pages
    sp = SamplingParams(max_new_tokens=6, temperature=0.8, top_k=20, seed=5)
    ids = [eng.add_request(p, sp) for p in prompts]
    outs = {o.request_id: o for o in eng.serving()}
    for i, p in zip(ids, prompts):
        assert outs[i].output_token_ids == plain_sampled_generate(folder, p, 6, 0.8, 20, 5, i)
    assert eng.stats.prefix_hit_tokens >= 16
    assert eng.stats.prefill_tokens + eng.stats.prefix_hit_tokens >= sum(len(p) for p in prompts)


def test_preemption_does_not_change_the_tokens(model_folders, cpu_ops):
    name = "tiny-a"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, 10, 90 + i) for i in range(3)]
    # 3 requests of up to 10 + 14 tokens need 18 pages of 4; with 12 someone has to wait
    eng = make_engine(folder, name, F32, device="cpu", num_blocks=12, max_model_len=32, enable_prefix_cache=False)
    ids = eng.submit(prompts, max_new_tokens=14)
    outs = {o.request_id: o for o in eng.serving()}
    assert eng.stats.preemptions >= 1
    for i, p in zip(ids, prompts):
        assert outs[i].output_token_ids == _plain_greedy(folder, p, 14)
    assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("prefix_cache", [False, True])
def test_steps_launched_ahead_change_nothing(model_folders, cpu_ops, prefix_cache):
    """With run_ahead a decode step is launched before the host has read the step before it.  The
    outputs, finish reasons and final page counts are those of the step-by-step engine: requests of
    different lengths that end by a count (known beforehand, not carried along) and by a stop token
    (found out one step late: the token of the step launched ahead is dropped); pages of 4 tokens fill
    up and are registered for sharing while a token's id is still on the device."""
    name = "tiny-a"
    folder = model_folders[name]
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, n, 120 + n) for n in (6, 9, 4, 11)]
    lengths = [5, 12, 9, 16]
    results = {}
    for ahead in (False, True):
        eng = make_engine(folder, name, F32, device="cpu", run_ahead=ahead, enable_prefix_cache=prefix_cache,
                          max_model_len=64)
        # the stop token of each request: what the plain implementation produces at its 4th step
        # (for the last request none: it ends by the count)
        ids = []
        for i, (p, n) in enumerate(zip(prompts, lengths)):
            plain = _plain_greedy(folder, p, n)
            stops = (plain[3],) if i in (1, 2) else ()
            ids.append(eng.add_request(p, SamplingParams(max_new_tokens=n, stop_token_ids=stops, ignore_eos=True)))
        launched_ahead = 0
        done = []
        while eng.has_work():
            done.extend(eng.step())
            launched_ahead += eng._flight is not None
        eng.cache.check_invariants()
        assert eng.cache.pages_in_use() == 0
        assert (launched_ahead > 0) == ahead
        results[ahead] = {s.seq_id: (list(s.output_token_ids), s.finish_reason) for s in done}
        assert len(done) == len(prompts)
    assert results[True] == results[False]
    for i, (p, n) in enumerate(zip(prompts, lengths)):
        toks, reason = results[True][i]
        plain = _plain_greedy(folder, p, n)
        if i in (1, 2):
            cut = plain.index(plain[3]) + 1
            assert toks == plain[:cut] and reason == "stop"
        else:
            assert toks == plain and reason == "length"


def _arrivals_with_portions(folder, name, dtype, device, plain_of):
    """Requests that arrive while others decode, prompts in portions of at most 6 tokens under a budget of 8, three
    slots, few pages: with steps launched ahead, prompt portions, admissions and decoded tokens go into one step
    that is scheduled while the step before it is still in flight; tokens and finish reasons equal the
    step-by-step engine's and (``plain_of`` given) the plain implementation's."""
    V = helpers.vocab_of(name)
    prompts = [random_tokens(V, n, 300 + n) for n in (23, 9, 31, 5, 17)]
    lengths = [9, 14, 6, 11, 8]
    arrive_at = [0, 0, 3, 5, 9]
    results = {}
    for ahead in (False, True):
        eng = make_engine(folder, name, dtype, device=device, run_ahead=ahead, max_model_len=64, max_num_seqs=3,
                          max_num_batched_tokens=8, prefill_chunk_size=6, num_blocks=28)
        done, steps, mixed_ahead, admitted_ahead = [], 0, 0, 0
        added = 0
        while eng.has_work() or added < len(prompts):
            while added < len(prompts) and arrive_at[added] <= steps:
                eng.add_request(prompts[added], SamplingParams(max_new_tokens=lengths[added], ignore_eos=True))
                added += 1
            waiting_before = len(eng.scheduler.waiting)
            flight_before = eng._flight
            done.extend(eng.step())
            steps += 1
            fl = eng._flight
            if fl is not None and fl is not flight_before:
                mixed_ahead += fl.prefill_tokens > 0 and fl.decode_tokens > 0
                admitted_ahead += len(fl.out.admitted)
        eng.cache.check_invariants()
        assert eng.cache.pages_in_use() == 0
        if ahead:
            assert mixed_ahead > 0, "no step with prompt portions beside decoded tokens was launched ahead"
            assert admitted_ahead > 0, "no request was admitted by a step launched ahead"
        else:
            assert mixed_ahead == 0 and admitted_ahead == 0
        results[ahead] = {s.seq_id: (list(s.output_token_ids), s.finish_reason) for s in done}
        assert len(done) == len(prompts)
    assert results[True] == results[False]
    for i, (p, n) in enumerate(zip(prompts, lengths)):
        if plain_of is not None:
            assert results[True][i] == (plain_of(p, n), "length")


def test_prompt_portions_and_admissions_go_into_steps_launched_ahead(model_folders, cpu_ops):
    folder = model_folders["tiny-a"]
    _arrivals_with_portions(folder, "tiny-a", F32, "cpu", lambda p, n: _plain_greedy(folder, p, n))


def test_uniform_numbers_are_a_function_of_seed_request_and_position():
    assert uniform_for(1, 2, 3) == uniform_for(1, 2, 3)
    vals = {uniform_for(s, r, p) for s in range(3) for r in range(3) for p in range(3)}
    assert len(vals) == 27 and all(0.0 <= v < 1.0 for v in vals)
    assert torch.tensor(uniform_for(9, 9, 9), dtype=torch.float32).item() == uniform_for(9, 9, 9)


def test_bad_requests_are_refused(model_folders, cpu_ops):
    eng = make_engine(model_folders["tiny-a"], "tiny-a", F32, device="cpu")
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([1, 2, 999999])
    with pytest.raises(ValueError, match="tokenizer"):
        eng.add_request("some text")
    with pytest.raises(ValueError):
        eng.add_request(list(range(1, 200)))


def test_profile_option_on_the_cpu_and_its_table(model_folders, cpu_ops):
    """``EngineConfig.profile`` times steps with CUDA events: on the CPU there is nothing to time, the
    engine runs as without it and says so; the table of a filled profile has a row per kind of step."""
    from qwen_engine_b200.engine.llm import EngineStats
    folder = model_folders["tiny-a"]
    prompt = random_tokens(helpers.vocab_of("tiny-a"), 9, 71)
    eng = make_engine(folder, "tiny-a", F32, device="cpu", profile=True)
    eng.submit([prompt], max_new_tokens=4)
    outs = eng.serving()
    assert outs[0].output_token_ids == _plain_greedy(folder, prompt, 4)
    assert eng.stats.profile is None and "no profile" in eng.stats.profile_table()
    st = EngineStats(profile={"prefill": {"steps": 2, "tokens": 4096, "device_ms": 8.0},
                              "decode": {"steps": 10, "tokens": 80, "device_ms": 10.0}})
    lines = st.profile_table().splitlines()
    assert lines[1].split() == ["prefill", "2", "4096", "8.00", "4.000", "512000"]
    assert lines[2].split() == ["decode", "10", "80", "10.00", "1.000", "8000"]


def test_a_wait_that_ran_out_on_the_device_surfaces_as_an_error(model_folders, cpu_ops, monkeypatch):
    """Kernels give up a bounded wait by returning without their output and leaving a code in a status
    word; the engine reads the words when ``serving`` is through and raises, instead of handing out the
    tokens of such a step as if they were right."""
    from qwen_engine_b200 import ops
    eng = make_engine(model_folders["tiny-a"], "tiny-a", F32, device="cpu")
    eng._checks_device = True                         # as on a CUDA device
    cleared = []
    monkeypatch.setattr(ops, "device_status", lambda: {} if cleared else {"gemm_tc": 2})
    monkeypatch.setattr(ops, "clear_device_status", lambda: cleared.append(True))
    eng.submit([[1, 2, 3]], max_new_tokens=2)
    with pytest.raises(ops.DeviceWaitTimeout, match="gemm_tc .code 2."):
        eng.serving()
    assert cleared
    eng.check_device()                                  # cleared: the next check passes


def test_a_length_limit_beyond_the_models_positions_is_refused_at_construction(model_folders, cpu_ops):
    """tiny-a has 512 positions: an engine that would let a request grow past them is refused when it is
    built, not in the middle of serving, where the other live requests would be lost with it."""
    with pytest.raises(ValueError, match="max_position_embeddings = 512"):
        make_engine(model_folders["tiny-a"], "tiny-a", F32, device="cpu", max_model_len=513, num_blocks=8)
    make_engine(model_folders["tiny-a"], "tiny-a", F32, device="cpu", max_model_len=512, num_blocks=8)
