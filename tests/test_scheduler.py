"""The scheduler's decisions, with a fake step function (no model): admission in arrival order,
portions under a token budget, decoding first, finishing and freeing, and what happens when
pages run out (the newest request is preempted and recomputed later)."""
import pytest
import torch

from qwen_engine_b200.cache import CacheManager, PagedKVSpec
from qwen_engine_b200.engine.scheduler import Scheduler
from qwen_engine_b200.engine.sequence import Sequence, SequenceStatus
from qwen_engine_b200.sampling import SamplingParams


def _setup(num_pages=16, page=4, max_seqs=4, budget=16, chunk=None, max_len=64, eos=None, prefix=True):
    cm = CacheManager([PagedKVSpec(1, 8)], page, num_pages, max_seqs, torch.float32, "cpu", enable_prefix_cache=prefix)
    return cm, Scheduler(cm, max_seqs, budget, chunk, max_len, eos_token_id=eos)


def _seq(i, n, max_new=4, base=100, **kw):
    return Sequence(i, [base * (i + 1) + j for j in range(n)], SamplingParams(max_new_tokens=max_new, **kw))


def _fake_step(cm, out, token_of=lambda seq: 7):
    """What the engine does around a step, without a model."""
    sampled = {}
    for sch in out.scheduled:
        cm.append(sch.seq.cache, sch.seq.get_tokens(sch.start, sch.num_tokens))
        cm.commit(sch.seq.cache)
        if sch.wants_logits:
            sampled[sch.seq.seq_id] = token_of(sch.seq)
    cm.check_invariants()
    return sampled


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first():
    cm, s = _setup(budget=10, num_pages=32)
    a, b = _seq(0, 14), _seq(1, 5)
    s.add(a), s.add(b)
    out = s.schedule()
    assert [(x.seq.seq_id, x.start, x.num_tokens, x.wants_logits) for x in out.scheduled] == [(0, 0, 10, False)]
    s.update(out, _fake_step(cm, out))
    out = s.schedule()                                 # rest of a (4), then b whole (5) within 10
    assert [(x.seq.seq_id, x.start, x.num_tokens, x.wants_logits) for x in out.scheduled] == [(0, 10, 4, True), (1, 0, 5, True)]
    s.update(out, _fake_step(cm, out))
    assert a.output_token_ids == [7] and b.output_token_ids == [7]
    c = _seq(2, 30)
    s.add(c)
    out = s.schedule()                                 # two decodes first, the new prompt gets what is left
    assert [(x.seq.seq_id, x.num_tokens) for x in out.scheduled] == [(0, 1), (1, 1), (2, 8)]
    assert out.scheduled[2].wants_logits is False


def test_portion_size_limit_and_two_token_portions():
    cm, s = _setup(budget=64, chunk=2, num_pages=32)
    a = _seq(0, 5)
    s.add(a)
    sizes = []
    while not a.output_token_ids:
        out = s.schedule()
        sizes.append(out.scheduled[0].num_tokens)
        s.update(out, _fake_step(cm, out))
    assert sizes == [2, 2, 1]


def test_admission_is_in_arrival_order_and_bounded_by_slots():
    cm, s = _setup(max_seqs=2, budget=64, num_pages=32)
    seqs = [_seq(i, 3) for i in range(4)]
    for q in seqs:
        s.add(q)
    out = s.schedule()
    assert [x.seq.seq_id for x in out.scheduled] == [0, 1] and len(s.waiting) == 2
    s.update(out, _fake_step(cm, out))
    out = s.schedule()
    assert [x.seq.seq_id for x in out.scheduled] == [0, 1]      # no free slot for request 2


def test_a_waiting_request_is_not_overtaken():
    cm, s = _setup(num_pages=6, budget=64, max_len=24)          # 24 tokens in all
    big, small = _seq(0, 20), _seq(1, 2)
    first = _seq(2, 8)
    s.add(first)
    out = s.schedule()
    s.update(out, _fake_step(cm, out))
    s.add(big), s.add(small)
    out = s.schedule()                                          # big does not fit; small must not jump the queue
    assert [x.seq.seq_id for x in out.scheduled] == [2]
    assert [q.seq_id for q in s.waiting] == [0, 1]


def test_finishing_frees_pages_and_slot_at_once():
    cm, s = _setup(max_seqs=2, budget=64)
    a = _seq(0, 6, max_new=2)
    s.add(a)
    out = s.schedule()
    assert s.update(out, _fake_step(cm, out)) == []
    assert cm.pages_in_use() == 2
    out = s.schedule()
    ended = s.update(out, _fake_step(cm, out))
    assert ended == [a] and a.finish_reason == "length" and a.status is SequenceStatus.FINISHED
    assert cm.pages_in_use() == 0 and cm.slots.num_free == 2 and not s.has_work()


def test_stop_reasons():
    cm, s = _setup(eos=7, max_len=10, budget=64)
    a = _seq(0, 3, max_new=50)
    s.add(a)
    out = s.schedule()
    assert s.update(out, _fake_step(cm, out)) == [a] and a.finish_reason == "stop"
    b = _seq(1, 3, max_new=50, ignore_eos=True)
    s.add(b)
    for _ in range(20):
        if not s.has_work():
            break
        out = s.schedule()
        s.update(out, _fake_step(cm, out))
    assert b.finish_reason == "length" and b.total_len == 10        # the model's length limit
    c = _seq(2, 3, max_new=50, ignore_eos=True, stop_token_ids=(9,))
    s.add(c)
    out = s.schedule()
    assert s.update(out, _fake_step(cm, out, lambda q: 9)) == [c] and c.finish_reason == "stop"


def test_requests_that_can_never_run_are_refused_at_once():
    cm, s = _setup(num_pages=4, max_len=64)
    with pytest.raises(ValueError, match="pages"):
        s.add(_seq(0, 3))
    cm, s = _setup(max_len=8)
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(_seq(0, 8))
    with pytest.raises(ValueError):
        s.add(Sequence(1, [], SamplingParams()))


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    cm, s = _setup(num_pages=6, page=4, max_seqs=3, budget=64, max_len=24, prefix=False)
    a, b = _seq(0, 8, max_new=12), _seq(1, 8, max_new=12)
    s.add(a), s.add(b)
    out = s.schedule()
    s.update(out, _fake_step(cm, out))                  # 2 + 2 pages, both full; 2 pages free
    preempted_at = None
    for step in range(40):
        if not s.has_work():
            break
        out = s.schedule()
        if out.preempted and preempted_at is None:
            preempted_at = step
            assert out.preempted == [b], "the request admitted last is the one that goes"
            assert b.status is SequenceStatus.WAITING and b.cache is None and s.waiting[0] is b
            assert b.output_token_ids, "it keeps the tokens it has generated"
            assert [x.seq for x in out.scheduled] == [a]
            assert out.admitted == [], "no admission in a step that had to preempt"
        s.update(out, _fake_step(cm, out))
    assert preempted_at is not None and s.num_preemptions >= 1
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert len(a.output_token_ids) == 12 and len(b.output_token_ids) == 12
    assert b.num_preemptions >= 1
    assert cm.pages_in_use() == 0
    cm.check_invariants()


def test_a_lone_request_that_cannot_fit_is_an_error():
    cm, s = _setup(num_pages=16, page=4, max_len=64, budget=64, prefix=False)
    a = _seq(0, 8, max_new=40)
    s.add(a)
    hog = cm.open("hog")                                # something outside the scheduler holds the pages
    cm.append(hog, list(range(52)))
    cm.commit(hog)
    out = s.schedule()
    s.update(out, _fake_step(cm, out))                  # 13 + 2 pages used, 1 free
    with pytest.raises(RuntimeError, match="single running request"):
        for _ in range(12):
            out = s.schedule()
            s.update(out, _fake_step(cm, out))


def test_prefix_hits_are_counted_and_preempted_work_comes_back_cheaply():
    cm, s = _setup(num_pages=32, budget=64)
    a = Sequence(0, list(range(10)), SamplingParams(max_new_tokens=1))
    s.add(a)
    out = s.schedule()
    s.update(out, _fake_step(cm, out))
    b = Sequence(1, list(range(8)) + [50, 51, 52], SamplingParams(max_new_tokens=1))
    s.add(b)
    out = s.schedule()
    assert [(x.start, x.num_tokens) for x in out.scheduled] == [(8, 3)]
    assert b.shared_prefix_len == 8 and s.prefix_hit_tokens == 8


def test_tokens_with_a_place_kept_for_them_holds_and_late_stops():
    """What the engine does when it launches a step ahead: the requests' outputs get a place
    (UNKNOWN_TOKEN) for the token on its way, a request that ends by a count with that token is
    held back from the next step, the step launched ahead is scheduled from the lengths alone,
    update() puts the tokens into their places, and a request that ended by a stop token is
    passed over when the step that still carried it reports."""
    from qwen_engine_b200.cache.manager import UNKNOWN_TOKEN
    cm, s = _setup(num_pages=32)
    a = _seq(0, 3, max_new=2)                          # ends by the count after two tokens
    b = _seq(1, 5, max_new=9, stop_token_ids=(9,), ignore_eos=True)
    c = _seq(2, 4, max_new=9)
    for x in (a, b, c):
        s.add(x)
    first = s.schedule()
    assert [x.num_tokens for x in first.scheduled] == [3, 5, 4]
    s.update(first, _fake_step(cm, first, lambda seq: 7))
    cur = s.schedule()                                  # the step whose tokens are "on the device"
    step_tokens = _fake_step(cm, cur, lambda seq: 9 if seq is b else 8)
    # ahead: places for cur's tokens; a ends with its second token whatever it is
    placed = {}
    for sch in cur.scheduled:
        sch.seq.hold = s.ends_by_length_after(sch.seq, 1)
        placed[sch.seq.seq_id] = sch.seq.output_len
        sch.seq.output_token_ids.append(UNKNOWN_TOKEN)
    assert a.hold and not b.hold and not c.hold
    ahead = s.schedule()
    assert [x.seq.seq_id for x in ahead.scheduled] == [1, 2] and not ahead.preempted and not ahead.admitted
    assert ahead.scheduled[0].seq.get_tokens(ahead.scheduled[0].start, 1) == [UNKNOWN_TOKEN]
    ahead_tokens = _fake_step(cm, ahead, lambda seq: 5)
    assert b.cache.first_unknown == b.prompt_len + 1
    # cur's tokens arrive: into their places; a ends by the count, b by its stop token
    ended = s.update(cur, step_tokens, placed)
    assert {x.seq_id: x.finish_reason for x in ended} == {0: "length", 1: "stop"}
    assert a.output_token_ids == [7, 8] and b.output_token_ids == [7, 9] and c.output_token_ids == [7, 8]
    assert c.cache.first_unknown is None and c.cache.tokens[-1] == 8
    # the step launched ahead reports: b is passed over, c goes on
    ended = s.update(ahead, ahead_tokens)
    assert ended == [] and b.output_token_ids == [7, 9] and c.output_token_ids == [7, 8, 5]
    cm.check_invariants()
    assert [x.seq_id for x in s.running] == [2]
    with pytest.raises(RuntimeError):
        s.update(cur, {2: 1}, {2: 0})                   # no place is waiting there


def test_a_step_scheduled_ahead_leaves_out_who_finds_no_pages_and_may_admit():
    """``schedule(may_preempt=False)`` is what the engine calls while a step is in flight: a running request that
    needs a page when none is free is left out (nobody is preempted, its turn comes when pages are back or when
    the next step is scheduled with preemption allowed); prompt portions and admissions go in as in any step."""
    cm, s = _setup(num_pages=7, page=4, max_seqs=3, budget=64, max_len=24, prefix=False)
    a, b = _seq(0, 8, max_new=12), _seq(1, 7, max_new=12)
    s.add(a), s.add(b)
    out = s.schedule()
    s.update(out, _fake_step(cm, out))                  # a: 2 pages, full; b: 2 pages, one slot left; 3 pages free
    c = _seq(2, 8, max_new=2)
    s.add(c)
    out = s.schedule(may_preempt=False)                 # a takes a page, b needs none, c is admitted on the last two
    assert [x.seq.seq_id for x in out.scheduled] == [0, 1, 2] and out.admitted == [c] and not out.preempted
    assert out.scheduled[2].num_tokens == 8
    s.update(out, _fake_step(cm, out))
    free = cm.paged_groups[0].pool.num_free
    out = s.schedule(may_preempt=False)
    who = [x.seq.seq_id for x in out.scheduled]
    assert not out.preempted and s.num_preemptions == 0
    needs_page = [q.seq_id for q in (a, b, c) if cm.pages_needed(q.cache, 1)[0] > 0]
    assert len(needs_page) > free, "the case is meant to run out of pages"
    assert all(i in who for i in (0, 1, 2) if i not in needs_page), "who needs no page runs"
    assert len([i for i in who if i in needs_page]) == free, "the free pages go to the oldest that need one"
    s.update(out, _fake_step(cm, out))
    # when nobody can go on the step scheduled ahead is empty, and the next one, with preemption, makes room
    for _ in range(40):
        if not s.has_work():
            break
        out = s.schedule(may_preempt=False)
        if not out.scheduled:
            out = s.schedule()
            assert out.preempted
        s.update(out, _fake_step(cm, out))
    assert not s.has_work() and s.num_preemptions >= 1
    assert [len(q.output_token_ids) for q in (a, b, c)] == [12, 12, 2]
    assert cm.pages_in_use() == 0
    cm.check_invariants()


def test_any_of_several_end_of_sequence_ids_stops_a_request():
    cm, s = _setup(eos=(7, 9))
    a, b, c = _seq(0, 3, max_new=5), _seq(1, 3, max_new=5), _seq(2, 3, max_new=5, ignore_eos=True)
    for q in (a, b, c):
        s.add(q)
    out = s.schedule()
    ended = s.update(out, _fake_step(cm, out, token_of=lambda seq: (7, 9, 9)[seq.seq_id]))
    assert {q.seq_id: q.finish_reason for q in ended} == {0: "stop", 1: "stop"}
    assert c.status is SequenceStatus.RUNNING
