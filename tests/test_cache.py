"""The cache manager on the host: no page lost, held twice or freed twice under random orders
of requests; sharing of full pages, the private copy of a fully shared prompt's last page,
reuse of freed pages, windows that give pages back early, state slots."""
import random

import pytest
import torch

from qwen_engine_b200.cache import (CacheManager, FixedStateSpec, OutOfPages, OutOfSlots, PagedKVSpec,
                                    PagePool, StateSlotPool, hash_block)

F32 = torch.float32


def _manager(num_pages=16, page=4, slots=4, specs=None, prefix=True):
    specs = specs or [PagedKVSpec(2, 8)] * 3
    return CacheManager(specs, page, num_pages, slots, F32, "cpu", enable_prefix_cache=prefix)


def _feed(cm, rc, tokens):
    cm.append(rc, tokens)
    cm.commit(rc)


def test_pool_hands_out_page_zero_first_and_reuses_freed_pages():
    pool = PagePool(4, 4)
    a, b = pool.allocate(), pool.allocate()
    assert (a, b) == (0, 1)
    pool.release(a)
    assert pool.allocate() == 0                      # a freed page is used again
    pool.check_invariants({0: 1, 1: 1})


def test_pool_refuses_double_free_and_bad_ids():
    pool = PagePool(2, 4)
    p = pool.allocate()
    pool.release(p)
    with pytest.raises(RuntimeError):
        pool.release(p)
    with pytest.raises(ValueError):
        pool.release(7)
    with pytest.raises(RuntimeError):
        pool.retain(1)                               # never handed out
    pool.allocate(), pool.allocate()
    with pytest.raises(OutOfPages):
        pool.allocate()


def test_hash_chain_depends_on_parent_and_tokens():
    h1 = hash_block(0, [1, 2, 3, 4])
    assert h1 == hash_block(0, [1, 2, 3, 4])
    assert h1 != hash_block(0, [1, 2, 3, 5])
    assert hash_block(h1, [9, 9, 9, 9]) != hash_block(0, [9, 9, 9, 9])


def test_groups_by_need_have_pages_of_their_own():
    specs = [PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=6), PagedKVSpec(2, 8), FixedStateSpec((3, 5)), None,
             PagedKVSpec(1, 16)]
    cm = CacheManager(specs, 4, 10, 3, F32, "cpu")
    assert [g.cache_slots for g in cm.groups] == [[0, 2], [1], [3], [5]]
    assert cm.groups[0].tensor.shape == (2, 10, 2, 2, 4, 8)
    assert cm.groups[2].tensor.shape == (1, 3, 3, 5)
    assert cm.layer_view(2).shape == (10, 2, 2, 4, 8) and cm.layer_view(4) is None
    assert not cm.prefix_cache                        # state of fixed size cannot be handed over: nothing is shared
    rc = cm.open("a")
    _feed(cm, rc, list(range(9)))
    assert len(rc.tables[0]) == 3 and len(rc.tables[1]) == 3 and len(rc.tables[3]) == 3
    cm.check_invariants()


def test_window_gives_pages_back_while_the_request_runs():
    cm = CacheManager([PagedKVSpec(1, 8, window=6)], 4, 8, 2, F32, "cpu")
    rc = cm.open("a")
    _feed(cm, rc, list(range(5)))                     # next query at 5 needs keys >= 0
    assert rc.tables[0] == [0, 1]
    _feed(cm, rc, list(range(5)))                     # next query at 10 needs keys >= 5: page 0 (keys 0-3) goes
    assert rc.tables[0][0] == -1 and rc.tables[0][1:] == [1, 2]
    assert cm.groups[0].pool.num_free == 6
    for _ in range(30):                               # long decoding in constant space
        _feed(cm, rc, [1])
        assert sum(p >= 0 for p in rc.tables[0]) <= 3
        cm.check_invariants()
    cm.close(rc)
    assert cm.pages_in_use() == 0


def test_full_pages_are_shared_and_the_last_token_is_left_to_compute():
    cm = _manager()
    a = cm.open("a", known_tokens=list(range(10)))
    assert a.num_tokens == 0
    _feed(cm, a, list(range(10)))                     # pages 0,1 full (tokens 0-7), page 2 partial
    b = cm.open("b", known_tokens=list(range(8)) + [77, 78])
    assert b.num_tokens == 8 and b.tables[0] == a.tables[0][:2]
    pool = cm.groups[0].pool
    assert pool.refcounts[a.tables[0][0]] == 2
    _feed(cm, b, [77, 78])
    assert b.tables[0][2] != a.tables[0][2]
    cm.check_invariants()
    # a prompt that is found whole: its last page is copied, one token is left to run
    c = cm.open("c", known_tokens=list(range(8)))
    assert c.num_tokens == 7 and c.tables[0][0] == a.tables[0][0] and c.tables[0][1] not in a.tables[0]
    assert cm.take_page_copies() == [(0, a.tables[0][1], c.tables[0][1])]
    _feed(cm, c, [7])
    cm.check_invariants()
    for rc in (a, b, c):
        cm.close(rc)
    assert cm.pages_in_use() == 0
    cm.check_invariants()


def test_a_page_is_sharable_only_once_it_is_full_and_written():
    cm = _manager()
    a = cm.open("a", known_tokens=list(range(8)))
    cm.append(a, list(range(8)))                      # appended, step not yet run
    b = cm.open("b", known_tokens=list(range(8)))
    assert b.num_tokens == 0                          # nothing to share yet
    cm.commit(a)
    cm.close(b)
    c = cm.open("c", known_tokens=list(range(8)) + [1])
    assert c.num_tokens == 8


def test_a_page_with_a_token_not_yet_known_is_sharable_once_it_is_known():
    """A step launched ahead runs a token whose id is still on the device: the request's record
    holds UNKNOWN_TOKEN in its place, the page it completes is not offered for sharing, and later
    pages wait too (their hashes chain through it), until resolve_token brings the id."""
    from qwen_engine_b200.cache.manager import UNKNOWN_TOKEN
    cm = _manager()
    a = cm.open("a", known_tokens=[1, 2, 3])
    _feed(cm, a, [1, 2, 3])
    _feed(cm, a, [UNKNOWN_TOKEN])                     # completes the first page of 4
    assert a.first_unknown == 3 and a.hashes[0] == []
    _feed(cm, a, [UNKNOWN_TOKEN])                     # a second one before the first is known
    cm.resolve_token(a, 3, 40)
    assert a.first_unknown == 4 and len(a.hashes[0]) == 1 and a.tokens[:4] == [1, 2, 3, 40]
    _feed(cm, a, [6, 7, 8])                           # fills the second page, whose first token is not known yet
    assert len(a.hashes[0]) == 1
    cm.resolve_token(a, 4, 50)
    assert a.first_unknown is None and len(a.hashes[0]) == 2
    with pytest.raises(RuntimeError):
        cm.resolve_token(a, 4, 51)                    # nothing waits there any more
    b = cm.open("b", known_tokens=[1, 2, 3, 40, 50, 6, 7, 8, 9])
    assert b.num_tokens == 8                          # both pages found by their tokens
    wrong = cm.open("c", known_tokens=[1, 2, 3, 41, 50, 6, 7, 8, 9])
    assert wrong.num_tokens == 0
    for rc in (a, b, wrong):
        cm.close(rc)
    cm.check_invariants()
    # a request that ended before its token arrived is passed over
    cm.resolve_token(a, 3, 1)


def test_freed_pages_stay_findable_until_they_are_reused():
    cm = _manager(num_pages=4)
    a = cm.open("a")
    _feed(cm, a, list(range(8)))
    cm.close(a)
    assert cm.pages_in_use() == 0
    b = cm.open("b", known_tokens=list(range(8)) + [5])
    assert b.num_tokens == 8                          # found although its owner is gone
    cm.close(b)
    c = cm.open("c")
    _feed(cm, c, [9] * 16)                            # takes all four pages: the hashes are dropped
    cm.close(c)
    d = cm.open("d", known_tokens=list(range(8)) + [5])
    assert d.num_tokens == 0
    cm.check_invariants()


def test_max_shared_tokens_limits_the_match():
    cm = _manager()
    a = cm.open("a")
    _feed(cm, a, list(range(12)))
    b = cm.open("b", known_tokens=list(range(12)), max_shared_tokens=5)
    assert b.num_tokens == 4


def test_append_is_all_or_nothing():
    cm = _manager(num_pages=3)
    a = cm.open("a")
    _feed(cm, a, list(range(6)))
    b = cm.open("b")
    with pytest.raises(OutOfPages):
        cm.append(b, list(range(9)))
    assert b.tables[0] == [] and cm.groups[0].pool.num_free == 1
    cm.check_invariants()
    assert cm.can_append(b, 4) and not cm.can_append(b, 5)
    assert not cm.can_append(b, 4, reserved={0: 1})


def test_state_slots():
    pool = StateSlotPool(2)
    a, b = pool.allocate(), pool.allocate()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfSlots):
        pool.allocate()
    pool.release(a)
    with pytest.raises(RuntimeError):
        pool.release(a)
    assert pool.allocate() == a
    cm = CacheManager([FixedStateSpec((4,)), PagedKVSpec(1, 8)], 4, 8, 2, F32, "cpu")
    r1, r2 = cm.open(1), cm.open(2)
    with pytest.raises(OutOfSlots):
        cm.open(3)
    cm.groups[0].tensor.fill_(5.0)
    cm.zero_fresh_state([r1])
    assert float(cm.groups[0].tensor[0, r1.state_slot].abs().sum()) == 0
    assert float(cm.groups[0].tensor[0, r2.state_slot].sum()) == 20.0
    cm.close(r1)
    r3 = cm.open(3)
    assert r3.state_slot == r1.state_slot and r3.fresh_state


def test_closing_twice_is_refused():
    cm = _manager()
    a = cm.open("a")
    cm.close(a)
    with pytest.raises(RuntimeError):
        cm.close(a)
    with pytest.raises(RuntimeError):
        cm.append(a, [1])


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("prefix", [True, False])
def test_random_orders_keep_every_page_accounted_for(seed, prefix):
    rng = random.Random(seed)
    specs = [PagedKVSpec(2, 8)] * 2 if prefix else [PagedKVSpec(2, 8), PagedKVSpec(2, 8, window=7)]
    cm = CacheManager(specs, 4, 24, 5, F32, "cpu", enable_prefix_cache=prefix)
    prompts = [[rng.randrange(3) for _ in range(rng.randrange(1, 30))] for _ in range(6)]  # few symbols: prefixes collide
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            toks = list(rng.choice(prompts))
            try:
                rc = cm.open(next_id, known_tokens=toks)
            except OutOfPages:
                continue
            live[next_id] = (rc, toks)
            next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            rc, toks = live[rid]
            rest = toks[rc.num_tokens:]
            new = rest[:rng.randrange(1, 9)] if rest else [rng.randrange(3)]
            try:
                cm.append(rc, new)
            except OutOfPages:
                victim = rng.choice(list(live))
                cm.close(live.pop(victim)[0])
            else:
                if rng.random() < 0.1:
                    cm.abort_pending(rc)
                else:
                    cm.commit(rc)
                    if not rest:
                        toks.extend(new)
        elif live:
            rid = rng.choice(list(live))
            cm.close(live.pop(rid)[0])
        cm.check_invariants()
        cm.take_page_copies()
    for rc, _ in live.values():
        cm.close(rc)
    cm.check_invariants()
    assert cm.pages_in_use() == 0 and cm.slots.num_free == 5


def test_a_group_that_keeps_a_window_shares_what_its_window_still_reaches():
    """Two groups, one keeping all keys and one keeping a window of 6: a second request with the same 16-token
    prefix gets every page of the prefix in the first group and, in the windowed group, only the pages the next
    query still reads (the earlier entries of its table stay -1); pages the first request already gave back are
    found again as long as nobody has taken them.  When a needed page of the windowed group is gone, the shared
    prefix shrinks to what both groups can hand over."""
    specs = [PagedKVSpec(1, 8), PagedKVSpec(1, 8, window=6)]
    cm = CacheManager(specs, 4, 12, 3, F32, "cpu", num_pages_of_group={1: 6})
    assert cm.prefix_cache
    prefix = list(range(100, 116))
    a = cm.open("a", known_tokens=prefix + [1, 2, 3, 4])
    _feed(cm, a, prefix + [1, 2, 3, 4])               # 20 tokens: the window (next query at 20) reaches back to key 15
    assert a.tables[1][:3] == [-1, -1, -1] and all(p >= 0 for p in a.tables[0])
    b = cm.open("b", known_tokens=prefix + [9, 9])
    assert b.num_tokens == 16 and b.shared_tokens == 16
    assert b.tables[0] == a.tables[0][:4]
    # the next query (position 16) reads keys 11..: blocks 2 and 3; block 2 is a page that a gave back, found again
    assert b.tables[1][:2] == [-1, -1] and b.tables[1][2] >= 0 and b.tables[1][3] == a.tables[1][3]
    cm.check_invariants()
    _feed(cm, b, [9, 9])
    cm.check_invariants()
    cm.close(b)
    # take pages until the freed, findable ones of the windowed group are handed out again: block 2 is gone
    hog = cm.open("hog")
    assert cm.groups[1].pool.num_free == 4            # one page never shared, three that a gave back and that are still findable
    _feed(cm, hog, list(range(500, 516)))
    c = cm.open("c", known_tokens=prefix + [7])
    assert c.num_tokens == 0, "without block 2 of the windowed group nothing of the prefix can be handed over whole"
    cm.check_invariants()
    for rc in (a, hog, c):
        cm.close(rc)
    assert cm.pages_in_use() == 0
    cm.check_invariants()


def test_random_requests_with_a_windowed_group_keep_the_books_right():
    """Random opens, appends and closes over two groups (all keys / a window) with shared prefixes: after every
    action no page is lost, held twice or freed twice, and a request's shared prefix is never longer than what it
    asked for."""
    import random
    rng = random.Random(5)
    cm = CacheManager([PagedKVSpec(1, 8), PagedKVSpec(1, 8, window=9)], 4, 40, 6, F32, "cpu")
    stems = [[rng.randrange(50) for _ in range(24)] for _ in range(3)]
    live = {}
    for step in range(400):
        action = rng.random()
        if action < 0.35 and len(live) < 5:
            toks = rng.choice(stems)[:rng.choice([8, 12, 16, 24])] + [rng.randrange(50) for _ in range(rng.randrange(1, 6))]
            try:
                rc = cm.open(step, known_tokens=toks)
            except OutOfPages:
                continue
            assert rc.num_tokens < len(toks) and rc.num_tokens % 4 in (0, 3)
            live[step] = (rc, toks)
        elif action < 0.8 and live:
            key = rng.choice(list(live))
            rc, toks = live[key]
            rest = toks[rc.num_tokens:] or [rng.randrange(50)]
            n = rng.randrange(1, len(rest) + 1)
            try:
                cm.append(rc, rest[:n])
            except OutOfPages:
                continue
            cm.commit(rc)
            if rc.num_tokens >= len(toks):
                live[key] = (rc, rc.tokens + [rng.randrange(50)])
        elif live:
            key = rng.choice(list(live))
            cm.close(live.pop(key)[0])
        cm.take_page_copies()
        cm.check_invariants()
    for rc, _ in live.values():
        cm.close(rc)
    assert cm.pages_in_use() == 0
