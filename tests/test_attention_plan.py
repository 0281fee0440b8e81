"""The host's plan for the tcgen05 attention kernel (no GPU): tiles, their parts, and the schedule that deals the work
units out to the kernel's CTAs.  The library is loaded for its host-side functions only."""
import random

import pytest
import torch

from qwen_engine_b200 import ops

GEOS = [(16, 8, 128, 0), (4, 2, 128, 0), (8, 1, 128, 0), (4, 4, 128, 300)]


def _items(plan, key="tc0_items"):
    flat = plan[key]
    return [flat[i:i + ops.FLASH_ITEM_INTS] for i in range(0, len(flat), ops.FLASH_ITEM_INTS)]


def _random_batch(rng):
    n = rng.randint(1, 6)
    q_lens = [rng.choice([70, 128, 129, 300, 700, 1500, 2048, 3000]) for _ in range(n)]
    ctx_lens = [rng.choice([0, 0, 17, 128, 1000, 5000]) for _ in range(n)]
    return q_lens, ctx_lens


@pytest.mark.parametrize("seed", range(12))
def test_tiles_and_parts_cover_every_row_and_key_once(seed):
    rng = random.Random(seed)
    Hq, Hkv, D, window = GEOS[seed % len(GEOS)]
    q_lens, ctx_lens = _random_batch(rng)
    plan = ops.plan_attention(q_lens, ctx_lens, 16, ((Hq, Hkv, D, window),), torch.bfloat16)
    G = Hq // Hkv
    tile_tokens = ops.TC_ROWS // G
    seen = {}                                           # (request, first token of the tile) -> key ranges of its items
    for req, q0, lo, hi, part, n_parts, split, row0, q_len, ctx, _, _ in _items(plan):
        assert q_len == q_lens[req] and ctx == ctx_lens[req] and q0 % tile_tokens == 0 and q0 < q_len
        assert row0 == sum(q_lens[:req])
        seen.setdefault((req, q0), []).append((lo, hi, part, n_parts, split))
    for req, n in enumerate(q_lens):
        if n * G < ops.TC_MIN_ROWS:
            assert not any(r == req for r, _ in seen), "a request of few rows belongs to the other kernel"
            continue
        assert sorted(q0 for r, q0 in seen if r == req) == list(range(0, n, tile_tokens))
    for (req, q0), ranges in seen.items():
        ranges.sort()
        frontier = ctx_lens[req] + min(q_lens[req], q0 + tile_tokens)
        assert ranges[-1][1] == frontier, "a tile's keys end at its last token's position"
        if len(ranges) == 1:
            assert ranges[0][2] == -1 and ranges[0][0] >= 0
            continue
        first = ranges[0][2]
        for i, (lo, hi, part, n_parts, split) in enumerate(ranges):
            assert (part, n_parts, split) == (first + i, len(ranges), i)
            assert lo < hi and (i == 0 or lo == ranges[i - 1][1]), "the parts of a tile follow one another"
            assert i == 0 or lo % ops.TC_BN == 0, "a part begins with a whole key step"
    assert plan["tc0_info"][0] == sum(len(r) for r in seen.values() if len(r) > 1)


@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("ctas", [1, 5, 148])
def test_every_unit_is_dealt_out_once_and_no_cta_is_left_behind(seed, ctas, monkeypatch):
    rng = random.Random(100 + seed)
    Hq, Hkv, D, window = GEOS[seed % len(GEOS)]
    q_lens, ctx_lens = _random_batch(rng)
    monkeypatch.setattr(ops, "TC_TARGET_CTAS", ctas)
    plan = ops.plan_attention(q_lens, ctx_lens, 16, ((Hq, Hkv, D, window),), torch.bfloat16)
    if "tc0_items" not in plan:
        pytest.skip("no request brings enough rows")
    items = _items(plan)
    units = len(items) * Hkv
    parts, rows, n = plan["tc0_info"]
    sched = plan["tc0_sched"]
    assert rows == ops.TC_ROWS and n == min(units, ctas)
    assert sched[0] == n + 1 and sched[n] == len(sched) == n + 1 + units
    assert all(sched[c] <= sched[c + 1] for c in range(n))
    assert sorted(sched[n + 1:]) == list(range(units))

    def cost(unit):
        req, q0, lo, hi, part = items[unit // Hkv][:5]
        return -(-(hi - lo // ops.TC_BN * ops.TC_BN) // ops.TC_BN) + ops.TC_ITEM_COST_STEPS + (ops.TC_PART_COST_STEPS if part >= 0 else 0)
    loads = [sum(cost(u) for u in sched[sched[c]:sched[c + 1]]) for c in range(n)]
    assert min(loads) > 0, "with as many CTAs as units at most, every CTA has work"
    # longest first to the least loaded: no CTA carries more than the lightest one plus one unit
    assert max(loads) - min(loads) <= max(cost(u) for u in range(units)) + 1e-3
    again = ops.plan_attention(q_lens, ctx_lens, 16, ((Hq, Hkv, D, window),), torch.bfloat16)
    assert again["tc0_sched"] == sched and again["tc0_items"] == plan["tc0_items"]


def test_long_tiles_are_cut_only_where_the_schedule_gains():
    geo = ((16, 8, 128, 0),)
    one = ops.plan_attention([2048], [0], 16, geo, torch.bfloat16)
    assert 0 < one["tc0_info"][0] <= 16, "a single long prompt: its longest tiles are cut, in few parts"
    many = ops.plan_attention([1024] * 16, [0] * 16, 16, geo, torch.bfloat16)
    assert many["tc0_info"][0] == 0, "enough tiles for every SM: nothing is cut"
    behind = ops.plan_attention([128], [30000], 16, geo, torch.bfloat16)
    assert behind["tc0_info"][0] >= 2, "one tile behind a long context is cut so that more than 8 SMs work"
