"""The four replay families at head size 128, where the kernels that serving real models runs live:
attention with scores and output in tensor memory (prompt portions), the tensor-core kernel for
decoded tokens, the products by pairs of CTAs with the rotary and SiLU epilogues, the swapped product
and the one that shares K within a cluster.  tiny-a/b/c (head sizes 16, 32, 48) never reach them.

Every test compares the engine with the plain implementation and says which entry points of the
library had to serve it.  The cache starts out filled with a large finite number (bfloat16; NaN in
32-bit): the attention kernel for prompt portions reads the slots of a held page that lie past a
request's length and masks them, so a mask that is off by one shows as a huge logit, where 0 x NaN would
spoil rows that are right."""
import pytest
import torch

import helpers
from helpers import (LaunchSpy, check_requests, live_tokens_needed, make_replayer, mixed_steps,
                     random_tokens, run_steps)

pytestmark = pytest.mark.gpu
NAME = "tiny-d"
DTYPES = [torch.float32, torch.bfloat16]
# which kernels a selection must show (bfloat16); "shipped": the thresholds as they are
SELECTIONS = {
    "shipped": {},
    # pairs of CTAs (and their epilogues: rotary + cache write, SiLU-mul) at shapes this small
    "pairs": dict(PAIR_MIN_TILES=1, QKV_ROPE_MIN_TILES=1),
    # some tens of rows: the swapped product instead of the one that shares K within a cluster
    "swap": dict(SPLITK=False, SWAP_MIN_N=256),
}


def _poison(dtype):
    return 3.0e4 if dtype == torch.bfloat16 else True


def _select(monkeypatch, selection):
    from qwen_engine_b200 import ops
    for k, v in SELECTIONS[selection].items():
        monkeypatch.setattr(ops, k, v)


def _served(spy, dtype, *names):
    if dtype != torch.bfloat16:
        return
    from qwen_engine_b200 import ops
    missing = [n for n in names if spy.count(n) == 0]
    assert not missing, f"not served by {missing}; calls: {sorted(spy.counts)}"
    assert ops.tcgen05_status() == 0 and ops.tc_attention_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("selection", list(SELECTIONS))
def test_whole_requests(model_folders, monkeypatch, dtype, selection):
    _select(monkeypatch, selection)
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    reqs = {"a": random_tokens(V, 17, 1), "b": random_tokens(V, 200, 2), "c": random_tokens(V, 700, 3),
            "d": random_tokens(V, 47, 4)}
    rep = make_replayer(folder, NAME, dtype, 704, poison=_poison(dtype))
    steps = [{"entries": [{"id": rid, "tokens": t, "want": list(range(len(t)))}], "end": [rid]}
             for rid, t in reqs.items()]
    with LaunchSpy() as spy:
        got = run_steps(rep, steps)
    check_requests(got, folder, reqs, dtype, f"whole {selection}")
    assert rep.cache.pages_in_use() == 0
    _served(spy, dtype, "qe_flash_attention_tc", "qe_flash_attention_fused_merge")
    if selection == "shipped":
        _served(spy, dtype, "qe_linear_tcgen05", "qe_linear_tcgen05_splitk")
    elif selection == "pairs":
        _served(spy, dtype, "qe_linear_tcgen05_pair", "qe_linear_swiglu_tcgen05_pair", "qe_linear_qkv_rope_tcgen05_pair")
    else:
        _served(spy, dtype, "qe_linear_tcgen05_swap")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("selection", ["shipped", "pairs"])
def test_last_32_decoded(model_folders, monkeypatch, dtype, selection):
    _select(monkeypatch, selection)
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    toks = random_tokens(V, 600, 5)
    rep = make_replayer(folder, NAME, dtype, 640, poison=_poison(dtype))
    head = len(toks) - 32
    steps = [{"entries": [{"id": "r", "tokens": toks[:head], "want": [0, 100, head - 1]}]}]
    steps += [{"entries": [{"id": "r", "tokens": [toks[i]], "want": [0]}]} for i in range(head, len(toks))]
    steps[-1]["end"] = ["r"]
    with LaunchSpy() as spy:
        got = run_steps(rep, steps)
    assert sorted(got["r"]) == [0, 100, head - 1] + list(range(head, len(toks)))
    check_requests(got, folder, {"r": toks}, dtype, f"last32 {selection}")
    _served(spy, dtype, "qe_flash_attention_tc", "qe_decode_attention_mma", "qe_linear_small_m")
    assert dtype != torch.bfloat16 or rep.runner.num_graph_replays >= 20


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("selection", list(SELECTIONS))
def test_changing_portions(model_folders, monkeypatch, dtype, selection):
    _select(monkeypatch, selection)
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    toks = random_tokens(V, 700, 6)
    rep = make_replayer(folder, NAME, dtype, 704, poison=_poison(dtype))
    sizes = [100, 37, 200, 2, 64, 17, 33, 129, 40, 16, 62]
    assert sum(sizes) == len(toks)
    steps, p = [], 0
    for n in sizes:
        steps.append({"entries": [{"id": "r", "tokens": toks[p:p + n], "want": list(range(n))}]})
        p += n
    with LaunchSpy() as spy:
        got = run_steps(rep, steps)
    check_requests(got, folder, {"r": toks}, dtype, f"portions {selection}")
    _served(spy, dtype, "qe_flash_attention_tc", "qe_flash_attention_fused_merge")
    if selection == "pairs":
        _served(spy, dtype, "qe_linear_qkv_rope_tcgen05_pair", "qe_linear_swiglu_tcgen05_pair")
    if selection == "swap":
        _served(spy, dtype, "qe_linear_tcgen05_swap")


MIXED_LENS = [300, 64, 523, 90, 700, 17, 255, 640, 101, 33, 128, 72]
MIXED_SIZES = (2, 5, 21, 40, 64, 130, 300)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("selection", list(SELECTIONS))
@pytest.mark.parametrize("prefix_cache", [True, False])
def test_mixed_with_few_pages(model_folders, monkeypatch, dtype, selection, prefix_cache):
    """Up to four live requests, portions of some (long enough for the tensor-memory attention kernel)
    beside decoded tokens of others in one batch, over exactly as many pages as the live requests need at
    their fullest, so that pages of finished requests, with what they held, are handed to new ones."""
    _select(monkeypatch, selection)
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    reqs = {f"r{i}": random_tokens(V, n, 10 + i) for i, n in enumerate(MIXED_LENS)}
    steps = mixed_steps(reqs, seed=4, sizes=MIXED_SIZES)
    need = live_tokens_needed(steps)
    rep = make_replayer(folder, NAME, dtype, need, prefix_cache=prefix_cache, poison=_poison(dtype))
    total_pages = rep.cache.paged_groups[0].pool.num_pages
    assert total_pages * rep.cache.page_size == need
    assert sum(-(-n // rep.cache.page_size) for n in MIXED_LENS) > 2 * total_pages, "the trace must reuse pages"
    assert any(len(st["entries"]) == 4 and any(len(e["tokens"]) == 1 for e in st["entries"])
               and any(len(e["tokens"]) >= 40 for e in st["entries"]) for st in steps)
    with LaunchSpy() as spy:
        got = run_steps(rep, steps)
    check_requests(got, folder, reqs, dtype, f"mixed {selection}")
    assert rep.cache.pages_in_use() == 0
    _served(spy, dtype, "qe_flash_attention_tc", "qe_flash_attention_fused_merge", "qe_decode_attention_mma")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_the_block_table_bucket(model_folders, dtype):
    """Steps of decoded tokens are replayed from CUDA graphs keyed by the width of the block tables in
    units of 64 pages, and the number of parts a context is cut into follows the width: a request that
    grows from 1 000 to 1 060 tokens (page 16: from 63 to 67 pages) crosses it, beside two shorter ones."""
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    reqs = {"long": random_tokens(V, 1060, 21), "mid": random_tokens(V, 330, 22), "short": random_tokens(V, 75, 23)}
    rep = make_replayer(folder, NAME, dtype, 1088 + 384 + 128, poison=_poison(dtype))
    n_dec = 60
    steps = [{"entries": [{"id": rid, "tokens": t[:len(t) - n_dec], "want": [len(t) - n_dec - 1]}]} for rid, t in reqs.items()]
    for i in range(n_dec):
        steps.append({"entries": [{"id": rid, "tokens": [t[len(t) - n_dec + i]], "want": [0]} for rid, t in reqs.items()]})
    with LaunchSpy() as spy:
        got = run_steps(rep, steps)
    check_requests(got, folder, reqs, dtype, "across the bucket")
    keys = [k for k in rep.runner._graphs if len(k) == 3]
    assert {k[2] for k in keys} == {(64,), (128,)}, keys
    assert rep.runner.num_graph_replays >= n_dec - 4
    _served(spy, dtype, "qe_decode_attention_mma")


@pytest.mark.parametrize("selection", ["shipped", "pairs"])
def test_cuts_at_the_edges_of_pages_and_key_tiles(model_folders, monkeypatch, selection):
    """A prompt cut where the attention kernel for prompt portions has its own edges: at multiples of its
    128-key steps, one token before and after them, inside a page, and with a one-token portion between
    long ones; the logits at the first, middle and last place of every portion."""
    _select(monkeypatch, selection)
    folder, V = model_folders[NAME], helpers.vocab_of(NAME)
    toks = random_tokens(V, 515, 31)
    for cuts in ([128, 128, 128, 131], [127, 129, 1, 258], [384, 3, 128]):
        rep = make_replayer(folder, NAME, torch.bfloat16, 576, poison=3.0e4)
        steps, p = [], 0
        for n in cuts:
            steps.append({"entries": [{"id": "r", "tokens": toks[p:p + n], "want": sorted({0, n // 2, n - 1})}]})
            p += n
        assert p == len(toks)
        check_requests(run_steps(rep, steps), folder, {"r": toks}, torch.bfloat16, f"cuts {cuts}")
