"""Which kernel serves a product of a few or of some tens of rows, by the shapes of the three model sizes (no GPU: the
choice is host arithmetic).  The figures behind the rules were measured on a B200, in a chain of the product alone
and then in the decode step."""
import pytest
import torch

from qwen_engine_b200 import ops

BF = torch.bfloat16
# (hidden, intermediate, q heads, kv heads) with head size 128
SIZES = {"0.6b": (1024, 3072, 16, 8), "1.7b": (2048, 6144, 16, 8), "4b": (2560, 9728, 32, 8)}


def _products(name):
    H, I, Hq, Hkv = SIZES[name]
    return {"qkv": ((Hq + 2 * Hkv) * 128, H), "o": (H, Hq * 128), "gate_up": (2 * I, H), "down": (H, I)}


@pytest.mark.parametrize("name", list(SIZES))
def test_up_to_eight_rows_stream_the_weights(name):
    """... but for the one product whose K is so long and whose weight rows are so awkward a number (2 560: 160 CTAs of
    16 rows for 148 SMs) that clusters sharing K are faster at any number of rows: Qwen3-4B's down projection."""
    for what, (N, K) in _products(name).items():
        for M in (1, 4, 8):
            assert ops.splitk_splits(M, N, K, BF) == (4 if (name, what) == ("4b", "down") else 0)


def test_nine_to_sixteen_rows_share_k_only_where_the_streaming_kernel_is_at_its_worst():
    for name in ("0.6b", "1.7b"):
        for N, K in _products(name).values():
            assert ops.splitk_splits(12, N, K, BF) == 0, (name, N, K)
    p = _products("4b")
    assert ops.splitk_splits(9, *p["o"], BF) == 4 and ops.splitk_splits(16, *p["down"], BF) == 4
    assert ops.splitk_splits(16, *p["qkv"], BF) == 0 and ops.splitk_splits(16, *p["gate_up"], BF) == 0


def test_some_tens_of_rows_share_k_in_clusters_that_find_room():
    # 1 024 weight rows: 8 clusters of 8 CTAs; 2 048 and 2 560: 16 and 20 clusters, of 4
    assert ops.splitk_splits(32, *_products("0.6b")["o"], BF) == 8 and ops.splitk_splits(64, *_products("0.6b")["down"], BF) == 8
    assert ops.splitk_splits(32, *_products("1.7b")["o"], BF) == 4 and ops.splitk_splits(32, *_products("1.7b")["down"], BF) == 4
    assert ops.splitk_splits(32, *_products("4b")["o"], BF) == 4
    # many weight rows: fewer CTAs a cluster, or none (the swapped kernel or the streaming one serves)
    assert ops.splitk_splits(32, *_products("0.6b")["qkv"], BF) == 4 and ops.splitk_splits(32, *_products("0.6b")["gate_up"], BF) == 2
    assert ops.splitk_splits(32, *_products("4b")["gate_up"], BF) == 0
    for s in (2, 4, 8):        # whatever is chosen fits the GPU at once and leaves every CTA two blocks of K at least
        for name in SIZES:
            for N, K in _products(name).values():
                got = ops.splitk_splits(40, N, K, BF)
                assert got == 0 or (-(-N // 128) * got <= ops.SPLITK_MAX_CTAS and -(-K // 64) >= 2 * got)


def test_other_types_and_many_rows_are_not_for_that_kernel():
    assert ops.splitk_splits(32, 1024, 2048, torch.float32) == 0
    assert ops.splitk_splits(65, 1024, 2048, BF) == 0
    assert ops.splitk_splits(32, 1024, 2052, BF) == 0          # K must be a multiple of 8
