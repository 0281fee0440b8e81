"""Each CUDA kernel alone against its plain PyTorch restatement (tests/ref_ops.py), in float32
and bfloat16, at sizes other than the engine's models: widths and vocabularies that are no
power of two, head sizes in steps of 16, odd numbers of heads and groups."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import ref_ops
from qwen_engine_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _close(got, want, dtype, scale=None, tol32=2e-5, tol16=1.6e-2):
    got, want = got.float().cpu(), want.float().cpu()
    s = max(1.0, float(want.abs().max())) if scale is None else scale
    tol = tol32 if dtype == torch.float32 else tol16
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all()
    assert err <= tol * s, f"max |diff| {err:.3e} > {tol} * {s:.3f}"


def _randn(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


def test_extension_loads():
    assert ops.lib().qe_abi_version() == 1


def test_cpu_tensor_is_refused():
    with pytest.raises(ops.ExtensionMissing):
        ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,V", [(1, 64, 300), (37, 200, 1001), (5, 1000, 50)])
def test_embedding(dtype, T, H, V):
    table = _randn((V, H), dtype, 1)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    want = torch.empty(T, H)
    ref_ops.embedding(ids, table, want)
    got = torch.empty(T, H, device=DEV)
    ops.embedding(ids.to(DEV), table.to(DEV), got)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 48), (33, 200), (7, 1000), (3, 4100)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(dtype, T, H, with_delta):
    resid = _randn((T, H), torch.float32, 3, 2.0)
    delta = _randn((T, H), dtype, 4) if with_delta else None
    w = 1 + 0.3 * _randn((H,), torch.float32, 5)
    eps = 1e-5
    r_ref, out_ref = resid.clone(), torch.empty(T, H, dtype=dtype)
    ref_ops.add_rmsnorm(r_ref, delta, w, eps, out_ref)
    r_gpu, out_gpu = resid.to(DEV), torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r_gpu, delta.to(DEV) if with_delta else None, w.to(DEV), eps, out_gpu)
    _close(r_gpu, r_ref, torch.float32, tol32=1e-6)
    _close(out_gpu, out_ref, dtype)
    # the rows variant: chosen rows, stream untouched
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    out_ref2 = torch.empty(3, H, dtype=dtype)
    ref_ops.add_rmsnorm_rows(resid, delta, rows, w, eps, out_ref2)
    r_gpu2, out_gpu2 = resid.to(DEV), torch.empty(3, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm_rows(r_gpu2, delta.to(DEV) if with_delta else None, rows.to(DEV), w.to(DEV), eps, out_gpu2)
    assert torch.equal(r_gpu2.cpu(), resid)
    _close(out_gpu2, out_ref2, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 17, 5), (3, 389, 80), (70, 130, 224), (129, 64, 1000), (16, 1030, 72),
                                   (8, 4096, 1024), (64, 1000, 3072), (33, 389, 224), (1, 20011, 64), (17, 24, 2048),
                                   (9, 130, 8), (40, 16, 1032)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear(dtype, M, N, K, out_f32):
    x = _randn((M, K), dtype, 6)
    w = _randn((N, K), dtype, 7, 0.1)
    odt = torch.float32 if out_f32 else dtype
    want = torch.empty(M, N, dtype=odt)
    ref_ops.linear(x, w, want)
    got = torch.empty(M, N, dtype=odt, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), got)
    _close(got, want, odt, tol16=8e-3)


@pytest.mark.parametrize("M,N,K", [(256, 128, 64), (130, 72, 8), (300, 200, 136), (512, 256, 640), (2048, 1024, 2048),
                                   (1000, 24, 2048), (2048, 4096, 1024), (2304, 4360, 192), (5000, 3000, 72)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear_tcgen05_pairs(M, N, K, out_f32):
    """Pairs of CTAs on one 256-row tile (cta_group::2): 256 x 128 tiles where tiles are few,
    256 x 256 where they are many; edges in M, N and K; several tiles per pair of SMs."""
    x = _randn((M, K), torch.bfloat16, 26)
    w = _randn((N, K), torch.bfloat16, 27, 0.1)
    odt = torch.float32 if out_f32 else torch.bfloat16
    want = torch.empty(M, N, dtype=odt)
    ref_ops.linear(x, w, want)
    got = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
    ops.linear_pairs(x.to(DEV), w.to(DEV), got)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(got, want, torch.bfloat16, scale=float(want.float().abs().max()))


@pytest.mark.parametrize("M,N,K,splits", [(2048, 1024, 2048, 2), (2048, 1024, 3072, 2), (528, 2048, 6144, 2), (300, 1024, 1024, 4),
                                          (128, 512, 4104, 4), (1000, 1000, 2056, 2), (65, 2048, 2048, 4), (700, 2560, 9728, 2)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear_tcgen05_pairs_that_split_k(M, N, K, splits, out_f32):
    """Products with too few 256 x 256 tiles for every pair of SMs: 2 or 4 pairs of a cluster take a share of K of
    the same tile and their sums meet through distributed shared memory, every CTA finishing a share of the
    columns; edges in M, N and K (a last k-block that is not whole, shares of unequal length)."""
    assert ops.pair_k_splits(M, N, K) == splits
    x = _randn((M, K), torch.bfloat16, 28)
    w = _randn((N, K), torch.bfloat16, 29, 0.1)
    odt = torch.float32 if out_f32 else torch.bfloat16
    want = torch.empty(M, N, dtype=odt)
    ref_ops.linear(x, w, want)
    got = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
    ops.linear_pairs(x.to(DEV), w.to(DEV), got)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(got, want, torch.bfloat16, scale=float(want.float().abs().max()))
    if ops.tc_product_plan(M, N, K) != 0:              # the route that `linear` takes where the pairs are the faster kernel
        got2 = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), got2)
        assert torch.equal(got2, got)


def test_the_plan_of_the_tcgen05_products():
    """Which kernel `linear` picks for products of many rows (a model of the kernels' times in the library): the
    single-CTA kernel for few rows and a short K, CTA pairs with wide tiles where those fill most pairs of SMs, K
    split over pairs where tiles are few and K is long."""
    plan = ops.tc_product_plan
    assert plan(128, 4096, 1024) == 0
    assert plan(2048, 4096, 1024) == 2 and plan(2048, 6144, 1024) == 2
    assert plan(2048, 2048, 2048) == 2                 # 64 tiles for 74 pairs: wide tiles, one round
    assert plan(528, 4096, 1024) == 2
    assert plan(2048, 1024, 2048) == 3 and plan(2048, 1024, 3072) == 3
    assert plan(528, 1024, 3072) == 4
    assert plan(8192, 2560, 9728) == 2


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (300, 200, 136), (2048, 3072, 1024), (1000, 1032, 72), (4100, 392, 200)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear_swiglu_fused(M, I, K, out_f32):
    """silu(x w_gate^T) * (x w_up^T) out of the epilogue of the CTA-pair product over the stacked
    weights (the activation is formed on the float32 sums; the two-kernel route rounds gate and up
    to bfloat16 first: both are compared with the plain float32 formula); edges in M, I and K."""
    x = _randn((M, K), torch.bfloat16, 36)
    w = _randn((2 * I, K), torch.bfloat16, 37, 0.1)
    g = x.float() @ w[:I].float().t()
    u = x.float() @ w[I:].float().t()
    want = g / (1 + torch.exp(-g)) * u
    odt = torch.float32 if out_f32 else torch.bfloat16
    got = torch.full((M, I), float("nan"), dtype=odt, device=DEV)
    ops.linear_swiglu(x.to(DEV), w.to(DEV), got)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(got, want, torch.bfloat16, scale=float(want.abs().max()), tol16=1e-2)


@pytest.mark.parametrize("M", [17, 31, 48, 64])
@pytest.mark.parametrize("N,K", [(3072, 64), (3080, 1024), (6144, 1032), (4100, 200)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear_tcgen05_swapped(M, N, K, out_f32, monkeypatch):
    """Some tens of rows against many weight rows in bfloat16: the kernel with the weights on the
    128-row side of the instruction; edges in M (not a multiple of 16), N and K."""
    assert ops.SWAP_MIN_M <= M <= ops.SMALL_M_MAX and N >= ops.SWAP_MIN_N
    monkeypatch.setattr(ops, "SPLITK", False)
    x = _randn((M, K), torch.bfloat16, 18)
    w = _randn((N, K), torch.bfloat16, 19, 0.1)
    odt = torch.float32 if out_f32 else torch.bfloat16
    want = torch.empty(M, N, dtype=odt)
    ref_ops.linear(x, w, want)
    got = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), got)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(got, want, torch.bfloat16, scale=float(want.float().abs().max()))


@pytest.mark.parametrize("M", [1, 9, 17, 33, 64])
@pytest.mark.parametrize("N,K,splits", [(1024, 2048, 8), (1024, 3072, 8), (1000, 1032, 4), (132, 200, 2), (4096, 1024, 4),
                                        (256, 192, 8), (6144, 1024, 2), (2560, 4096, 4)])
@pytest.mark.parametrize("mode", ["bf16", "f32", "add"])
def test_linear_splitk(M, N, K, splits, mode):
    """Up to 64 rows against few weight rows in bfloat16: clusters of CTAs that share K and add their partial
    sums through distributed shared memory; edges in M, N and K, a K that leaves some CTAs of a
    cluster without a share (192 = 3 blocks for 8 CTAs), and the sum added to a float32 stream."""
    x = _randn((M, K), torch.bfloat16, 28)
    w = _randn((N, K), torch.bfloat16, 29, 0.1)
    odt = torch.bfloat16 if mode == "bf16" else torch.float32
    want = torch.empty(M, N, dtype=torch.float32)
    ref_ops.linear(x, w, want)
    if mode == "add":
        start = _randn((M, N), torch.float32, 30)
        want = want + start
        got = start.to(DEV)
    else:
        got = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
    ops.linear_splitk(x.to(DEV), w.to(DEV), got, splits, add=mode == "add")
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(got, want.to(odt), odt, scale=float(want.abs().max()), tol16=8e-3)
    # the same call again gives the same bits: the order of the sum is fixed
    again = start.to(DEV) if mode == "add" else torch.empty_like(got)
    ops.linear_splitk(x.to(DEV), w.to(DEV), again, splits, add=mode == "add")
    assert torch.equal(again, got)


def test_linear_picks_splitk():
    """`linear` sends some tens of rows to the cluster kernel where the weight rows are too few for every SM, also
    when the product is added to the residual stream; a few rows and many rows go elsewhere."""
    assert ops.splitk_splits(64, 1024, 3072, torch.bfloat16) == 8
    assert ops.splitk_splits(17, 4096, 1024, torch.bfloat16) == 4
    assert ops.splitk_splits(32, 2048, 6144, torch.bfloat16) == 4      # 16 clusters: of 4 CTAs, not of 8
    assert ops.splitk_splits(12, 2560, 9728, torch.bfloat16) == 4      # a long K and more CTAs of 16 rows than SMs: from 9 rows on
    assert ops.splitk_splits(8, 2560, 9728, torch.bfloat16) == 4 and ops.splitk_splits(8, 2560, 4096, torch.bfloat16) == 0
    assert ops.splitk_splits(12, 4096, 1024, torch.bfloat16) == 0
    assert ops.splitk_splits(12, 6144, 4096, torch.bfloat16) == 0      # (only two CTAs a cluster would fit)
    assert ops.splitk_splits(32, 6144, 1024, torch.bfloat16) == 2
    assert ops.splitk_splits(8, 1024, 3072, torch.bfloat16) == 0
    assert ops.splitk_splits(65, 1024, 3072, torch.bfloat16) == 0
    assert ops.splitk_splits(64, 151936, 1024, torch.bfloat16) == 0
    assert ops.splitk_splits(64, 1024, 3072, torch.float32) == 0
    M, N, K = 40, 1024, 3072
    x = _randn((M, K), torch.bfloat16, 31)
    w = _randn((N, K), torch.bfloat16, 32, 0.1)
    want = torch.empty(M, N, dtype=torch.float32)
    ref_ops.linear(x, w, want)
    got = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), got)
    _close(got, want.to(torch.bfloat16), torch.bfloat16, scale=float(want.abs().max()))


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (65, 128, 64), (300, 200, 136), (2048, 4096, 1024),
                                   (130, 1000, 3072), (257, 389 * 8, 80), (1000, 24, 2048), (128, 6144, 1024),
                                   (2304, 4360, 192), (1280, 2568, 320)])
@pytest.mark.parametrize("out_f32", [False, True])
def test_linear_tcgen05(M, N, K, out_f32):
    """More than 64 rows in bfloat16: the TMA + tcgen05 kernel, with edges in M, N and K; wide and
    narrow tiles; up to three tiles per CTA, so that both accumulators and the ring wrap around."""
    x = _randn((M, K), torch.bfloat16, 16)
    w = _randn((N, K), torch.bfloat16, 17, 0.1)
    odt = torch.float32 if out_f32 else torch.bfloat16
    want = torch.empty(M, N, dtype=odt)
    ref_ops.linear(x, w, want)
    got = torch.empty(M, N, dtype=odt, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), got)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0, "a bounded wait of the tcgen05 kernel ran out"
    _close(got, want, odt, tol16=8e-3)


@pytest.mark.parametrize("M,H,N", [(1, 64, 40), (8, 1024, 4096), (16, 80, 389), (5, 1032, 72), (17, 128, 64)])
@pytest.mark.parametrize("norm_rows", [0, 16])
def test_branch_into_stream_then_fused_norm(M, H, N, norm_rows, monkeypatch):
    """A branch's product added into the float32 stream by the product's own epilogue (which leaves
    the rows' sums of squares), then the next norm: by its own kernel (the engine's setting), or fused
    into the next product from those sums (few rows, bfloat16; an option that is off in the engine);
    more rows fall back to the delta buffer and the separate norm kernel.  Same numbers every way."""
    monkeypatch.setattr(ops, "FUSED_NORM_MAX_M", norm_rows)
    dt = torch.bfloat16
    K1 = 136
    resid = _randn((M, H), torch.float32, 50, 2.0)
    x1 = _randn((M, K1), dt, 51)
    w1 = _randn((H, K1), dt, 54, 0.1)
    gu = _randn((M, 2 * K1), dt, 55)
    nw = 1 + 0.3 * _randn((H,), torch.float32, 52)
    w2 = _randn((N, H), dt, 53, 0.1)

    # plain reference: resid += x1 w1^T (rounded as the delta buffer would hold it is NOT applied: the
    # fused route adds the float32 product), then += silu-mul branch, then norm and product
    want_resid = resid + x1.float() @ w1.float().t()
    g, u = gu[:, :K1].float(), gu[:, K1:].float()
    want_resid = want_resid + (g / (1 + torch.exp(-g)) * u).to(dt).float() @ w1.float().t()
    normed = want_resid * torch.rsqrt((want_resid ** 2).mean(-1, keepdim=True) + 1e-5) * nw
    want = normed.to(dt).float() @ w2.float().t()

    alloc = lambda shape, d: torch.empty(shape, dtype=d, device=DEV)
    ssq = torch.full((M, -(-(-(-H // 16)) // 4) * 4), float("nan"), device=DEV)
    st = ops.ResidualStream(resid.to(DEV), torch.empty(M, H, dtype=dt, device=DEV), ssq)
    ops.linear(x1.to(DEV), w1.to(DEV), ops.ResidualSink(st))
    ops.linear_silu_mul(gu.to(DEV), w1.to(DEV), ops.ResidualSink(st), alloc)
    fused = M <= ops.SMALL_M_MAX
    assert (st.n_ssq == -(-H // 16) and not st.has_delta) if fused else st.has_delta
    out = torch.empty(M, N, dtype=dt, device=DEV)
    ops.linear(ops.NormedInput(st, nw.to(DEV), 1e-5, alloc, dt), w2.to(DEV), out)
    assert not st.has_delta
    _close(st.resid, want_resid, torch.float32, tol32=2e-2)          # bfloat16 operands, float32 sums
    _close(out, want, dt, tol16=2e-2)
    if fused:
        got_ssq = st.ssq[:, :st.n_ssq].sum(-1).cpu()
        assert torch.allclose(got_ssq, (st.resid.cpu() ** 2).sum(-1), rtol=1e-4)


def test_linear_row_does_not_depend_on_batch():
    """A row's product is the same bits whatever else is in the batch (32-bit path)."""
    x = _randn((67, 200), torch.float32, 8).to(DEV)
    w = _randn((150, 200), torch.float32, 9).to(DEV)
    full = torch.empty(67, 150, device=DEV)
    ops.linear(x, w, full)
    for r in (0, 13, 66):
        one = torch.empty(1, 150, device=DEV)
        ops.linear(x[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 10), (9, 224), (33, 1001)])
def test_silu_mul(dtype, T, I):
    gu = _randn((T, 2 * I), dtype, 10, 3.0)
    want = torch.empty(T, I, dtype=dtype)
    ref_ops.silu_mul(gu, want)
    got = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.silu_mul(gu.to(DEV), got)
    _close(got, want, dtype, tol32=1e-6, tol16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,I", [(1, 40, 56), (8, 1024, 3072), (33, 80, 224), (64, 72, 152), (70, 100, 64), (5, 30, 10)])
def test_linear_silu_mul(dtype, M, N, I):
    """The feed-forward's activation fused into its output projection (few rows, bfloat16), and the
    two-kernel route for everything else."""
    gu = _randn((M, 2 * I), dtype, 40, 2.0)
    w = _randn((N, I), dtype, 41, 0.1)
    want = torch.empty(M, N, dtype=dtype)
    ref_ops.linear_silu_mul(gu, w, want, lambda shape, dt: torch.empty(shape, dtype=dt))
    got = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.linear_silu_mul(gu.to(DEV), w.to(DEV), got, lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    _close(got, want, dtype, tol16=1.2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P,rot", [(4, 2, 16, 4, 16), (6, 3, 48, 8, 48), (5, 1, 128, 16, 128),
                                            (2, 2, 80, 2, 32), (3, 1, 256, 16, 256)])
@pytest.mark.parametrize("norm", [True, False])
def test_qk_norm_rope_kv_write(dtype, Hq, Hkv, D, P, rot, norm):
    T, pages = 11, 9
    qkv = _randn((T, (Hq + 2 * Hkv) * D), dtype, 11)
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 7, 40000, 9, 10, 11], dtype=torch.int32)
    qw = (1 + 0.2 * _randn((D,), torch.float32, 12)) if norm else None
    kw = (1 + 0.2 * _randn((D,), torch.float32, 13)) if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    slots = torch.randperm(pages * P, generator=torch.Generator().manual_seed(14))[:T].to(torch.int32)
    cache_ref = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype)
    qkv_ref = qkv.clone()
    ref_ops.qk_norm_rope_kv_write(qkv_ref, positions, qw, kw, 1e-6, inv_freq, rot, cache_ref, slots, Hq, Hkv, D)
    cache_gpu = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype, device=DEV)
    qkv_gpu = qkv.to(DEV)
    ops.qk_norm_rope_kv_write(qkv_gpu, positions.to(DEV), qw.to(DEV) if norm else None, kw.to(DEV) if norm else None,
                              1e-6, inv_freq.to(DEV), rot, cache_gpu, slots.to(DEV), Hq, Hkv, D)
    _close(qkv_gpu, qkv_ref, dtype, tol32=3e-5)
    _close(cache_gpu, cache_ref, dtype, tol32=3e-5)
    # untouched slots stay zero
    mask = torch.ones(pages * P, dtype=torch.bool)
    mask[slots.long()] = False
    flat = cache_gpu.cpu().permute(0, 3, 1, 2, 4).reshape(pages * P, -1)
    assert float(flat[mask].abs().max()) == 0.0


@pytest.mark.parametrize("T,Hq,Hkv,K,P", [(300, 4, 2, 136, 16), (1000, 3, 1, 72, 4), (2048, 16, 8, 1024, 16), (257, 2, 2, 64, 256)])
@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("write_kv", [True, False])
def test_linear_qkv_rope_fused(T, Hq, Hkv, K, P, norm, write_kv):
    """The QKV product with per-head norm, rotation and cache write in its epilogue (head size 128), against
    the plain product followed by the plain norm + rotation + cache write: q in place, k and v in the cache
    only, untouched slots and (without a cache write) the whole cache unchanged; also rows and heads
    that do not fill the 256 x 256 tiles."""
    D, dtype = 128, torch.bfloat16
    N = (Hq + 2 * Hkv) * D
    x = _randn((T, K), dtype, 21)
    w = (_randn((N, K), torch.float32, 22) / math.sqrt(K)).to(dtype)
    positions = torch.randint(0, 40000, (T,), generator=torch.Generator().manual_seed(23), dtype=torch.int32)
    positions[:4] = torch.tensor([0, 1, 2, 39999], dtype=torch.int32)
    qw = (1 + 0.2 * _randn((D,), torch.float32, 24)) if norm else None
    kw = (1 + 0.2 * _randn((D,), torch.float32, 25)) if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    pages = -(-T // P) + 3
    slots = torch.randperm(pages * P, generator=torch.Generator().manual_seed(26))[:T].to(torch.int32)
    # plain: product rounded to bfloat16, then norm + rotation + cache write
    qkv_ref = (x.float() @ w.float().t()).to(dtype)
    cache_ref = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype)
    ref_ops.qk_norm_rope_kv_write(qkv_ref, positions, qw, kw, 1e-6, inv_freq, D, cache_ref, slots, Hq, Hkv, D, write_kv=write_kv)
    table = torch.empty(T, D // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(positions.to(DEV), inv_freq.to(DEV), table)
    cache_gpu = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype, device=DEV)
    qkv_gpu = torch.zeros(T, N, dtype=dtype, device=DEV)
    ops.linear_qkv_rope(x.to(DEV), w.to(DEV), qkv_gpu, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, 1e-6,
                        table, cache_gpu, slots.to(DEV), Hq, Hkv, write_kv=write_kv)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() == 0
    _close(qkv_gpu[:, :Hq * D], qkv_ref[:, :Hq * D], dtype)
    assert float(qkv_gpu[:, Hq * D:].abs().max()) == 0.0          # k and v are not written to the product's buffer
    _close(cache_gpu, cache_ref, dtype)
    mask = torch.ones(pages * P, dtype=torch.bool)
    if write_kv:
        mask[slots.long()] = False
    flat = cache_gpu.cpu().permute(0, 3, 1, 2, 4).reshape(pages * P, -1)
    assert float(flat[mask].abs().max()) == 0.0


@pytest.mark.parametrize("T,Hq,Hkv,K,P", [(1, 16, 8, 1024, 16), (8, 16, 8, 1024, 16), (3, 4, 2, 136, 16), (13, 3, 1, 72, 4),
                                          (16, 32, 8, 2560, 16), (9, 2, 2, 64, 24), (16, 4, 2, 256, 16)])
@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("angles", ["positions", "table", "none"])
@pytest.mark.parametrize("write_kv", [True, False])
def test_linear_qkv_rope_small(T, Hq, Hkv, K, P, norm, angles, write_kv):
    """The QKV product of a few rows with per-head norm, rotation and cache write in its epilogue (a cluster of 8 CTAs
    per head of 128, which exchange sums of squares and rotation partners through distributed shared memory), against
    the plain product followed by the plain norm + rotation + cache write: q in place, k and v in the cache only,
    untouched slots and (without a cache write) the whole cache unchanged; 1 to 16 rows, K down to one slice of a
    single warp, a page size that is no power of two, angles from positions, from the step's table, or none."""
    D, dtype = 128, torch.bfloat16
    N = (Hq + 2 * Hkv) * D
    x = _randn((T, K), dtype, 31)
    w = (_randn((N, K), torch.float32, 32) / math.sqrt(K)).to(dtype)
    positions = torch.randint(0, 40000, (T,), generator=torch.Generator().manual_seed(33), dtype=torch.int32)
    positions[:1] = 39999
    qw = (1 + 0.2 * _randn((D,), torch.float32, 34)) if norm else None
    kw = (1 + 0.2 * _randn((D,), torch.float32, 35)) if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    pages = -(-T // P) + 3
    slots = torch.randperm(pages * P, generator=torch.Generator().manual_seed(36))[:T].to(torch.int32)
    qkv_ref = (x.float() @ w.float().t()).to(dtype)
    cache_ref = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype)
    rotates = angles != "none"
    ref_ops.qk_norm_rope_kv_write(qkv_ref, positions, qw, kw, 1e-6, inv_freq if rotates else None, D if rotates else 0,
                                  cache_ref, slots, Hq, Hkv, D, write_kv=write_kv)
    table = None
    if angles == "table":
        table = torch.empty(T, D // 2, 2, dtype=torch.float32, device=DEV)
        ops.rope_table(positions.to(DEV), inv_freq.to(DEV), table)
    cache_gpu = torch.zeros(pages, 2, Hkv, P, D, dtype=dtype, device=DEV)
    qkv_gpu = torch.zeros(T, N, dtype=dtype, device=DEV)
    assert not ops.QKV_ROPE_SMALL and not ops.qkv_rope_small_applies(T, N, K, dtype, D, D)      # off by default (measured slower than the two kernels)
    ops.linear_qkv_rope_small(x.to(DEV), w.to(DEV), qkv_gpu, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, 1e-6,
                              positions.to(DEV), inv_freq.to(DEV) if rotates else None, table, cache_gpu, slots.to(DEV),
                              Hq, Hkv, write_kv=write_kv)
    torch.cuda.synchronize()
    _close(qkv_gpu[:, :Hq * D], qkv_ref[:, :Hq * D], dtype)
    assert float(qkv_gpu[:, Hq * D:].abs().max()) == 0.0          # k and v are not written to the product's buffer
    _close(cache_gpu, cache_ref, dtype)
    mask = torch.ones(pages * P, dtype=torch.bool)
    if write_kv:
        mask[slots.long()] = False
    flat = cache_gpu.cpu().permute(0, 3, 1, 2, 4).reshape(pages * P, -1)
    assert float(flat[mask].abs().max()) == 0.0


def _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed, spike=None):
    """Build a paged cache with scattered pages for requests with ctx_lens[r] cached tokens and
    q_lens[r] new ones; returns everything both implementations need."""
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    blocks = [-(-t // P) for t in totals]
    n_pages = sum(blocks) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    mb = max(blocks)
    table = torch.full((R, mb), -1, dtype=torch.int32)
    it = iter(perm)
    for r in range(R):
        for b in range(blocks[r]):
            table[r, b] = next(it)
    cache = (torch.randn(n_pages, 2, Hkv, P, D, generator=g)).to(dtype)
    T = sum(q_lens)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).to(dtype)
    if spike is not None:
        # make one far key decide the output: scale the query and that key so its score stands out
        r, key_pos, head = spike
        kvh = head // (Hq // Hkv)
        page, off = int(table[r, key_pos // P]), key_pos % P
        direction = torch.randn(D, generator=g)
        direction = direction / direction.norm()
        cache[page, 0, kvh, off, :] = (direction * 6.0).to(dtype)
        row = sum(q_lens[:r]) + q_lens[r] - 1
        qkv[row, head * D:(head + 1) * D] = (direction * 6.0 * math.sqrt(D)).to(dtype)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    return dict(qkv=qkv, cache=cache, table=table, cu_q=torch.tensor(cu, dtype=torch.int32),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32), T=T)


def _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, fn, dev, flash=True, uniform=None):
    """Run one implementation.  On the GPU ``flash`` lets the step's plan carry the tensor-core
    kernel's work items (used when the kernel takes the geometry); without it the generic kernel runs.
    ``uniform``: every request's context in that many parts, as in a decode step replayed from a graph."""
    from qwen_engine_b200.engine.runner import ModelRunner
    from qwen_engine_b200.parts.base import Arena
    scale = 1.0 / math.sqrt(D)
    geos = ((Hq, Hkv, D, window),) if (flash and dev != "cpu") else ()
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, geos, dtype,
                              uniform_splits={geos[0]: uniform} if uniform and geos else None)
    devplan = ModelRunner._device_plan(
        plan, {"plan_" + k: torch.tensor(v, dtype=torch.int32, device=dev) for k, v in plan.items()}, geos)
    ctx = SimpleNamespace(cu_q=case["cu_q"].to(dev), ctx_lens=case["ctx"].to(dev), attn_plan=devplan,
                          q_lens_host=list(q_lens), ctx_lens_host=list(ctx_lens), arena=Arena(dev))
    out = torch.zeros(case["T"], Hq * D, dtype=dtype, device=dev)
    fn(case["qkv"].to(dev), case["cache"].to(dev), case["table"].to(dev), ctx, out, scale, window, Hq, Hkv, D)
    if dev != "cpu":
        torch.cuda.synchronize()
    return out


ATTN_SHAPES = [(4, 2, 16, 4), (6, 2, 48, 8), (4, 1, 32, 8), (8, 4, 128, 16), (3, 3, 80, 2), (2, 1, 256, 16)]
ATTN_BATCHES = [
    ([13], [0]),                          # a whole short prompt
    ([1], [77]),                          # one decoded token
    ([1, 1, 1], [5, 130, 33]),            # a decode batch
    ([7, 1, 2, 1], [9, 40, 0, 63]),       # portions beside decoded tokens
    ([40], [25]),                         # a portion with earlier context, several query tiles
    ([2, 33], [64, 31]),                  # starts at a page's edge; crosses key tiles
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,P", ATTN_SHAPES)
@pytest.mark.parametrize("q_lens,ctx_lens", ATTN_BATCHES)
@pytest.mark.parametrize("flash", [False, True])
def test_paged_attention(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, flash):
    """flash=False: the generic kernel (the 32-bit path's, and the fallback); flash=True: the
    tensor-core kernel where it takes the geometry (bfloat16), with split contexts merged."""
    if flash and not ops.flash_supported(dtype, Hq, Hkv, D):
        pytest.skip("the generic kernel serves this case")
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=21)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV, flash=flash)
    _close(got, want, dtype, tol32=2e-5, tol16=1.6e-2)


@pytest.mark.parametrize("Hq,Hkv,D,P", [(16, 8, 128, 16), (4, 1, 32, 8), (6, 2, 48, 4), (8, 1, 64, 16)])
@pytest.mark.parametrize("q_lens,ctx_lens", [([1], [1024]), ([1, 1], [257, 2000]), ([3, 1], [700, 511]),
                                             ([1] * 8, [1024] * 8), ([70, 1], [300, 900])])
def test_flash_attention_split_contexts(Hq, Hkv, D, P, q_lens, ctx_lens):
    """Long contexts of decoded tokens are cut into parts that are merged afterwards."""
    dtype = torch.bfloat16
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, 0),), dtype)
    assert plan["fa0_info"][0] > 1, "the case must split"
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=24)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
    _close(got, want, dtype)


@pytest.fixture(params=["mma", "mma4"])
def decode_kernel(request):
    """Which form of the kernel for decoded tokens ``ops.paged_attention`` picks: CTAs of 8 warps where they are
    few (mma), or always 4 warps (mma4)."""
    saved = ops.DECODE_ATTENTION_MMA_WIDE
    ops.DECODE_ATTENTION_MMA_WIDE = request.param == "mma"
    yield request.param
    ops.DECODE_ATTENTION_MMA_WIDE = saved


@pytest.mark.parametrize("Hq,Hkv,P", [(16, 8, 16), (4, 4, 8), (8, 2, 32), (4, 1, 16), (6, 3, 4), (2, 1, 256)])
@pytest.mark.parametrize("q_lens,ctx_lens", [([1], [77]), ([1, 1, 1], [5, 130, 333]), ([1] * 8, [1024] * 8),
                                             ([1, 1], [257, 2000]), ([1, 1, 1, 1], [0, 159, 160, 161]),
                                             ([1], [5000])])
@pytest.mark.parametrize("window", [0, 100])
def test_decode_attention(Hq, Hkv, P, q_lens, ctx_lens, window, decode_kernel):
    """Decoded tokens, head size 128: the kernels made for them (few rows per kv head; key groups or
    chunks, split contexts merged by the last CTA, a window), against the plain reference, and against
    the pipelined mma.sync kernel that serves the same items when they are switched off."""
    D, dtype = 128, torch.bfloat16
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, window),), dtype)
    assert 1 <= plan["fa0_info"][3] <= 4
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=41)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    launches = ops.launch_count
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    assert ops.last_attention_kernel == "decode_attention_mma"
    _close(got, want, dtype)
    saved = ops.DECODE_ATTENTION_MMA
    ops.DECODE_ATTENTION_MMA = False
    try:
        other = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    finally:
        ops.DECODE_ATTENTION_MMA = saved
    assert ops.last_attention_kernel == "flash_attention"
    _close(other, want, dtype)
    assert ops.launch_count == launches + 2


@pytest.mark.parametrize("Hq,Hkv,P", [(16, 8, 16), (4, 4, 8), (8, 1, 32), (6, 3, 4)])
@pytest.mark.parametrize("ctx_lens", [[77], [5, 130, 333], [1024] * 8, [0, 63, 64, 1500], [2000, 1, 700]])
@pytest.mark.parametrize("parts", [2, 4, 8])
@pytest.mark.parametrize("window", [0, 100])
def test_decode_attention_parts_in_clusters(Hq, Hkv, P, ctx_lens, parts, window, decode_kernel):
    """A decode step whose requests are all cut into the same 2, 4 or 8 parts: the parts of a request run as a
    thread-block cluster and meet through distributed shared memory (also parts that hold no key at
    all: short contexts, parts outside the window); the same items merged through scratch memory by the
    last CTA give the same bits."""
    D, dtype = 128, torch.bfloat16
    q_lens = [1] * len(ctx_lens)
    geo = (Hq, Hkv, D, window)
    plan = ops.plan_attention(q_lens, list(ctx_lens), P, (geo,), dtype, uniform_splits={geo: parts})
    assert plan["fa0_info"][4] == parts and plan["fa0_info"][0] == parts * len(ctx_lens)
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=45)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    try:
        got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV, uniform=parts)
        ops.DECODE_ATTENTION_CLUSTERS = False
        other = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV, uniform=parts)
    finally:
        ops.DECODE_ATTENTION_CLUSTERS = True
    _close(got, want, dtype)
    assert torch.equal(got, other)


@pytest.mark.parametrize("Hq,Hkv,P", [(16, 1, 16), (32, 4, 16), (8, 1, 8), (12, 3, 4), (5, 1, 32)])
@pytest.mark.parametrize("q_lens,ctx_lens", [([1], [77]), ([2, 1], [100, 37]), ([1, 1, 1], [5, 130, 1333]), ([1, 2], [3000, 15]),
                                             ([1, 1, 1, 1], [0, 47, 48, 49])])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("stages", [2, 3, 8])
def test_decode_attention_mma_many_rows(Hq, Hkv, P, q_lens, ctx_lens, window, stages, monkeypatch):
    """The tensor-core kernel for decoded tokens with up to 16 rows per kv head (large groups of query
    heads, two tokens of a request in one item), page sizes below and above its key groups, contexts
    that are split and not; against the plain reference.  The case must reach that kernel."""
    D, dtype = 128, torch.bfloat16
    G = Hq // Hkv
    if max(q_lens) * G > 16:
        pytest.skip("more than 16 rows per item: not this kernel's case")
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, window),), dtype)
    assert 1 <= plan["fa0_info"][3] <= 16 and "tc0_items" not in plan
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=47)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    assert ops.DECODE_ATTENTION_MMA
    monkeypatch.setattr(ops, "DECODE_ATTENTION_MMA_WIDE", stages == 8)     # 8: the form with 8 warps (3 stages)
    monkeypatch.setattr(ops, "DECODE_ATTENTION_MMA_STAGES", min(stages, 3))
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    assert ops.last_attention_kernel == "decode_attention_mma"
    _close(got, want, dtype)


def test_decode_attention_mma_asks_for_the_next_layers_cache(monkeypatch):
    """With another layer's cache given (and allowed by size), the kernel asks L2 for that layer's keys and
    values: the output is the same bits, and nothing of the other cache changes."""
    Hq, Hkv, D, P, dtype = 16, 8, 128, 16, torch.bfloat16
    q_lens, ctx_lens = [1, 1, 1], [5, 530, 1333]
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=48)
    plain = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
    assert ops.last_attention_kernel == "decode_attention_mma"
    other = torch.randn_like(case["cache"]).to(DEV)
    before = other.clone()
    monkeypatch.setattr(ops, "DECODE_PREFETCH_KV_MB", 64)

    def with_next(*a, **k):
        return ops.paged_attention(*a, next_pages=other, **k)
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, with_next, DEV)
    assert torch.equal(got, plain) and torch.equal(other, before)


@pytest.mark.parametrize("M,N,K", [(8, 1024, 2048), (3, 389, 80), (16, 72, 1032)])
def test_linear_with_a_hint_of_the_next_weights(M, N, K):
    """A product of a few rows that is told which weights the step reads next asks L2 for them and gives
    the same bits; the hint is used once."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    nxt = torch.randn(1000, 1032, generator=g).bfloat16().to(DEV)          # 2 064 000 bytes: the last piece is partial
    keep = nxt.clone()
    out0 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    out1 = torch.empty_like(out0)
    ops.linear(x, w, out0)
    ops.prefetch_next(nxt)
    ops.linear(x, w, out1)
    assert ops._next_w is None
    torch.cuda.synchronize()
    assert torch.equal(out0, out1) and torch.equal(nxt, keep)


@pytest.mark.parametrize("key_pos", [0, 15, 16, 159, 160, 161, 255, 256, 700, 899])
def test_decode_attention_far_key_stands_out(key_pos, decode_kernel):
    """One key among hundreds carries almost all the weight: the output must be its value.  A kernel
    that misses a page, a chunk or a part would return something else."""
    Hq, Hkv, D, P = 4, 2, 128, 16
    dtype = torch.bfloat16
    q_lens, ctx_lens = [1, 1], [900, 760]
    for r, head in ((0, 1), (1, 2)):
        if key_pos > ctx_lens[r]:
            continue
        case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=42, spike=(r, key_pos, head))
        got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
        want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
        _close(got, want, dtype)


TC_SHAPES = [(16, 8, 128, 16), (4, 4, 128, 8), (8, 1, 128, 32), (4, 2, 128, 128), (2, 1, 128, 256)]
TC_BATCHES = [
    ([300], [0]),                         # a whole prompt: several tiles, the diagonal inside a step
    ([200, 1, 70], [100, 50, 0]),         # portions with and without context beside a decoded token
    ([129, 640], [1000, 77]),             # a long context before a portion; one row more than a half tile
    ([33, 70], [95, 64]),                 # few rows: the second softmax group stays idle for some tiles
]


@pytest.mark.parametrize("Hq,Hkv,D,P", TC_SHAPES)
@pytest.mark.parametrize("q_lens,ctx_lens", TC_BATCHES)
def test_tc_attention(Hq, Hkv, D, P, q_lens, ctx_lens):
    """Prompt portions on the tcgen05 kernel (the plan sends requests with many rows there and the
    rest to the mma.sync kernel), against the plain reference."""
    dtype = torch.bfloat16
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, 0),), dtype)
    assert plan.get("tc0_items"), "the case must reach the tcgen05 kernel"
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=31)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
    assert ops.tc_attention_status() == 0
    _close(got, want, dtype)


@pytest.mark.parametrize("q_lens,ctx_lens", [([2048], [0]), ([1024, 600], [3000, 0]), ([130], [5000])])
def test_tc_attention_parts(q_lens, ctx_lens):
    """Tiles with many key steps are cut into parts that the last CTA merges."""
    Hq, Hkv, D, P = 4, 2, 128, 16
    dtype = torch.bfloat16
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, 0),), dtype)
    assert plan["tc0_info"][0] > 1, "the case must cut tiles into parts"
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=32)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    for _ in range(2):                     # twice: the counters are back at zero after a launch
        got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
        assert ops.tc_attention_status() == 0
        _close(got, want, dtype)


@pytest.mark.parametrize("ctas", [1, 3, 7])
@pytest.mark.parametrize("Hq,Hkv,P,q_lens,ctx_lens,window,cap", [
    (16, 8, 16, [300], [0], 0, 0),                      # three tiles of eight kv heads: every CTA runs several units
    (4, 2, 16, [200, 40, 70], [100, 50, 0], 0, 0),       # units with one softmax group between units with two
    (4, 2, 32, [33, 70, 129, 640], [95, 64, 1000, 77], 0, 0),
    (4, 2, 16, [2048], [0], 0, 8),                      # parts of a tile, merged by whichever CTA comes last
    (4, 2, 16, [1024, 600], [3000, 0], 0, 3),             # many short parts: a CTA may hold several parts of one tile
    (2, 1, 256, [130, 515], [5000, 0], 0, 2),
    (4, 2, 16, [260, 35, 150], [30, 70, 400], 100, 0),   # a window: units of one step, units that begin late
    (4, 4, 8, [700], [0], 129, 2),
])
def test_tc_attention_units_one_after_the_other(ctas, Hq, Hkv, P, q_lens, ctx_lens, window, cap, monkeypatch):
    """With fewer CTAs than work units a CTA runs its units one after the other through the same pipelines (the ring of
    keys and values, tensor memory and the barriers' phases run on across units).  The outputs must be those of the
    plain reference, and to the bit those of a CTA per unit.  (Every request here brings enough rows for this kernel: the
    number of CTAs also sways which form of the kernel for decoded tokens is picked.)"""
    D, dtype = 128, torch.bfloat16
    monkeypatch.setattr(ops, "TC_FORCE_CAP", cap)
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=36)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, window),), dtype)
    units = len(plan["tc0_items"]) // ops.FLASH_ITEM_INTS * Hkv
    assert plan["tc0_info"][2] == min(units, ops.TC_TARGET_CTAS) and not plan.get("fa0_items")
    each = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    _close(each, want, dtype)
    monkeypatch.setattr(ops, "TC_TARGET_CTAS", ctas)
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, window),), dtype)
    sched, n = plan["tc0_sched"], plan["tc0_info"][2]
    assert n == min(ctas, units) and sched[0] == n + 1 and sched[n] == len(sched)
    assert sorted(sched[n + 1:]) == list(range(units)), "every unit is run once"
    for _ in range(2):                     # twice: the merge counters are back at zero after a launch
        got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
        assert ops.tc_attention_status() == 0
        assert torch.equal(got, each)


@pytest.mark.parametrize("seed", range(24))
def test_tc_attention_random_batches(seed, monkeypatch):
    """Random batches, geometries, windows, page sizes, numbers of CTAs and ways of cutting the tiles, against the plain
    reference: whatever the schedule, a row's output is that of its keys."""
    rng = random.Random(1000 + seed)
    Hq, Hkv = rng.choice([(16, 8), (4, 2), (8, 1), (4, 4), (2, 1), (32, 8)])
    P = rng.choice([8, 16, 32, 128])
    window = rng.choice([0, 0, 0, 70, 128, 513])
    n = rng.randint(1, 5)
    q_lens = [rng.choice([1, 2, 40, 64, 65, 127, 128, 129, 200, 333, 700, 1300]) for _ in range(n)]
    ctx_lens = [rng.choice([0, 0, 5, 64, 127, 128, 900, 2100]) for _ in range(n)]
    D, dtype = 128, torch.bfloat16
    monkeypatch.setattr(ops, "TC_TARGET_CTAS", rng.choice([1, 2, 5, 31, 148]))
    monkeypatch.setattr(ops, "TC_FORCE_CAP", rng.choice([-1, -1, 0, 1, 2, 3, 5]))
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=2000 + seed)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    assert ops.tc_attention_status() == 0 and ops.device_status() == {}
    _close(got, want, dtype)


@pytest.mark.parametrize("q_lens,ctx_lens", [([200], [30000]), ([1, 1], [30000, 17]), ([3], [40000])])
def test_attention_long_context(q_lens, ctx_lens):
    """Tens of thousands of keys (the model's limit is 40 960 positions): a portion on the tcgen05
    kernel with its tiles cut into parts, and decoded tokens with split contexts."""
    Hq, Hkv, D, P = 4, 2, 128, 16
    dtype = torch.bfloat16
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=35)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
    assert ops.tc_attention_status() == 0
    _close(got, want, dtype)


@pytest.mark.parametrize("window", [1, 100, 128, 129, 300])
def test_tc_attention_window(window):
    Hq, Hkv, D, P = 4, 2, 128, 16
    dtype = torch.bfloat16
    q_lens, ctx_lens = [260, 1, 150], [30, 70, 400]
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=33)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    assert ops.tc_attention_status() == 0
    _close(got, want, dtype)


@pytest.mark.parametrize("key_pos", [0, 15, 16, 127, 128, 255, 256, 700, 1100])
def test_tc_attention_far_key_stands_out(key_pos):
    """One key among a thousand carries almost all the weight of the last query: the output must
    be its value.  A kernel that misses a page, a step or a part would return something else."""
    Hq, Hkv, D, P = 4, 2, 128, 16
    dtype = torch.bfloat16
    q_lens, ctx_lens = [400, 300], [800, 0]
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=34, spike=(0, key_pos, 3))
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
    assert ops.tc_attention_status() == 0
    _close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 32, 33])
def test_paged_attention_window(dtype, window):
    Hq, Hkv, D, P = 4, 2, 32, 8
    q_lens, ctx_lens = [9, 1, 40], [30, 70, 3]
    case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, seed=22)
    want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ref_ops.paged_attention, "cpu")
    got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, window, ops.paged_attention, DEV)
    _close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("key_pos", [0, 15, 16, 255, 256, 700])
def test_paged_attention_far_key_stands_out(dtype, key_pos):
    """One key among hundreds carries almost all the weight: the output must be its value.
    A kernel that misses a page, a tile or a split would return something else."""
    Hq, Hkv, D, P = 4, 2, 64, 16
    q_lens, ctx_lens = [1, 3], [900, 760]
    for r, head in ((0, 1), (1, 2)):
        case = _attention_case(dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, seed=23, spike=(r, key_pos, head))
        got = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ops.paged_attention, DEV)
        want = _run_attention(case, dtype, Hq, Hkv, D, P, q_lens, ctx_lens, 0, ref_ops.paged_attention, "cpu")
        _close(got, want, dtype)
        row = sum(q_lens[:r]) + q_lens[r] - 1
        page, off = int(case["table"][r, key_pos // P]), key_pos % P
        value = case["cache"][page, 1, head // (Hq // Hkv), off, :].float()
        out = got[row, head * D:(head + 1) * D].float().cpu()
        assert float((out - value).abs().max()) < 0.05, "the far key's value did not come through"


@pytest.mark.parametrize("V", [5, 389, 16383, 16384, 20011, 151936])
def test_argmax(V):
    """Short rows by one CTA, long ones by a cluster whose CTAs take a share of the row each: the largest at
    either end, ties across and within shares, a row of equal values."""
    logits = _randn((6, V), torch.float32, 30)
    logits[1, V - 1] = 50.0
    logits[2, 0] = 50.0
    logits[3, V // 2] = 9.0
    logits[3, V // 3] = 9.0          # a tie: the lower index wins
    logits[3].clamp_(max=9.0)
    logits[4] = -3.5                 # all equal: index 0
    logits[5, V - 2:] = 40.0         # a tie between the last two
    want = torch.empty(6, dtype=torch.int32)
    ref_ops.argmax(logits, want)
    got = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(logits.to(DEV), got)
    assert got.cpu().tolist() == want.tolist()
    assert got[3].item() == min(V // 2, V // 3)


@pytest.mark.parametrize("V", [7, 389, 50021])
def test_sample(V):
    N = 16
    logits = _randn((N, V), torch.float32, 31, 2.0)
    temps = torch.tensor([0.0, 0.8, 1.0, 1.5] * 4)
    top_k = torch.tensor([0, 0, 5, 1, 3, 0, V, V + 5, 2, 50, 0, 0, 7, 7, 1, 0], dtype=torch.int32)
    u = torch.rand(N, generator=torch.Generator().manual_seed(32))
    u[5] = 0.0
    u[6] = 0.99999994
    want = torch.empty(N, dtype=torch.int32)
    ref_ops.sample(logits, temps, top_k, u, want)
    got = torch.empty(N, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), temps.to(DEV), top_k.to(DEV), u.to(DEV), got)
    assert got.cpu().tolist() == want.tolist()
    # top_k = 1 is argmax whatever the temperature
    assert got[3].item() == int(torch.argmax(logits[3]))


def test_a_bounded_wait_that_runs_out():
    """Every wait on an mbarrier inside the tcgen05 kernels is bounded.  Here one is made to run out on
    purpose, without any fault: one CTA of the product kernel whose loads are withheld (no barrier is ever
    armed) and whose waits give up after 10 000 polls.  The kernel must return, store nothing (the output
    keeps its fill value), leave the code of the wait that gave up in the status word, and free its tensor
    memory: the same product launched normally right afterwards is served and is right."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 100, 128, 512                      # 8 k-blocks for a ring of 6 slots: the producer waits for a slot as well
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.clear_device_status()
    assert ops.device_status() == {}
    ops.selftest_starved_product(x, w, out, limit=10000)
    torch.cuda.synchronize()
    assert ops.tcgen05_status() in (1, 2, 3)
    assert set(ops.device_status()) == {"gemm_tc"}
    assert bool((out == 7.0).all()), "a kernel that gave up stored something"
    with pytest.raises(ops.DeviceWaitTimeout, match="gemm_tc"):
        ops.check_device_status()
    assert ops.device_status() == {}             # cleared by the check
    for _ in range(3):                           # tensor memory was freed: the same SMs take full-size products again
        big_x = torch.randn(300, K, generator=g).to(torch.bfloat16).to(DEV)
        got = torch.empty(300, N, dtype=torch.bfloat16, device=DEV)
        lib = ops.lib()
        import ctypes
        rc = lib.qe_linear_tcgen05(ctypes.c_void_p(big_x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(got.data_ptr()),
                                   300, N, K, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        want = big_x.float() @ w.float().t()
        assert float((got.float() - want).abs().max()) <= 2e-2 * float(want.abs().max())
    assert ops.tcgen05_status() == 0


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("I,K", [(3072, 1024), (200, 72), (1032, 264), (16, 8), (9728, 2560)])
def test_linear_swiglu_small(M, I, K):
    """The gate and up projections of a few rows with the activation formed in the product's epilogue (a CTA takes
    the gate rows and the up rows of the same 16 columns), against the plain operations: product, rounding to
    bfloat16, silu(g) * u in float32.  Widths that are no multiple of a warp's share of K, columns no multiple of 16."""
    x = _randn((M, K), torch.bfloat16, 1)
    w = _randn((2 * I, K), torch.bfloat16, 2, K ** -0.5)
    gu = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    want = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).to(torch.bfloat16)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.swiglu_small_applies(M, I, K, torch.bfloat16)
    ops.linear_swiglu_small(x.to(DEV), w.to(DEV), out)
    _close(out, want, torch.bfloat16)


@pytest.mark.parametrize("M", [1, 3, 8, 16])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1024, 3072), (264, 4096)])
def test_cluster_sums_pushed_and_pulled_are_the_same_to_the_bit(M, N, K, monkeypatch):
    """The CTAs of a cluster that share K meet in the first CTA either by pushing their sums into its shared memory
    (st.async counted on its mbarrier; used for single rows) or by being read from there between two cluster
    barriers: the order of the sum is the CTAs' either way, so the results are identical, also when the product
    adds into the residual stream; no status word is set."""
    monkeypatch.setattr(ops, "SMALL_M_ROWS8", False)       # (clusters of two, where 8 rows a CTA would serve otherwise)
    x = _randn((M, K), torch.bfloat16, 13).to(DEV)
    w = _randn((N, K), torch.bfloat16, 14, K ** -0.5).to(DEV)
    outs = {}
    try:
        for mode in (0, 2):
            ops.lib().qe_small_m_push(mode)
            out = torch.empty(M, N, dtype=torch.float32, device=DEV)
            ops.linear(x, w, out)
            stream = ops.ResidualStream.for_step(lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=DEV), M, N, torch.bfloat16)
            stream.resid.fill_(0.25)
            ops.linear(x, w, ops.ResidualSink(stream))
            outs[mode] = (out.cpu(), stream.resid.cpu(), stream.ssq[:, :stream.n_ssq].cpu())
    finally:
        ops.lib().qe_small_m_push(1)
    torch.cuda.synchronize()
    assert ops.device_status() == {}
    for a, b in zip(outs[0], outs[2]):
        assert torch.equal(a, b)
    _close(outs[2][0], x.float().cpu() @ w.float().cpu().t(), torch.bfloat16)


@pytest.mark.parametrize("M", [1, 8, 13, 40])
@pytest.mark.parametrize("N,K", [(1024, 2048), (1024, 3072), (1000, 1032), (592, 4096), (100, 2064), (1184, 1024)])
@pytest.mark.parametrize("mode", ["bf16", "f32", "stream"])
@pytest.mark.parametrize("rows8", [True, False])
def test_linear_small_m_shares_k_in_clusters(M, N, K, mode, rows8, monkeypatch):
    """Weight matrices of few rows: the CTAs of a cluster share 16 weight rows and a part of K each, and meet in
    distributed shared memory (2 or 4 CTAs, chosen from the weight matrix alone); or, where clusters of two would
    serve and 8 rows a CTA fill the SMs (``rows8``), CTAs of 8 rows and the whole of K, no meeting.  Plain output,
    float32 output, and the add into the residual stream with the sums of squares left behind."""
    monkeypatch.setattr(ops, "SPLITK", False)              # (the tcgen05 kernel for some tens of rows is tested elsewhere)
    monkeypatch.setattr(ops, "SMALL_M_ROWS8", rows8)
    ops.lib().qe_small_m_rows8(int(rows8))
    cols = int(ops.lib().qe_small_m_tile_cols(N, K))
    assert cols == (8 if rows8 and (N, K) in ((1024, 2048), (1024, 3072), (1000, 1032), (1184, 1024)) else 16)
    x = _randn((M, K), torch.bfloat16, 3)
    w = _randn((N, K), torch.bfloat16, 4, K ** -0.5)
    want = x.float() @ w.float().t()
    if mode == "stream":
        resid = _randn((M, N), torch.float32, 5)
        stream = ops.ResidualStream.for_step(lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=DEV), M, N, torch.bfloat16)
        stream.resid.copy_(resid)
        ops.linear(x.to(DEV), w.to(DEV), ops.ResidualSink(stream))
        assert not stream.has_delta and stream.n_ssq == -(-N // cols)
        got = stream.resid.cpu()
        _close(got, resid + want, torch.bfloat16)
        ssq = stream.ssq[:, :stream.n_ssq].sum(dim=1).cpu()
        assert torch.allclose(ssq, (got * got).sum(dim=1), rtol=1e-4)
    else:
        out = torch.empty(M, N, dtype=torch.float32 if mode == "f32" else torch.bfloat16, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), out)
        _close(out, want, torch.bfloat16)
