"""The attention entry point that allocates nothing (qwen_engine_b200/csrc/no_alloc.h).

Some users of the library cannot ask for device memory at the moment they need attention: the
device belongs to a pool of their own, or an allocation would stall a loop that has to keep its
timing.  For them the library keeps the scratch memory of flash decoding (the parts of split
contexts) in a fixed 8 MiB array of its own.  This test calls that entry point through its exported
C symbol, twice in a row with different inputs (the array keeps the first call's contents, which
must not leak into the second), and compares with the ordinary entry point, whose scratch comes
from the caller, and with the plain PyTorch attention of tests/ref_ops.py (so that both entry points
being wrong alike would show); it also checks that a request beyond the fixed size is refused, not
truncated.

The file name sorts last, so a run that stops at the first failure has run every other test before.
"""
import ctypes
import math
from types import SimpleNamespace

import pytest
import torch

import ref_ops
from qwen_engine_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, Hq, Hkv, D, P, q_lens, ctx_lens):
    g = torch.Generator().manual_seed(seed)
    totals = [c + n for c, n in zip(ctx_lens, q_lens)]
    blocks = [-(-t // P) for t in totals]
    n_pages = sum(blocks) + 2
    perm = iter(torch.randperm(n_pages, generator=g).tolist())
    table = torch.full((len(q_lens), max(blocks)), -1, dtype=torch.int32)
    for r, nb in enumerate(blocks):
        for b in range(nb):
            table[r, b] = next(perm)
    cache = torch.randn(n_pages, 2, Hkv, P, D, generator=g).to(torch.bfloat16)
    qkv = torch.randn(sum(q_lens), (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    return dict(qkv=qkv.to(DEV), cache=cache.to(DEV), table=table.to(DEV),
                cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV))


def _plan(Hq, Hkv, D, P, q_lens, ctx_lens):
    plan = ops.plan_attention(list(q_lens), list(ctx_lens), P, ((Hq, Hkv, D, 0),), torch.bfloat16)
    items = torch.tensor(plan["fa0_items"], dtype=torch.int32, device=DEV)
    merge = torch.tensor(plan["fa0_merge"], dtype=torch.int32, device=DEV)
    n_parts, part_rows = plan["fa0_info"][:2]
    return items, merge, n_parts, part_rows


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


def _run(entry, case, plan, Hq, Hkv, D, P, with_scratch):
    items, merge, n_parts, part_rows = plan
    T = case["qkv"].shape[0]
    out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    lib = ops.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [_p(case["qkv"]), ctypes.c_long(case["qkv"].stride(0)), _p(case["cache"]), _p(case["table"]),
              int(case["table"].shape[1]), _p(case["cu_q"]), _p(case["ctx"]), _p(items), items.numel() // ops.FLASH_ITEM_INTS,
              _p(merge), merge.numel() // 4, _p(out)]
    tail = [ctypes.c_float(1.0 / math.sqrt(D)), 0, Hq, Hkv, D, P, stream]
    if with_scratch:
        slots = max(1, n_parts * Hkv * part_rows)
        acc = torch.empty(slots, D, dtype=torch.float32, device=DEV)
        ml = torch.empty(slots, 2, dtype=torch.float32, device=DEV)
        rc = lib.qe_flash_attention(*common, _p(acc), _p(ml), int(part_rows), *tail)
        torch.cuda.synchronize()
        return rc, out, 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]        # what the driver has left: any cudaMalloc would lower it
    rc = entry(*common, int(n_parts), int(part_rows), *tail)
    torch.cuda.synchronize()
    return rc, out, free_before - torch.cuda.mem_get_info()[0]


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = ops.lib()
    entry = lib.qe_flash_attention_noalloc          # the exported C symbol
    Hq, Hkv, D, P = 16, 8, 128, 16
    shapes = [([1] * 8, [1024] * 8), ([1, 3, 1], [2000, 300, 515])]
    for i, (q_lens, ctx_lens) in enumerate(shapes):            # two calls in a row, different inputs
        case = _case(100 + i, Hq, Hkv, D, P, q_lens, ctx_lens)
        plan = _plan(Hq, Hkv, D, P, q_lens, ctx_lens)
        assert plan[2] > 1, "the case must split contexts, or no scratch is used"
        rc, got, taken = _run(entry, case, plan, Hq, Hkv, D, P, with_scratch=False)
        assert rc == 0, lib.qe_last_error().decode()
        if i > 0:                                  # (the very first launch of a kernel may load its code)
            assert taken == 0, f"the call took {taken} bytes of device memory"
        rc, want, _ = _run(entry, case, plan, Hq, Hkv, D, P, with_scratch=True)
        assert rc == 0, lib.qe_last_error().decode()
        assert torch.isfinite(got.float()).all()
        scale = max(1.0, float(want.float().abs().max()))
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1.6e-2 * scale, f"call {i}: max |diff| {err}"
        assert torch.equal(got, want), "same kernels, same order of sums: the bits agree"
        # and against the plain attention (float32 on the CPU, from the same bfloat16 inputs)
        plain = torch.zeros(got.shape, dtype=torch.float32)
        ref_ops.paged_attention(case["qkv"].cpu(), case["cache"].cpu(), case["table"].cpu(),
                                SimpleNamespace(cu_q=case["cu_q"].cpu(), ctx_lens=case["ctx"].cpu()), plain,
                                1.0 / math.sqrt(D), 0, Hq, Hkv, D)
        err = float((got.float().cpu() - plain).abs().max())
        assert err <= 1.6e-2 * max(1.0, float(plain.abs().max())), f"call {i}: max |diff| to the plain attention {err}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = ops.lib()
    Hq, Hkv, D, P = 32, 32, 256, 16
    q_lens, ctx_lens = [1] * 2, [9000] * 2
    case = _case(7, Hq, Hkv, D, P, q_lens, ctx_lens)
    items, merge, n_parts, part_rows = _plan(Hq, Hkv, D, P, q_lens, ctx_lens)
    big_parts = 4096                                  # 4096 x 32 x 1 x 258 x 4 bytes = 129 MiB > 8 MiB
    rc, out, _ = _run(lib.qe_flash_attention_noalloc, case, (items, merge, big_parts, part_rows), Hq, Hkv, D, P, False)
    assert rc == 1
    assert "scratch" in lib.qe_last_error().decode()
    assert float(out.float().abs().max()) == 0.0, "a refused call launches nothing"
