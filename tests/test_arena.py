"""The step's scratch allocator (qwen_engine_b200/parts/base.py: Arena) on the CPU: stack discipline for
the layers' intermediates, memory that lives for the whole step beside it, growth after an overflow."""
import torch

from qwen_engine_b200.parts.base import Arena


def _span(t):
    return t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()


def _overlap(a, b):
    (a0, a1), (b0, b1) = _span(a), _span(b)
    return a0 < b1 and b0 < a1


def test_layers_reuse_their_scratch_and_step_memory_survives_them():
    ar = Arena("cpu", 1 << 16)
    ar.reset()
    m = ar.mark()
    a = ar.alloc((10, 64), torch.float32)
    table = ar.alloc_step((8, 64, 2), torch.float32)           # made inside the first layer's frame
    b = ar.alloc((10, 64), torch.float32)
    ar.release(m)
    for _ in range(3):                                         # the next layers: the same frame again
        m = ar.mark()
        a2 = ar.alloc((10, 64), torch.float32)
        c = ar.alloc((40, 64), torch.float32)                  # more than the first layer took after `a`
        assert a2.data_ptr() == a.data_ptr()
        assert not _overlap(c, table) and not _overlap(a2, table)
        ar.release(m)
    assert not _overlap(b, table)
    # the same sequence in the next step gives the same addresses (steps replayed from CUDA graphs rely on it)
    ar.reset()
    m = ar.mark()
    assert ar.alloc((10, 64), torch.float32).data_ptr() == a.data_ptr()
    assert ar.alloc_step((8, 64, 2), torch.float32).data_ptr() == table.data_ptr()


def test_bump_and_step_allocations_never_meet():
    ar = Arena("cpu", 4096)
    ar.reset()
    s1 = ar.alloc_step((256,), torch.float32)                  # 1 KB from the far end
    x = ar.alloc((512,), torch.float32)                        # 2 KB from the near end
    y = ar.alloc((512,), torch.float32)                        # does not fit between them: a tensor of its own
    s2 = ar.alloc_step((512,), torch.float32)                  # nor does this
    ts = [s1, x, y, s2]
    assert all(not _overlap(p, q) for i, p in enumerate(ts) for q in ts[i + 1:])
    assert ar._overflow
    ar.reset()                                                 # grown: now everything fits in the buffer
    lo, hi = ar.buffer.data_ptr(), ar.buffer.data_ptr() + ar.capacity
    ts = [ar.alloc_step((256,), torch.float32), ar.alloc((512,), torch.float32), ar.alloc((512,), torch.float32),
          ar.alloc_step((512,), torch.float32)]
    assert not ar._overflow
    assert all(lo <= _span(t)[0] and _span(t)[1] <= hi for t in ts)
    assert all(not _overlap(p, q) for i, p in enumerate(ts) for q in ts[i + 1:])


def test_a_remembered_view_is_not_handed_out_over_step_memory():
    ar = Arena("cpu", 4096)
    ar.reset()
    big = ar.alloc((768,), torch.float32)                      # 3 KB: remembered for offset 0
    ar.reset()
    s = ar.alloc_step((512,), torch.float32)                   # 2 KB at the far end
    again = ar.alloc((768,), torch.float32)                    # the remembered view would run into it
    assert not _overlap(again, s)
