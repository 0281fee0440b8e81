"""The engine's operations: thin Python fronts of the hand-written CUDA kernels.

Every function works on CUDA tensors, writes into an output the caller
provides, and launches on torch's current stream.  There is no CPU path and no
library fallback: without the compiled extension, or with a tensor that is not
on a CUDA device, a call raises.  The plain PyTorch restatement of each
operation lives with the tests (tests/ref_ops.py).
"""
from __future__ import annotations

import ctypes
import os
import struct
from typing import Optional

import torch

from ..csrc import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_lib = None

ATTN_TILE_Q = 16        # queries per work item of the generic attention kernel
SMALL_M_MAX = 64        # rows up to which the weight-streaming product is used
SPLITK = True           # products of some tens of rows by clusters of CTAs that share K (gemm_tcgen05_splitk.cu)
SPLITK_MIN_M = 17       # rows from which, up to SPLITK_MAX_M, that kernel serves
SPLITK_MAX_M = 64
SPLITK_MAX_CTAS = 148   # clusters x CTAs at most: all on the GPU at once
SPLITK_LONG_K = 4096    # K from which that kernel serves from SPLITK_LONG_K_MIN_M rows on, where the weight rows / 16 exceed the SMs (0: never)
SPLITK_LONG_K_MIN_M = 9
SPLITK_VERY_LONG_K = 8192   # K from which, under the same conditions, every number of rows goes there (Qwen3-4B's down product)
SPLITK_VERY_LONG_K_MIN_M = 1
SPLITK_MAX_CLUSTERS_OF_8 = 8   # clusters of 8 CTAs at most (16 of them, 2 048 weight rows, took 8.9 us where 16 clusters of 4 take 5.5: a
                               # cluster needs its SMs in one part of the GPU)
SWAP_MIN_M = 17         # rows from which, up to SMALL_M_MAX, wide products go to the swapped tcgen05 kernel
SWAP_MIN_N = 3072       # weight rows from which it has enough CTAs (one per 128) to pull the weights fast enough
SWIGLU_FUSED = True     # SiLU-mul in the epilogue of the gate/up product where the CTA-pair kernel serves it
TCGEN05_PAIRS = True    # CTA pairs for large products
PAIR_MIN_TILES = 74     # 256 x 256 tiles from which they are used (one per pair of SMs)
TCGEN05_ENABLED = True  # the tcgen05 product for more rows (False: the generic kernel serves them)
FLASH_ROWS = 64         # rows (query token x query head of a group) per work item of the flash kernel
FLASH_BN = 64           # keys per tile of the flash kernel
FLASH_ITEM_INTS = 12    # int32 per work item of the flash kernel
FLASH_SPLIT = 256       # keys per part when a decoded token's context is split (reference attn.py:605)
FLASH_TARGET_CTAS = 296  # two CTAs per SM: long contexts are split into as many parts as fit in one wave
DECODE_ATTENTION_CLUSTERS = True    # parts of a request as a thread-block cluster that combines them through distributed shared memory
DECODE_ATTENTION_MMA = True         # decoded tokens (up to 16 rows per kv head, head size 128): warps with key groups and pipelines of their own, mma.sync arithmetic
DECODE_ATTENTION_MMA_MIN_CTAS = 0   # CTAs from which that kernel is used
DECODE_ATTENTION_MMA_STAGES = 3     # key groups a warp of that kernel keeps in flight (2 or 3; measured: 3 is 2.5 % ahead in the step)
DECODE_ATTENTION_MMA_EARLY = True   # that kernel requests earlier steps' keys before it waits for the kernel before it
DECODE_ATTENTION_MMA_BESIDE_TC = True   # also for the decoded tokens of a step whose prompt portions go to the tcgen05 kernel
DECODE_ATTENTION_MMA_WIDE = True    # steps with at most as many attention CTAs as SMs: CTAs of 8 warps, one per SM (and contexts split for 148 CTAs, not 296)
DECODE_PREFETCH_KV_MB = 12          # that kernel asks L2 for the next layer's keys and values when a layer's are at most this many MB (0: never).  Measured (0.6B, context 1 024, asked for before the kernel's dependency wait): 4.4 MB (one request) 0.698 -> 0.690 ms a step, 8.8 MB 0.777 -> 0.765, 17.6 MB equal, 35 MB (eight) 0.915 -> 0.957
TC_ROWS = 256           # rows per work item of the tcgen05 attention kernel (two halves of 128)
TC_BN = 128             # keys per step of the tcgen05 attention kernel
TC_MIN_ROWS = 65        # rows of a request's portion from which the tcgen05 kernel serves it
TC_TARGET_CTAS = 148    # one CTA per SM
TC_MIN_PART_STEPS = 4   # key steps of a part at least, when tiles are cut to fill idle SMs
TC_MAX_PARTS = 8        # parts of one tile at most
TC_BALANCE_BELOW_CTAS = 592   # tiles x kv heads below which the tiles' schedule is laid out and long tiles are cut (4 per SM)
TC_ITEM_COST_STEPS = 2.0      # a work unit's first scores, masked step and output, in key steps
TC_PART_COST_STEPS = 5.0      # a part's scratch or merge on top, in key steps (the parts of a step move through L2 together)
TC_FORCE_CAP = -1       # the most key steps of a work item (0: cut nothing); below 0 the library works it out


class ExtensionMissing(RuntimeError):
    """The CUDA extension could not be built or loaded."""


class KernelRefused(ValueError):
    """A kernel refused its arguments (a size it does not take, a wrong dtype)."""


def lib():
    """The loaded extension; builds it at the first call."""
    global _lib
    if _lib is None:
        try:
            path = _build.library_path()
            handle = ctypes.CDLL(path)
        except Exception as e:                       # noqa: BLE001 - re-raised with context
            raise ExtensionMissing(
                f"qwen_engine_b200 needs its CUDA extension and could not get it: {e}") from e
        handle.qe_last_error.restype = ctypes.c_char_p
        _lib = handle
    return _lib


def extension_path() -> str:
    return _build.library_path()


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ExtensionMissing("qwen_engine_b200 ops run on CUDA tensors only (there is no CPU path); "
                               f"got a tensor on {t.device}")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    """The current stream, for a launch."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# torch's own fast paths to the current device and its current stream's handle (the public
# torch.cuda.current_stream() builds a Stream object per call, which costs more than a launch)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


launch_count = 0        # kernels launched through this module since import (read by the benchmark)
last_attention_kernel = ""   # which kernel the last ``paged_attention`` call went to (read by tests)


def _check(rc: int, name: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        msg = lib().qe_last_error().decode("utf-8", "replace")
        if rc == 1:
            raise KernelRefused(msg or f"{name} refused its arguments")
        raise RuntimeError(msg or f"{name} failed with code {rc}")


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelRefused(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelRefused(msg)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------------------

def prepare_matrix(w: torch.Tensor) -> torch.Tensor:
    """A [out, in] matrix as the product kernels want it (row-major, contiguous)."""
    return w.contiguous()


def embedding(token_ids: torch.Tensor, table: torch.Tensor, out,
              ssq: Optional[torch.Tensor] = None) -> None:
    """out[t] = float32(table[token_ids[t]]); out is the float32 residual stream [T, H].  With ``ssq``
    [T, P] float32, ssq[t, 0] gets the row's sum of squares (one partial sum per row).  ``out`` may be a
    ``ResidualStream``: its rows are written and, if it keeps sums of squares, those too."""
    if isinstance(out, ResidualStream):
        stream = out
        embedding(token_ids, table, stream.resid, stream.ssq)
        stream.has_delta, stream.n_ssq = False, (1 if stream.ssq is not None else 0)
        return
    _i32(token_ids, "token_ids")
    T, (V, H) = token_ids.numel(), table.shape
    _need(out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous(), "embedding: out must be float32 [T, H]")
    _need(table.is_contiguous(), "embedding: table must be contiguous")
    if ssq is not None:
        _need(ssq.dtype == torch.float32 and ssq.dim() == 2 and ssq.shape[0] == T and ssq.is_contiguous(),
              "embedding: ssq must be float32 [T, P]")
    _check(lib().qe_embedding(_ptr(token_ids), _ptr(table), _ptr(out), T, H, V, _dt(table), _ptr(ssq),
                              int(ssq.shape[1]) if ssq is not None else 0, _stream()), "embedding")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    """resid += delta (if given), in place in float32; out = rmsnorm(resid) * weight."""
    T, H = resid.shape
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "add_rmsnorm: resid must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,), "add_rmsnorm: weight must be float32 [H]")
    _need(out.shape == (T, H) and out.is_contiguous(), "add_rmsnorm: out must be contiguous [T, H]")
    if delta is not None:
        _need(delta.shape == (T, H) and delta.dtype == out.dtype and delta.is_contiguous(),
              "add_rmsnorm: delta must match out")
    _check(lib().qe_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(None), _ptr(weight), ctypes.c_float(eps),
                                _ptr(out), T, H, _dt(out), _stream()), "add_rmsnorm")


def add_rmsnorm_rows(resid: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor,
                     weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[n] = rmsnorm(resid[rows[n]] + delta[rows[n]]) * weight; resid is not changed."""
    _i32(rows, "rows")
    N, H = out.shape
    _need(rows.numel() >= N, "add_rmsnorm_rows: fewer rows than outputs")
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[1] == H,
          "add_rmsnorm_rows: resid must be contiguous float32 [T, H]")
    _need(weight.dtype == torch.float32 and weight.shape == (H,), "add_rmsnorm_rows: weight must be float32 [H]")
    _need(out.is_contiguous(), "add_rmsnorm_rows: out must be contiguous")
    if delta is not None:
        _need(delta.shape == resid.shape and delta.dtype == out.dtype and delta.is_contiguous(),
              "add_rmsnorm_rows: delta must match")
    _check(lib().qe_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), ctypes.c_float(eps),
                                _ptr(out), N, H, _dt(out), _stream()), "add_rmsnorm_rows")


class ResidualStream:
    """The float32 residual stream of a step, with the output of the last branch still to be added.

    ``resid`` [T, H] float32 is the stream.  A branch (mixer or feed-forward) either adds its output
    into it at once (``ResidualSink``), or leaves it in ``delta`` [T, H] (compute dtype) with
    ``has_delta`` set, to be added by the next norm.  ``ssq`` [T, P] float32 holds ``n_ssq`` partial
    sums of squares of every row of ``resid`` when the kernel that last wrote the stream left them
    (``n_ssq`` = 0: unknown); a norm fused into the next product starts from them."""

    def __init__(self, resid: torch.Tensor, delta: torch.Tensor, ssq: Optional[torch.Tensor] = None):
        self.resid, self.delta, self.ssq = resid, delta, ssq
        self.has_delta = False
        self.n_ssq = 0

    @classmethod
    def for_step(cls, alloc, num_tokens: int, width: int, dtype: torch.dtype) -> "ResidualStream":
        """The stream of a step of ``num_tokens`` rows of ``width``, from ``alloc(shape, dtype)``.  For a few rows
        in bfloat16 it also gets room for the partial sums of squares that the products which add into the
        stream leave behind (one per 16 or per 8 columns, padded to whole float4s): their layout is the kernels'
        business, so it is settled here, beside their fronts, and not by the model."""
        ssq = None
        if dtype == torch.bfloat16 and num_tokens <= SMALL_M_MAX:
            ssq = alloc((num_tokens, -(-(-(-width // 8)) // 4) * 4), torch.float32)
        return cls(alloc((num_tokens, width), torch.float32), alloc((num_tokens, width), dtype), ssq)


class ResidualSink:
    """Given to ``linear`` / ``linear_silu_mul`` as ``out``: the product is a branch's output and is to be
    added to the residual stream.  For a few rows in bfloat16 the add happens in the product's epilogue
    (which also leaves the rows' sums of squares for the next norm); otherwise the product goes to
    ``stream.delta`` and the next norm adds it."""

    def __init__(self, stream: ResidualStream):
        self.stream = stream

    def as_delta(self) -> torch.Tensor:
        st = self.stream
        st.has_delta, st.n_ssq = True, 0
        return st.delta


class NormedInput:
    """``rmsnorm(stream.resid + stream.delta) * weight`` that is not computed yet.

    ``linear`` takes it in the place of a tensor: for a few rows in bfloat16, when the stream is up to
    date and its sums of squares are known, the norm runs inside the product kernel (no kernel and no
    buffer between them); otherwise, and for any other consumer, ``materialize`` runs the add-and-norm
    kernel once and returns the tensor."""

    def __init__(self, stream: ResidualStream, weight: torch.Tensor, eps: float, alloc, dtype: torch.dtype):
        self.stream, self.weight, self.eps, self.alloc, self.dtype = stream, weight, float(eps), alloc, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.stream.resid.shape

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            st = self.stream
            out = self.alloc(tuple(st.resid.shape), self.dtype)
            add_rmsnorm(st.resid, st.delta if st.has_delta else None, self.weight, self.eps, out)
            if st.has_delta:
                st.has_delta, st.n_ssq = False, 0
            self._tensor = out
        return self._tensor


# What is fused into the products of a few rows was settled by measurement on a B200 (decode, batch 8,
# context 1024, tokens/s with / without):
#   the norm of the stream into the product that follows it   0.6B 6 480 / 6 920, 1.7B 4 340 / 4 580, 4B 1 570 / 1 970:
#       off.  Every CTA (16 weight rows) reads all of x; in float32 with the norm's arithmetic that costs
#       more than the norm kernel's launch.  Kept as a tested option.
#   SiLU-mul into the product that consumes it               0.6B equal, 4B 1 960 / 2 080: on up to 4 096 columns
#       of gate/up per half (every CTA reads both halves of gate_up).
#   the branch's add into the stream in the product's epilogue   0.6B 6 870 / 6 820, 4B 2 070 / 1 740: on.
SMALL_M_ROWS8 = False   # products of a few rows with so few weight rows that clusters of two share 16: 8 rows a CTA instead (a tested
                        # option that is off: no meeting, but every CTA reads all of x, and the batch-8 step went from 0.919 to 0.941 ms)
FUSED_NORM_MAX_M = 0    # rows up to which a norm is fused into the product that follows (0: never)
FUSED_SILU_MAX_M = 64   # rows up to which SiLU-mul is formed by the product that consumes it ...
FUSED_SILU_MAX_K = 4096  # ... when the activation has at most this many columns
RESID_SINK_MAX_M = 64   # rows up to which a branch's last product adds into the stream itself


def _linear_normed(x: NormedInput, w: torch.Tensor, out: torch.Tensor) -> bool:
    """The fused route of ``linear`` for a NormedInput; False if it does not apply."""
    st = x.stream
    M, K = st.resid.shape
    N = w.shape[0]
    if not (x._tensor is None and not st.has_delta and st.n_ssq > 0 and st.ssq is not None
            and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and M <= FUSED_NORM_MAX_M
            and K % 8 == 0 and st.resid.is_cuda and isinstance(out, torch.Tensor)):
        return False
    _need(w.shape == (N, K) and out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
          and w.is_contiguous() and out.is_contiguous(), "linear: operands do not fit the normed input")
    _check(lib().qe_linear_small_m_norm(_ptr(st.resid), _ptr(st.ssq), int(st.n_ssq), int(st.ssq.shape[1]),
                                        _ptr(x.weight), ctypes.c_float(x.eps), _ptr(w), _ptr(out), M, N, K,
                                        int(out.dtype == torch.float32), _stream()), "linear")
    return True


def splitk_splits(M: int, N: int, K: int, dtype: torch.dtype) -> int:
    """How many CTAs share a tile of 128 weight rows, each with a share of K, in the product of some tens
    of rows (``linear_splitk``): as many of 8, 4, 2 as keep all clusters on the GPU at once (8 only for few clusters); 0 where that
    kernel does not apply (few rows, enough weight rows for every SM, other types)."""
    if not (TCGEN05_ENABLED and SPLITK and dtype == torch.bfloat16 and M <= SPLITK_MAX_M and K % 8 == 0 and N % 4 == 0):
        return 0
    # From 9 rows on already (from the first, where K is very long) where the streaming kernel is at its worst: more CTAs of 16 weight rows than SMs (they do not
    # all start at once), a long K, and two tiles of tokens per instruction; then only with 4 or 8 CTAs per cluster.
    early = (SPLITK_LONG_K > 0 and K >= SPLITK_LONG_K and -(-N // 16) > SPLITK_MAX_CTAS
             and M >= (SPLITK_VERY_LONG_K_MIN_M if 0 < SPLITK_VERY_LONG_K <= K else SPLITK_LONG_K_MIN_M))
    if M < SPLITK_MIN_M and not early:
        return 0
    tiles = -(-N // 128)
    for s in (8, 4, 2):
        if s == 8 and tiles > SPLITK_MAX_CLUSTERS_OF_8:
            continue
        if tiles * s <= SPLITK_MAX_CTAS and -(-K // 64) >= 2 * s:
            return s if (M >= SPLITK_MIN_M or s >= 4) else 0
    return 0


def linear_splitk(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, splits: int, add: bool = False) -> None:
    """``linear`` in bfloat16 for up to 64 rows by clusters of ``splits`` CTAs that share 128 weight rows
    and meet through distributed shared memory; ``add``: out (float32) += the product."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape == (N, K), "linear_splitk: bfloat16 operands, w [N, K]")
    _need(out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32) and (not add or out.dtype == torch.float32),
          "linear_splitk: out must be [M, N], float32 to be added to")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_splitk: operands must be contiguous")
    mode = 2 if add else int(out.dtype == torch.float32)
    _check(lib().qe_linear_tcgen05_splitk(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(splits), mode, _stream()), "linear_splitk")


def _linear_into_stream(x: torch.Tensor, w: torch.Tensor, sink: ResidualSink, silu: bool) -> bool:
    """The fused route for a ResidualSink: resid += product, sums of squares left behind."""
    st = sink.stream
    M = x.shape[0]
    K = x.shape[1] // 2 if silu else x.shape[1]
    N = w.shape[0]
    if not silu and x.is_cuda and not st.has_delta and st.resid.shape == (M, N) and st.resid.is_contiguous():
        splits = splitk_splits(M, N, K, x.dtype)
        if splits:
            # some tens of rows: clusters that share K add their sum to the stream in their epilogue
            linear_splitk(x, w, st.resid, splits, add=True)
            st.n_ssq = 0
            return True
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= min(SMALL_M_MAX, RESID_SINK_MAX_M) and K % 8 == 0
            and not st.has_delta and st.ssq is not None and st.resid.shape == (M, N)):
        return False
    lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
    cols = int(lib().qe_small_m_tile_cols(N, K))        # columns of a CTA: it leaves one partial sum of squares per row
    if st.ssq.shape[1] < -(-N // cols):
        return False
    _need(w.shape == (N, K) and x.is_contiguous() and w.is_contiguous(), "linear: operands do not fit")
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_resid(_ptr(x), _ptr(w), _ptr(st.resid), _ptr(st.ssq), int(st.ssq.shape[1]),
                                         M, N, K, int(silu), _stream()), "linear")
    st.n_ssq = -(-N // cols)
    return True


PREFETCH_NEXT_WEIGHTS = True   # products of a few rows ask L2 for the weights of the product that follows them
PREFETCH_NEXT_MAX_MB = 32      # ... when those are at most this many MB


def prefetch_next(w: Optional[torch.Tensor]) -> None:
    """Tell the next ``linear`` / ``linear_silu_mul`` call which weights the step reads after its own
    (None: none).  Where that call is served by the kernel for a few rows, its CTAs ask L2 for them once
    their own weights are on their way; every other kernel ignores the hint.  One call takes it."""
    global _next_w
    _next_w = None
    if (w is not None and PREFETCH_NEXT_WEIGHTS and w.is_cuda and w.is_contiguous()
            and w.numel() * w.element_size() <= PREFETCH_NEXT_MAX_MB << 20):
        _next_w = w


_next_w: Optional[torch.Tensor] = None


def _hand_over_next_weights() -> None:
    """Before a launch of the kernel for a few rows: the pending hint goes to the library (and is cleared)."""
    global _next_w
    if _next_w is not None:
        w, _next_w = _next_w, None
        lib().qe_small_m_prefetch_next(_ptr(w), ctypes.c_ulonglong(w.numel() * w.element_size()))


def linear(x, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] · w[N, K]^T, float32 accumulation; out in x's dtype or float32.
    ``x`` may be a NormedInput (see there)."""
    if isinstance(x, NormedInput):
        if _linear_normed(x, w, out):
            return
        x = x.materialize()
    if isinstance(out, ResidualSink):
        if _linear_into_stream(x, w, out, silu=False):
            return
        out = out.as_delta()
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape == (N, K) and w.dtype == x.dtype, f"linear: w {tuple(w.shape)} {w.dtype} does not fit x {tuple(x.shape)} {x.dtype}")
    _need(out.shape == (M, N) and out.dtype in (x.dtype, torch.float32), "linear: out must be [M, N] in x's dtype or float32")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
    out_f32 = int(out.dtype == torch.float32)
    splits = splitk_splits(M, N, K, x.dtype)
    if splits:
        linear_splitk(x, w, out, splits)
        return
    if (x.dtype == torch.bfloat16 and SWAP_MIN_M <= M <= SMALL_M_MAX and N >= SWAP_MIN_N and K % 8 == 0
            and TCGEN05_ENABLED):
        # some tens of rows and many weight rows: the weights on the 128-row side of tcgen05.mma
        _check(lib().qe_linear_tcgen05_swap(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    if x.dtype == torch.bfloat16 and M <= SMALL_M_MAX and K % 8 == 0:
        # a few rows: stream every weight once through the tensor cores
        _hand_over_next_weights()
        lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
        _check(lib().qe_linear_small_m(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    if (x.dtype == torch.bfloat16 and TCGEN05_PAIRS and TCGEN05_ENABLED and K % 8 == 0
            and (-(-M // 256) * -(-N // 256) >= PAIR_MIN_TILES
                 or (PAIR_PLAN and M > SMALL_M_MAX and tc_product_plan(M, N, K) != 0))):
        # pairs of CTAs share a 256-row tile (tcgen05 cta_group::2): enough 256 x 256 tiles for every pair of SMs,
        # or the library's model of the kernels' times says so (fewer tiles: wide tiles all the same, or 2 or 4 pairs
        # per tile with a share of a long K each, meeting on chip)
        linear_pairs(x, w, out)
        return
    if x.dtype == torch.bfloat16 and M > SMALL_M_MAX and K % 8 == 0 and TCGEN05_ENABLED:
        # many rows: TMA-fed tcgen05 tensor cores with the accumulator in tensor memory
        _check(lib().qe_linear_tcgen05(_ptr(x), _ptr(w), _ptr(out), M, N, K, out_f32, _stream()), "linear")
        return
    _check(lib().qe_linear_generic(_ptr(x), _ptr(w), _ptr(out), M, N, K, _dt(x), out_f32, _stream()), "linear")


PAIR_PLAN = True        # products of many rows with fewer than PAIR_MIN_TILES tiles go where the library's model of the kernels' times sends them


def tc_product_plan(M: int, N: int, K: int) -> int:
    """Which tcgen05 kernel serves a plain bfloat16 product of more than 64 rows: 0 the single-CTA kernel, 1 CTA
    pairs with 256 x 128 tiles, 2 with 256 x 256 tiles, 3 / 4 with K split over 2 / 4 pairs per tile."""
    return int(lib().qe_tc_product_plan(int(M), int(N), int(K), 0))


def pair_k_splits(M: int, N: int, K: int) -> int:
    """Into how many CTA pairs per 256 x 256 tile ``linear_pairs`` splits K for this shape (1: it does not)."""
    return int(lib().qe_pair_k_splits(int(M), int(N), int(K), 0))


def linear_pairs(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` in bfloat16 by the kernel in which two CTAs share a 256-row tile; any number of rows
    (few tiles: 256 x 128 tiles; ``linear`` itself comes here only for large products)."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape == (N, K) and K % 8 == 0,
          "linear_pairs: bfloat16 operands with K a multiple of 8")
    _need(out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32), "linear_pairs: out must be [M, N]")
    _need(x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_pairs: operands must be contiguous")
    _check(lib().qe_linear_tcgen05_pair(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(out.dtype == torch.float32), _stream()),
           "linear_pairs")


def swiglu_fused_applies(M: int, I: int, K: int, dtype: torch.dtype) -> bool:
    """Whether ``linear_swiglu`` serves this shape: bfloat16, more rows than the weight-streaming products
    take, and enough 256-row x 128-column tiles of the activation for every pair of SMs (the kernel is the
    CTA-pair product)."""
    return (TCGEN05_PAIRS and TCGEN05_ENABLED and SWIGLU_FUSED and dtype == torch.bfloat16 and K % 8 == 0
            and M > SMALL_M_MAX and -(-M // 256) * -(-I // 128) >= PAIR_MIN_TILES)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(x · w[:I]^T) * (x · w[I:]^T) for the stacked weights w [2 I, K]: the feed-forward's
    activation formed in the product's epilogue on its float32 sums (bfloat16, many rows)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape == (2 * I, K) and K % 8 == 0,
          "linear_swiglu: bfloat16 operands, w [2 I, K] with K a multiple of 8")
    _need(out.shape == (M, I) and out.dtype in (torch.bfloat16, torch.float32), "linear_swiglu: out must be [M, I]")
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and out.is_contiguous(), "linear_swiglu: operands must be contiguous")
    _check(lib().qe_linear_swiglu_tcgen05_pair(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K,
                                               int(out.dtype == torch.float32), _stream()), "linear_swiglu")


SWIGLU_SMALL_MAX_M = 16     # rows up to which the weight-streaming product forms the activation in its epilogue


def swiglu_small_applies(M: int, I: int, K: int, dtype: torch.dtype) -> bool:
    """Whether ``linear_swiglu_small`` serves this shape: a few rows in bfloat16."""
    return dtype == torch.bfloat16 and 1 <= M <= SWIGLU_SMALL_MAX_M and K % 8 == 0


def linear_swiglu_small(x, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(x · w[:I]^T) * (x · w[I:]^T) for the stacked weights w [2 I, K] and a few rows (decode steps):
    a CTA streams the gate rows and the up rows of the same 16 columns and forms the activation in its epilogue, so
    that gate and up never exist in memory and the product that follows reads half the bytes, already activated."""
    if isinstance(x, NormedInput):
        x = x.materialize()
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_gate_up.shape == (2 * I, K) and K % 8 == 0,
          "linear_swiglu_small: bfloat16 operands, w [2 I, K] with K a multiple of 8")
    _need(out.shape == (M, I) and out.dtype == torch.bfloat16 and M <= SWIGLU_SMALL_MAX_M,
          f"linear_swiglu_small: out must be bfloat16 [M, I] with M <= {SWIGLU_SMALL_MAX_M}")
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and out.is_contiguous(), "linear_swiglu_small: operands must be contiguous")
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_swiglu(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K, _stream()), "linear_swiglu_small")


QKV_ROPE_FUSED = True       # many rows: per-head norm, rotation and cache write in the epilogue of the QKV product
QKV_ROPE_MIN_TILES = 74     # 256 x 256 tiles of the product from which it is used (one per pair of SMs)


def qkv_rope_fused_applies(M: int, N: int, K: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``linear_qkv_rope`` serves this shape: bfloat16, head size 128 rotated as a whole, and
    enough 256 x 256 tiles for every pair of SMs (the kernel is the CTA-pair product)."""
    return (QKV_ROPE_FUSED and TCGEN05_PAIRS and TCGEN05_ENABLED and dtype == torch.bfloat16
            and head_dim == 128 and rotary_dim == 128 and K % 8 == 0 and N % 128 == 0
            and M > SMALL_M_MAX and -(-M // 256) * -(-N // 256) >= QKV_ROPE_MIN_TILES)


def linear_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                    k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                    kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                    num_heads: int, num_kv_heads: int, write_kv: bool = True) -> None:
    """The QKV product with what ``qk_norm_rope_kv_write`` would do to it afterwards done in its epilogue
    (head size 128, bfloat16): qkv[:, :Hq 128] = rotated, normed q; the rotated, normed k and v go to their
    slots in ``kv_pages`` [pages, 2, Hkv, page, 128] only (the k and v columns of ``qkv`` are not written).
    ``cos_sin``: float32 [T, 64, 2], the step's table of angles (None: no rotation)."""
    M, K = x.shape
    Hq, Hkv = num_heads, num_kv_heads
    N = (Hq + 2 * Hkv) * 128
    _need(x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and w_qkv.shape == (N, K) and K % 8 == 0,
          "linear_qkv_rope: bfloat16 operands, w [(Hq + 2 Hkv) 128, K] with K a multiple of 8")
    _need(qkv.shape == (M, N) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and x.is_contiguous() and w_qkv.is_contiguous(),
          "linear_qkv_rope: qkv must be contiguous bfloat16 [M, (Hq + 2 Hkv) 128]")
    for wt in (q_norm_w, k_norm_w):
        _need(wt is None or (wt.dtype == torch.float32 and wt.shape == (128,)), "linear_qkv_rope: norm weights must be float32 [128]")
    _need(cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (M, 64, 2) and cos_sin.is_contiguous()),
          "linear_qkv_rope: cos_sin must be float32 [M, 64, 2]")
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None and kv_pages.dtype == torch.bfloat16 and kv_pages.is_contiguous()
              and kv_pages.dim() == 5 and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == 128,
              "linear_qkv_rope: kv_pages must be bfloat16 [pages, 2, Hkv, page, 128]")
        _i32(slot_mapping, "slot_mapping")
        _need(slot_mapping.numel() >= M, "linear_qkv_rope: a slot for every row")
        page_size = int(kv_pages.shape[3])
    _check(lib().qe_linear_qkv_rope_tcgen05_pair(
        _ptr(x), _ptr(w_qkv), _ptr(qkv), M, N, K, _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(cos_sin),
        _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None), Hq, Hkv, page_size,
        int(bool(write_kv)), _stream()), "linear_qkv_rope")


QKV_ROPE_SMALL = False       # a few rows: per-head norm, rotation and cache write in the epilogue of the QKV product (clusters of 8 CTAs per head).  Off: measured on a B200 (0.6B sizes, 8 rows, chains of 28): product + rotary kernel 3.83 us, fused 4.54 us (cluster launch + two cluster barriers cost more than the launch they save); the decode step 0.955 -> 0.978 ms.  Kept as a tested option.
QKV_ROPE_SMALL_MAX_M = 16


def qkv_rope_small_applies(M: int, N: int, K: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether ``linear_qkv_rope_small`` serves this shape: a few rows in bfloat16, head size 128 rotated as a whole."""
    return (QKV_ROPE_SMALL and dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == 128 and K % 8 == 0
            and N % 128 == 0 and 1 <= M <= QKV_ROPE_SMALL_MAX_M)


def linear_qkv_rope_small(x, w_qkv: torch.Tensor, qkv: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                          k_norm_w: Optional[torch.Tensor], eps: float, positions: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                          kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                          num_heads: int, num_kv_heads: int, write_kv: bool = True) -> None:
    """The QKV product of a few rows (decode steps) with what ``qk_norm_rope_kv_write`` would do to it afterwards in
    its epilogue (head size 128, bfloat16): a head's 128 columns are the work of a cluster of 8 CTAs, which exchange
    the sums of squares and the rotation's partners through distributed shared memory.  qkv[:, :Hq 128] = rotated,
    normed q; the rotated, normed k and v go to their slots in ``kv_pages`` [pages, 2, Hkv, page, 128] only.  Angles:
    ``cos_sin`` float32 [M, 64, 2] if given, else ``positions`` x ``inv_freq`` [64] (both None: no rotation)."""
    if isinstance(x, NormedInput):
        x = x.materialize()
    M, K = x.shape
    Hq, Hkv = num_heads, num_kv_heads
    N = (Hq + 2 * Hkv) * 128
    _need(x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and w_qkv.shape == (N, K) and K % 8 == 0,
          "linear_qkv_rope_small: bfloat16 operands, w [(Hq + 2 Hkv) 128, K] with K a multiple of 8")
    _need(qkv.shape == (M, N) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and x.is_contiguous() and w_qkv.is_contiguous()
          and M <= QKV_ROPE_SMALL_MAX_M, f"linear_qkv_rope_small: qkv must be contiguous bfloat16 [M <= {QKV_ROPE_SMALL_MAX_M}, (Hq + 2 Hkv) 128]")
    for wt in (q_norm_w, k_norm_w):
        _need(wt is None or (wt.dtype == torch.float32 and wt.shape == (128,)), "linear_qkv_rope_small: norm weights must be float32 [128]")
    _need(cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (M, 64, 2) and cos_sin.is_contiguous()),
          "linear_qkv_rope_small: cos_sin must be float32 [M, 64, 2]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == 64, "linear_qkv_rope_small: inv_freq must be float32 [64]")
        if cos_sin is None:
            _need(positions is not None and positions.numel() >= M, "linear_qkv_rope_small: a position for every row")
            _i32(positions, "positions")
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None and kv_pages.dtype == torch.bfloat16 and kv_pages.is_contiguous()
              and kv_pages.dim() == 5 and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == 128,
              "linear_qkv_rope_small: kv_pages must be bfloat16 [pages, 2, Hkv, page, 128]")
        _i32(slot_mapping, "slot_mapping")
        _need(slot_mapping.numel() >= M, "linear_qkv_rope_small: a slot for every row")
        page_size = int(kv_pages.shape[3])
    _hand_over_next_weights()
    _check(lib().qe_linear_small_m_qkv_rope(
        _ptr(x), _ptr(w_qkv), _ptr(qkv), M, N, K, _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(positions),
        _ptr(inv_freq), _ptr(cos_sin), _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None),
        Hq, Hkv, page_size, int(bool(write_kv)), _stream()), "linear_qkv_rope_small")


def linear_silu_mul(gate_up: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch) -> None:
    """out[M, N] = (silu(gate_up[:, :I]) * gate_up[:, I:]) · w[N, I]^T.  For a few rows in bfloat16 the
    activation is formed while the product loads it; otherwise ``silu_mul`` runs first into a buffer
    that ``scratch(shape, dtype)`` provides."""
    M, I2 = gate_up.shape
    I = I2 // 2
    N = w.shape[0]
    if M > FUSED_SILU_MAX_M or I > FUSED_SILU_MAX_K or splitk_splits(M, N, I, gate_up.dtype):
        act = scratch((M, I), gate_up.dtype)
        silu_mul(gate_up, act)
        linear(act, w, out)
        return
    if isinstance(out, ResidualSink):
        if _linear_into_stream(gate_up, w, out, silu=True):
            return
        out = out.as_delta()
    _need(I2 % 2 == 0 and w.shape == (N, I) and w.dtype == gate_up.dtype, "linear_silu_mul: w must be [N, I] for gate_up [M, 2I]")
    _need(out.shape == (M, N) and out.dtype in (gate_up.dtype, torch.float32), "linear_silu_mul: out must be [M, N]")
    _need(gate_up.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear_silu_mul: operands must be contiguous")
    if gate_up.dtype == torch.bfloat16 and M <= SMALL_M_MAX and I % 8 == 0:
        _hand_over_next_weights()
        lib().qe_small_m_rows8(int(SMALL_M_ROWS8))
        _check(lib().qe_linear_small_m_silu(_ptr(gate_up), _ptr(w), _ptr(out), M, N, I,
                                            int(out.dtype == torch.float32), _stream()), "linear_silu_mul")
        return
    act = scratch((M, I), gate_up.dtype)
    silu_mul(gate_up, act)
    linear(act, w, out)


def timeline_begin(capacity: int = 1 << 20) -> None:
    """Start recording in the timeline build of the library (QE_TIMELINE=1 in the environment when it is
    built and loaded): from now on thread 0 of every CTA notes the GPU's clock when it lets its dependents
    start and when its wait for the kernel before it returns.  Raises in the plain build."""
    lib().qe_timeline_begin.restype = ctypes.c_long
    got = int(lib().qe_timeline_begin(ctypes.c_long(int(capacity))))
    if got < 0:
        raise ExtensionMissing("this build of the library records no timeline (build and run with QE_TIMELINE=1)"
                               if got == -1 else "no memory for the timeline")


def timeline_events() -> list[tuple[str, int, int, int, int, int, int]]:
    """The events since ``timeline_begin``, in the order of their times: (source file, line, kind, CTA's linear
    index, CTAs of its grid, ns, SM); kind 0: the CTA let its dependents start (about its start), 1: its wait
    for the predecessor returned."""
    cap = 1 << 20
    buf = (ctypes.c_ulonglong * (4 * cap))()
    lib().qe_timeline_read.restype = ctypes.c_long
    n = int(lib().qe_timeline_read(buf, ctypes.c_long(cap)))
    if n < 0:
        raise ExtensionMissing("this build of the library records no timeline (build and run with QE_TIMELINE=1)")

    def fnv(name: str) -> int:
        h = 2166136261
        for ch in name.encode():
            h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
        return h
    names = {fnv(f): f for f in os.listdir(_build.CSRC_DIR) if f.endswith((".cu", ".cuh", ".h"))}
    out = []
    for i in range(n):
        w, c, t, sm = (int(buf[4 * i + j]) for j in range(4))
        out.append((names.get(w >> 32, hex(w >> 32)), (w >> 16) & 0xFFFF, w & 3, c >> 32, c & 0xFFFFFFFF, t, sm))
    out.sort(key=lambda e: e[5])
    return out


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch of the kernels (on by default): a kernel may start, and a
    product may begin to fetch its weights, while the kernel before it is still running."""
    lib().qe_set_pdl(int(bool(enabled)))


def tc_attention_status() -> int:
    """0, or the code of the first wait inside the tcgen05 attention kernel that ran out."""
    return int(lib().qe_flash_attention_tc_status())


def tcgen05_status() -> int:
    """0 if no bounded wait of the tcgen05 product kernels ever ran out; else the code of the first
    that did (1: a shared-memory slot never came free, 2: TMA bytes never landed, 3: the
    accumulator never completed, 4: an accumulator was never read out; 11-13: the same as 1-3 in the
    kernel for some tens of rows, 21-23 in its form that shares K within a cluster).  Synchronises the device."""
    return (int(lib().qe_gemm_tc_status()) or int(lib().qe_gemm_tc_swap_status()) or int(lib().qe_gemm_tc_pair_status())
            or int(lib().qe_gemm_tc_splitk_status()))


class DeviceWaitTimeout(RuntimeError):
    """A bounded wait inside a kernel ran out: the kernel gave up without storing its output, so what
    the step produced is not to be trusted."""


_STATUS_WORDS = ("qe_gemm_tc", "qe_gemm_tc_swap", "qe_gemm_tc_pair", "qe_gemm_tc_splitk", "qe_flash_attention_tc",
                 "qe_flash_attention", "qe_decode_attention_mma", "qe_small_m")


def device_status() -> dict[str, int]:
    """The status words of the kernels whose waits are bounded that are not zero: kernel family -> code
    of its first wait that ran out.  Synchronises the device (one small copy per word)."""
    if _lib is None:
        return {}                   # nothing was ever launched
    out = {}
    for name in _STATUS_WORDS:
        code = int(getattr(lib(), name + "_status")())
        if code:
            out[name[3:]] = code
    return out


def clear_device_status() -> None:
    """Set the status words back to zero, and the counters by which split contexts find their last part
    (a kernel that gave up may have left them counted up)."""
    if _lib is None:
        return
    for name in _STATUS_WORDS:
        getattr(lib(), name + "_clear_status")()
    for t in _merge_counter_tensors.values():
        t.zero_()


def check_device_status() -> None:
    """Raise ``DeviceWaitTimeout`` if any bounded wait ran out since the words were last cleared (and clear
    them).  The engine calls this where it synchronises anyway: at the end of ``serving``."""
    bad = device_status()
    if bad:
        clear_device_status()
        raise DeviceWaitTimeout(
            "a bounded wait inside a kernel ran out and the kernel returned without its output: "
            + ", ".join(f"{k} (code {v})" for k, v in bad.items())
            + "; the tokens of the steps since the last check are not to be trusted")


def selftest_starved_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, limit: int = 10000) -> None:
    """For tests: one CTA of the tcgen05 product kernel whose loads are withheld, with waits of ``limit``
    polls.  It must give up, store nothing into ``out``, free its tensor memory and leave a code in
    ``tcgen05_status()``; the device stays usable."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape == (M, N)
          and x.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "selftest: contiguous bfloat16 operands")
    _check(lib().qe_gemm_tc_selftest_starved(_ptr(x), _ptr(w), _ptr(out), M, N, K, int(limit), _stream()), "selftest")


ROPE_TABLE_MIN_T = 64   # tokens from which a step's rotation angles are computed once (below: in the kernel)


def rope_table_applies(num_tokens: int, dtype: torch.dtype, head_dim: int, rotary_dim: int) -> bool:
    """Whether the kernels that rotate q and k take a table of this step's cosines and sines (``rope_table``)
    instead of computing the angles themselves: many tokens, bfloat16, head size 128 rotated as a whole."""
    return num_tokens >= ROPE_TABLE_MIN_T and dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == head_dim


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = (cos, sin)(positions[t] * inv_freq[j]) in float32; out [T, len(inv_freq), 2]."""
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    _need(out.dtype == torch.float32 and out.shape == (T, half, 2) and out.is_contiguous(), "rope_table: out must be float32 [T, half, 2]")
    _check(lib().qe_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_table")


def qk_norm_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, q_norm_w: Optional[torch.Tensor],
                          k_norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor],
                          rotary_dim: int, kv_pages: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                          num_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool = True,
                          cos_sin: Optional[torch.Tensor] = None) -> None:
    """On the stacked projection output qkv [T, (Hq + 2 Hkv) D], in place: per-head RMS norm of q and
    k (if weights are given), half-split rotation by positions (if inv_freq is given); then k and v
    are written to the slots of ``slot_mapping`` in ``kv_pages`` [pages, 2, Hkv, page, D]."""
    T = qkv.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    _need(qkv.shape == (T, (Hq + 2 * Hkv) * D) and qkv.is_contiguous(), "qk_norm_rope_kv_write: qkv must be [T, (Hq+2Hkv)D]")
    _i32(positions, "positions")
    stride = qkv.shape[1]
    q = qkv
    k = qkv[:, Hq * D:]
    v = qkv[:, (Hq + Hkv) * D:]
    page_size = 1
    if write_kv:
        _need(kv_pages is not None and slot_mapping is not None, "qk_norm_rope_kv_write: cache write without a cache")
        _need(kv_pages.dtype == qkv.dtype and kv_pages.is_contiguous() and kv_pages.dim() == 5
              and kv_pages.shape[1] == 2 and kv_pages.shape[2] == Hkv and kv_pages.shape[4] == D,
              "qk_norm_rope_kv_write: kv_pages must be [pages, 2, Hkv, page, D] in qkv's dtype")
        _i32(slot_mapping, "slot_mapping")
        page_size = kv_pages.shape[3]
    for wt in (q_norm_w, k_norm_w):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.shape == (D,), "qk_norm_rope_kv_write: norm weights must be float32 [D]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2,
              "qk_norm_rope_kv_write: inv_freq must be float32 [rotary_dim / 2]")
    _check(lib().qe_qk_norm_rope_kv_write(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
        ctypes.c_long(stride), ctypes.c_long(stride), ctypes.c_long(stride), _ptr(positions),
        _ptr(q_norm_w), _ptr(k_norm_w), ctypes.c_float(eps), _ptr(inv_freq),
        _ptr(cos_sin if (cos_sin is not None and D == 128 and rotary_dim == D) else None), int(rotary_dim),
        _ptr(kv_pages if write_kv else None), _ptr(slot_mapping if write_kv else None),
        T, Hq, Hkv, D, page_size, int(bool(write_kv)), _dt(qkv), _stream()), "qk_norm_rope_kv_write")


def rope_neox(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
              rotary_dim: int) -> None:
    """Half-split rotation of q [T, Hq, D] and k [T, Hkv, D] in place (rows may be strided)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    _need(q.stride(2) == 1 and q.stride(1) == D and k.stride(2) == 1 and k.stride(1) == D,
          "rope_neox: heads of a token must be contiguous")
    _i32(positions, "positions")
    _check(lib().qe_qk_norm_rope_kv_write(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(0),
        ctypes.c_long(q.stride(0)), ctypes.c_long(k.stride(0)), ctypes.c_long(0), _ptr(positions),
        _ptr(None), _ptr(None), ctypes.c_float(0.0), _ptr(inv_freq), _ptr(None), int(rotary_dim),
        _ptr(None), _ptr(None), T, Hq, Hkv, D, 1, 0, _dt(q), _stream()), "rope_neox")


def flash_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes this geometry (else the generic kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and num_kv_heads >= 1 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= FLASH_ROWS)


def tc_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel takes this geometry (prompt portions; else the mma.sync kernel)."""
    if dtype != torch.bfloat16 or head_dim != 128 or num_kv_heads < 1 or num_heads % num_kv_heads:
        return False
    G = num_heads // num_kv_heads
    return G <= 128 and G & (G - 1) == 0 and page_size >= 8 and page_size & (page_size - 1) == 0


def _plan_tc_tiles(tiles: list, Hkv: int) -> tuple[list[int], int, list[int], int]:
    """Work items of the tcgen05 kernel from its tiles (key steps, first key, last key, item fields),
    sorted by their steps, longest first.  Where the tiles alone would leave SMs idle (a short portion
    behind a long context: few tiles; one prompt of a few thousand tokens: tiles as unequal as
    1 : 2 : ... : n), the longer tiles are cut into parts of whole steps; the library works out the most
    steps an item may have by laying out the candidates' schedules (a part costs its scratch and the
    merge, about as much as a step).  The kernel's CTAs, one per SM at most, run the units (an item for one kv
    head) one after the other; the library deals them out, longest first, each to the CTA with the least work
    so far.  Returns the items, the number of parts, the schedule (the CTAs' offsets into the list itself,
    then their unit numbers) and the number of CTAs."""
    cap = TC_FORCE_CAP
    if cap < 0:
        cap = 0
        if tiles and len(tiles) * Hkv < TC_BALANCE_BELOW_CTAS:
            steps = (ctypes.c_int * len(tiles))(*[t[0] for t in tiles])
            cap = int(lib().qe_flash_attention_tc_balance(steps, len(tiles), Hkv, TC_TARGET_CTAS, TC_MIN_PART_STEPS, TC_MAX_PARTS,
                                                          ctypes.c_float(TC_ITEM_COST_STEPS), ctypes.c_float(TC_PART_COST_STEPS)))
    out: list[tuple[int, list[int]]] = []
    n_parts = 0
    for steps, lo, hi, (r, q0, row0, n, c) in tiles:
        parts = min(TC_MAX_PARTS, -(-steps // cap)) if cap else 1
        if parts <= 1:
            out.append((steps, [r, q0, lo, hi, -1, 0, 0, row0, n, c, 0, 0]))
            continue
        per = -(-steps // parts)
        lo_al = lo // TC_BN * TC_BN
        parts = -(-steps // per)
        for sp in range(parts):
            k0 = lo if sp == 0 else lo_al + sp * per * TC_BN
            k1 = min(hi, lo_al + (sp + 1) * per * TC_BN)
            out.append((min(per, steps - sp * per), [r, q0, k0, k1, n_parts + sp, parts, sp, row0, n, c, 0, 0]))
        n_parts += parts
    out.sort(key=lambda kv: -kv[0])
    n_ctas = min(len(out) * Hkv, TC_TARGET_CTAS)
    costs = (ctypes.c_float * len(out))(*[st + TC_ITEM_COST_STEPS + (TC_PART_COST_STEPS if item[4] >= 0 else 0.0) for st, item in out])
    sched = (ctypes.c_int * (n_ctas + 1 + len(out) * Hkv))()
    n = int(lib().qe_flash_attention_tc_schedule(costs, len(out), Hkv, n_ctas, sched))
    _need(n == len(sched), "plan_attention: the schedule of the tcgen05 kernel could not be made")
    return [x for _, item in out for x in item], n_parts, list(sched), n_ctas


def plan_attention(q_lens: list[int], ctx_lens: list[int], page_size: int,
                   geometries=(), dtype: torch.dtype = torch.float32,
                   uniform_splits: Optional[dict] = None) -> dict[str, list[int]]:
    """Work lists of the attention kernels for one step's batch, as named int32 lists that the
    step function copies to the device with the rest of the step's metadata.

    ``geometries``: the (heads, kv heads, head size, window) of the model's attention layers.
    ``tiles`` serves the generic kernel; for each geometry the flash kernel takes, ``fa<i>_items``
    and ``fa<i>_merge`` hold its work and merge items and ``fa<i>_info`` = [parts, rows per part,
    whether every item has at most 16 rows, the most rows of an item, the number of parts of every
    request if all are cut into the same 2, 4 or 8 parts (they can then form clusters) else 0]; requests that bring many rows go to the tcgen05 kernel
    instead where it takes the geometry: ``tc<i>_items``, ``tc<i>_sched`` (which CTA runs which
    item for which kv head) and ``tc<i>_info`` = [parts, rows per part, CTAs].
    ``uniform_splits`` (geometry -> number of parts) fixes the number of parts of every request,
    so that the lists depend on the batch's shape only (for steps replayed from a CUDA graph)."""
    tiles: list[int] = []
    for r, n in enumerate(q_lens):
        for q0 in range(0, n, ATTN_TILE_Q):
            tiles += [r, q0]
    plan = {"tiles": tiles}
    for gi, geo in enumerate(geometries):
        Hq, Hkv, D, window = geo
        if not flash_supported(dtype, Hq, Hkv, D):
            continue
        G = Hq // Hkv
        tpt = FLASH_ROWS // G
        use_tc = uniform_splits is None and tc_attention_supported(dtype, Hq, Hkv, D, page_size)
        on_tc = [use_tc and n * G >= TC_MIN_ROWS for n in q_lens]
        tc_tiles: list = []
        base = sum(-(-n // tpt) for n, tc in zip(q_lens, on_tc) if not tc) * Hkv
        items: list[int] = []
        merge: list[int] = []
        n_parts, part_rows, row0, max_rows = 0, 1, 0, 0
        whole: list[tuple[int, list[int]]] = []        # (keys the tile visits, its work item)
        for r, (n, c) in enumerate(zip(q_lens, ctx_lens)):
            total = c + n
            if on_tc[r]:
                tc_tpt = TC_ROWS // G
                for q0 in range(0, n, tc_tpt):
                    lo = max(0, c + q0 - window + 1) if window else 0
                    hi = c + min(n, q0 + tc_tpt)
                    tc_tiles.append((-(-(hi - lo // TC_BN * TC_BN) // TC_BN), lo, hi, (r, q0, row0, n, c)))
                row0 += n
                continue
            if uniform_splits is not None:
                splits = uniform_splits[geo]
            else:
                lo = (max(0, c - window + 1) // FLASH_BN) * FLASH_BN if window else 0
                splits = 1
                if n <= tpt and base < FLASH_TARGET_CTAS and total - lo > FLASH_SPLIT:
                    splits = min(-(-(total - lo) // FLASH_SPLIT), max(1, FLASH_TARGET_CTAS // base))
            if splits > 1:
                for sp in range(splits):
                    items += [r, 0, 0, 0, n_parts + sp, splits, sp, row0, n, c, 0, 0]
                merge += [r, 0, n_parts, splits]
                n_parts += splits
                part_rows = max(part_rows, n * G)
            else:
                for q0 in range(0, n, tpt):
                    whole.append((c + min(n, q0 + tpt), [r, q0, 0, total, -1, 0, 0, row0, n, c, 0, 0]))
            row0 += n
            max_rows = max(max_rows, min(n, tpt) * G)
        # tiles that visit many keys start first, so that the last wave of CTAs is made of short ones
        whole.sort(key=lambda kv: -kv[0])
        items = [x for _, item in whole for x in item] + items
        plan[f"fa{gi}_items"] = items
        plan[f"fa{gi}_merge"] = merge
        sizes = {m for m in merge[3::4]}
        same = sizes.pop() if len(sizes) == 1 and not whole else 0
        plan[f"fa{gi}_info"] = [n_parts, part_rows, int(max_rows <= 16), max_rows, same if same in (2, 4, 8) else 0]
        if tc_tiles:
            tc_items, tc_parts, tc_sched, tc_ctas = _plan_tc_tiles(tc_tiles, Hkv)
            plan[f"tc{gi}_items"] = tc_items
            plan[f"tc{gi}_sched"] = tc_sched
            plan[f"tc{gi}_info"] = [tc_parts, TC_ROWS, tc_ctas]
    return plan


DECODE_CLUSTER4_MAX_SPAN = 4096   # keys up to which 4 parts in a cluster are preferred to more parts merged through memory


def decode_splits(num_reqs: int, max_tokens: int, geometries, dtype: torch.dtype) -> dict:
    """The fixed number of parts per request for a decode step of ``num_reqs`` requests whose block
    tables hold up to ``max_tokens`` tokens: enough parts to fill the GPU, none shorter than a split."""
    out = {}
    for geo in geometries:
        Hq, Hkv, D, window = geo
        span = min(max_tokens, window) if window else max_tokens
        target = FLASH_TARGET_CTAS
        if (DECODE_ATTENTION_MMA and DECODE_ATTENTION_MMA_WIDE and dtype == torch.bfloat16 and D == 128
                and Hq // Hkv <= 16 and num_reqs * Hkv <= TC_TARGET_CTAS):
            target = TC_TARGET_CTAS                                       # one CTA of 8 warps per SM
        want = max(1, target // max(1, num_reqs * Hkv))                   # all parts run in one wave
        parts = max(1, min(want, -(-span // FLASH_SPLIT)))
        if target == TC_TARGET_CTAS and DECODE_ATTENTION_CLUSTERS and parts > 2:
            # 2, 4 or 8 parts of a request form a thread-block cluster and meet on chip, which beats the merge through
            # global memory (measured at 0.6B sizes, context 1 024: 2 requests in 4 parts each 0.80 ms a step, in 5
            # parts 0.95); clusters of 8 only while all of them still fit the GPU at once (at most 8 of them: 0.95 ms
            # with 16 of them) or where 4 parts would be long ones
            few = num_reqs * Hkv * 8 <= 64
            if parts == 3:
                parts = 4 if num_reqs * Hkv * 4 <= target else 2
            elif parts < 8:
                parts = 8 if few else 4
            elif few or (parts == 8 and span > DECODE_CLUSTER4_MAX_SPAN):
                parts = 8
            elif span <= DECODE_CLUSTER4_MAX_SPAN:
                parts = 4
        out[geo] = parts
    return out


_MERGE_COUNTERS = 1 << 16
_merge_counter_tensors: dict = {}


def _merge_counters(device, kernel: str = "fa") -> torch.Tensor:
    """Zeroed ints, one per (part, kv head), that an attention kernel uses to find the CTA that finishes a
    split context last (it merges the parts and sets its counter back to zero).  One tensor per device
    and kernel for the life of the process, so that its address is the same in every captured step."""
    key = (torch.device(device).index, kernel)
    t = _merge_counter_tensors.get(key)
    if t is None:
        t = torch.zeros(_MERGE_COUNTERS, dtype=torch.int32, device=device)
        _merge_counter_tensors[key] = t
    return t


def _decode_mma_serves(plan, key, qkv: torch.Tensor, Hq: int, Hkv: int, D: int) -> bool:
    """Whether the step's requests that are not on the tcgen05 kernel (geometry index ``key`` of the plan) go to
    the tensor-core kernel for decoded tokens: items of at most 16 rows, head size 128."""
    if not DECODE_ATTENTION_MMA or key is None or f"fa{key}_items" not in plan or D != 128:
        return False
    if f"tc{key}_items" in plan and not DECODE_ATTENTION_MMA_BESIDE_TC:
        return False
    n_parts, part_rows, small_tiles, max_rows, same_parts = plan[f"fa{key}_info_host"]
    n_items = plan[f"fa{key}_items"].numel() // FLASH_ITEM_INTS
    return (1 <= max_rows <= 16 and Hq // Hkv <= 16 and n_items > 0 and n_items * Hkv >= DECODE_ATTENTION_MMA_MIN_CTAS
            and n_parts * Hkv <= _MERGE_COUNTERS and qkv.stride(0) % 8 == 0)


def paged_attention(qkv: torch.Tensor, kv_pages: torch.Tensor, block_tables: torch.Tensor, ctx,
                    out: torch.Tensor, scale: float, window: int, num_heads: int, num_kv_heads: int,
                    head_dim: int, next_pages: Optional[torch.Tensor] = None) -> None:
    """Attention of the step's queries (the q part of qkv [T, (Hq+2Hkv) D]) over the keys and values
    of their requests in ``kv_pages``; out [T, Hq D].  ``ctx`` is the StepContext (cu_q, ctx_lens,
    the plan that ``plan_attention`` made, and the arena for the parts of split contexts).

    ``next_pages``: the cache of the layer that runs after this one, if it has the same shape (the same
    pages at the same places): a decode step's kernel may ask L2 for that layer's keys and values."""
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    T = qkv.shape[0]
    _need(out.shape == (T, Hq * D) and out.is_contiguous() and out.dtype == qkv.dtype, "paged_attention: out must be [T, Hq D]")
    _need(kv_pages.dtype == qkv.dtype and kv_pages.dim() == 5 and kv_pages.is_contiguous(),
          "paged_attention: kv_pages must be [pages, 2, Hkv, page, D] in q's dtype")
    _i32(block_tables, "block_tables")
    global last_attention_kernel
    plan = ctx.attn_plan
    key = plan.get("geometry_index", {}).get((Hq, Hkv, D, window))
    if key is not None and f"tc{key}_items" in plan:
        last_attention_kernel = "flash_attention_tc"
        tc_items = plan[f"tc{key}_items"]
        tc_parts, tc_rows, tc_ctas = plan[f"tc{key}_info_host"]
        part_acc = part_ml = counters = None
        if tc_parts:
            _need(2 * tc_parts * Hkv <= _MERGE_COUNTERS, "paged_attention: too many parts")   # (two counters a tile and kv head)
            part_acc = ctx.arena.alloc((tc_parts * Hkv * tc_rows, D), torch.float32)
            part_ml = ctx.arena.alloc((tc_parts * Hkv * tc_rows, 2), torch.float32)
            counters = _merge_counters(qkv.device, "tc")
        _check(lib().qe_flash_attention_tc(
            _ptr(qkv), ctypes.c_long(qkv.stride(0)), T, _ptr(kv_pages), int(kv_pages.shape[0]), _ptr(block_tables),
            int(block_tables.shape[1]), _ptr(tc_items), tc_items.numel() // FLASH_ITEM_INTS,
            _ptr(plan[f"tc{key}_sched"]), int(tc_ctas), _ptr(out),
            _ptr(part_acc), _ptr(part_ml), int(tc_rows), _ptr(counters), ctypes.c_float(scale), int(window),
            Hq, Hkv, D, int(kv_pages.shape[3]), _stream()), "flash_attention_tc")
    if key is not None and f"fa{key}_items" in plan:
        items, merge = plan[f"fa{key}_items"], plan[f"fa{key}_merge"]
        n_parts, part_rows, small_tiles, max_rows, same_parts = plan[f"fa{key}_info_host"]
        n_items, n_merge = items.numel() // FLASH_ITEM_INTS, merge.numel() // 4
        if n_items == 0 and f"tc{key}_items" in plan:
            return                      # every request of the step went to the kernel above
        part_acc = part_ml = None
        if n_parts:
            part_acc = ctx.arena.alloc((n_parts * Hkv * part_rows, D), torch.float32)
            part_ml = ctx.arena.alloc((n_parts * Hkv * part_rows, 2), torch.float32)
        counters = _merge_counters(qkv.device) if 0 < n_parts * Hkv <= _MERGE_COUNTERS else None
        # every request in the same few parts: the parts of a request form a cluster and meet on chip
        cluster = int(same_parts) if DECODE_ATTENTION_CLUSTERS and n_items == n_parts else 0
        if _decode_mma_serves(plan, key, qkv, Hq, Hkv, D):
            # decoded tokens: every warp streams key groups of its own through the tensor cores
            last_attention_kernel = "decode_attention_mma"
            lib().qe_decode_attention_mma_stages(int(DECODE_ATTENTION_MMA_STAGES))
            lib().qe_decode_attention_mma_early(int(DECODE_ATTENTION_MMA_EARLY))
            ahead = None
            if (next_pages is not None and DECODE_PREFETCH_KV_MB > 0 and next_pages.shape == kv_pages.shape
                    and next_pages.dtype == kv_pages.dtype and next_pages.is_contiguous()):
                tokens = sum(ctx.ctx_lens_host) + sum(ctx.q_lens_host)
                if tokens * 2 * Hkv * D * kv_pages.element_size() <= DECODE_PREFETCH_KV_MB << 20:
                    ahead = next_pages
            _check(lib().qe_decode_attention_mma(
                _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(ahead), _ptr(block_tables), int(block_tables.shape[1]),
                _ptr(items), n_items, _ptr(out), _ptr(part_acc), _ptr(part_ml), int(part_rows), _ptr(counters),
                int(max_rows), cluster, int(DECODE_ATTENTION_MMA_WIDE and n_items * Hkv <= TC_TARGET_CTAS),
                ctypes.c_float(scale), int(window), Hq, Hkv, D, int(kv_pages.shape[3]), _stream()),
                "decode_attention_mma")
            return
        last_attention_kernel = "flash_attention"
        _check(lib().qe_flash_attention_fused_merge(
            _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(block_tables), int(block_tables.shape[1]),
            _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(items), n_items, _ptr(merge), n_merge, _ptr(out),
            _ptr(part_acc), _ptr(part_ml), int(part_rows), _ptr(counters), int(small_tiles), ctypes.c_float(scale), int(window),
            Hq, Hkv, D, int(kv_pages.shape[3]), _stream()), "flash_attention")
        return
    tiles = plan["tiles"]
    n_tiles = tiles.numel() // 2
    last_attention_kernel = "paged_attention_generic"
    _check(lib().qe_paged_attention_generic(
        _ptr(qkv), ctypes.c_long(qkv.stride(0)), _ptr(kv_pages), _ptr(block_tables), int(block_tables.shape[1]),
        _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), _ptr(tiles), n_tiles, _ptr(out), ctypes.c_float(scale), int(window),
        Hq, Hkv, D, int(kv_pages.shape[3]), _dt(qkv), _stream()), "paged_attention")


def place_tokens(token_ids: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, src_index: torch.Tensor) -> None:
    """token_ids[rows[i]] = src[src_index[i]], all int32 on the device."""
    for t, name in ((token_ids, "token_ids"), (rows, "rows"), (src, "src"), (src_index, "src_index")):
        _i32(t, name)
    _need(rows.numel() == src_index.numel(), "place_tokens: one source index per row")
    _check(lib().qe_place_tokens(_ptr(token_ids), _ptr(rows), _ptr(src), _ptr(src_index), rows.numel(), _stream()),
           "place_tokens")


def copy_pages(cache: torch.Tensor, pairs: torch.Tensor) -> None:
    """cache[s, pairs[2 i + 1]] = cache[s, pairs[2 i]] for every cache slot s of a group's tensor
    [slots, pages, ...] and every pair of the int32 list on the device: whole pages, one launch."""
    _i32(pairs, "pairs")
    _need(cache.dim() >= 3 and cache.is_contiguous(), "copy_pages: cache must be contiguous [slots, pages, ...]")
    _need(pairs.numel() % 2 == 0, "copy_pages: pairs of (source page, destination page)")
    n_slots, n_pages = int(cache.shape[0]), int(cache.shape[1])
    page_bytes = cache[0, 0].numel() * cache.element_size()
    _check(lib().qe_copy_pages(_ptr(cache), n_slots, n_pages, ctypes.c_long(page_bytes), _ptr(pairs), pairs.numel() // 2,
                               _stream()), "copy_pages")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    T, I2 = gate_up.shape
    _need(I2 % 2 == 0 and out.shape == (T, I2 // 2) and out.dtype == gate_up.dtype
          and out.is_contiguous() and gate_up.is_contiguous(), "silu_mul: out must be [T, I] for gate_up [T, 2I]")
    _check(lib().qe_silu_mul(_ptr(gate_up), _ptr(out), T, I2 // 2, _dt(out), _stream()), "silu_mul")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] = index of the largest logit of row n (the lowest index on a tie)."""
    N, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "argmax: logits must be contiguous float32")
    _i32(out, "out")
    _check(lib().qe_argmax(_ptr(logits), _ptr(out), N, V, _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """Row n: temperature 0 -> argmax; else inverse-CDF sampling of softmax(top-k logits / temperature)
    with the uniform number uniform[n] in [0, 1)."""
    N, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(temperature.dtype == torch.float32 and uniform.dtype == torch.float32, "sample: temperature and uniform must be float32")
    _i32(top_k, "top_k")
    _i32(out, "out")
    _check(lib().qe_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(uniform), _ptr(out), N, V, _stream()), "sample")
