"""Plain PyTorch restatements of the engine's operations, one per kernel, with the
same signatures as ``qwen_engine_b200.ops``.

Two uses: the ``-m gpu`` tests compare each CUDA kernel alone with its function
here; and the CPU tests put these functions in the place of the kernels
(``install``), so that the host side of the engine (cache manager, step function,
scheduler, replay) can be checked against the plain model without a GPU.  They
are test code: the product has no CPU path.

Arithmetic is float32 (inputs are converted up, results rounded to the output's
dtype), as in the kernels.
"""
from __future__ import annotations

import torch

ATTN_TILE_Q = 16


def prepare_matrix(w):
    return w.contiguous()


def embedding(token_ids, table, out, ssq=None):
    from qwen_engine_b200.ops import ResidualStream
    if isinstance(out, ResidualStream):
        out.has_delta, out.n_ssq = False, 0
        out = out.resid
    out.copy_(table[token_ids.long()].to(torch.float32))


def _rms(x, weight, eps):
    x = x.to(torch.float32)
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def add_rmsnorm(resid, delta, weight, eps, out):
    if delta is not None:
        resid.add_(delta.to(torch.float32))
    out.copy_(_rms(resid, weight, eps).to(out.dtype))


def add_rmsnorm_rows(resid, delta, rows, weight, eps, out):
    n = out.shape[0]
    idx = rows[:n].long()
    x = resid[idx]
    if delta is not None:
        x = x + delta[idx].to(torch.float32)
    out.copy_(_rms(x, weight, eps).to(out.dtype))


def linear(x, w, out):
    from qwen_engine_b200.ops import NormedInput, ResidualSink
    if isinstance(x, NormedInput):
        x = x.materialize()
    if isinstance(out, ResidualSink):
        out = out.as_delta()
    out.copy_((x.to(torch.float32) @ w.to(torch.float32).t()).to(out.dtype))


def _rotate(x, positions, inv_freq, rotary_dim):
    """x [T, heads, D] float32 -> rotated copy (half-split pairs over the first rotary_dim dims)."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    half = rotary_dim // 2
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    return torch.cat([c * x1 - s * x2, s * x1 + c * x2, x[..., rotary_dim:]], dim=-1)


def place_tokens(token_ids, rows, src, src_index):
    token_ids[rows.long()] = src[src_index.long()]


def swiglu_fused_applies(*args, **kwargs):
    return False


def rope_table(positions, inv_freq, out):
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    out[..., 0], out[..., 1] = torch.cos(ang), torch.sin(ang)


def qk_norm_rope_kv_write(qkv, positions, q_norm_w, k_norm_w, eps, inv_freq, rotary_dim, kv_pages,
                          slot_mapping, num_heads, num_kv_heads, head_dim, write_kv=True, cos_sin=None):
    T = qkv.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    q = qkv[:, :Hq * D].reshape(T, Hq, D).to(torch.float32)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).to(torch.float32)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    if q_norm_w is not None:
        q = _rms(q, q_norm_w, eps)
    if k_norm_w is not None:
        k = _rms(k, k_norm_w, eps)
    if inv_freq is not None:
        q = _rotate(q, positions, inv_freq, rotary_dim)
        k = _rotate(k, positions, inv_freq, rotary_dim)
    qkv[:, :Hq * D] = q.reshape(T, Hq * D).to(qkv.dtype)
    qkv[:, Hq * D:(Hq + Hkv) * D] = k.reshape(T, Hkv * D).to(qkv.dtype)
    if write_kv:
        P = kv_pages.shape[3]
        slots = slot_mapping.long()
        page, off = slots // P, slots % P
        kv_pages[page, 0, :, off, :] = k.to(kv_pages.dtype)
        kv_pages[page, 1, :, off, :] = v.to(kv_pages.dtype)


def rope_neox(q, k, positions, inv_freq, rotary_dim):
    q.copy_(_rotate(q.to(torch.float32), positions, inv_freq, rotary_dim).to(q.dtype))
    k.copy_(_rotate(k.to(torch.float32), positions, inv_freq, rotary_dim).to(k.dtype))


def plan_attention(q_lens, ctx_lens, page_size, geometries=(), dtype=None, uniform_splits=None):
    tiles = []
    for r, n in enumerate(q_lens):
        for q0 in range(0, n, ATTN_TILE_Q):
            tiles += [r, q0]
    return {"tiles": tiles}


def paged_attention(qkv, kv_pages, block_tables, ctx, out, scale, window, num_heads, num_kv_heads, head_dim, next_pages=None):
    """For each request: gather its keys and values from the pages by its block table, then
    softmax(scale q k^T + mask) v with key j allowed for the query at position i iff
    j <= i and (window == 0 or j > i - window)."""
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    P = kv_pages.shape[3]
    cu = ctx.cu_q.tolist()
    ctx_lens = ctx.ctx_lens.tolist()
    group = Hq // Hkv
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        n, c = b - a, ctx_lens[r]
        if n == 0:
            continue
        total = c + n
        q = qkv[a:b, :Hq * D].reshape(n, Hq, D).to(torch.float32)
        kpos = torch.arange(total)
        qpos = c + torch.arange(n)
        allowed = kpos[None, :] <= qpos[:, None]
        if window and window > 0:
            allowed &= kpos[None, :] > qpos[:, None] - window
        needed = allowed.any(dim=0)
        table = block_tables[r].long()
        pages = table[kpos // P]
        assert bool((pages[needed] >= 0).all()), "attention needs a key whose page was given back"
        pages = pages.clamp(min=0)
        k = kv_pages[pages, 0, :, kpos % P, :].to(torch.float32)      # [total, Hkv, D]
        v = kv_pages[pages, 1, :, kpos % P, :].to(torch.float32)
        k = torch.where(needed[:, None, None], k, torch.zeros_like(k))
        v = torch.where(needed[:, None, None], v, torch.zeros_like(v))
        for h in range(Hq):
            s = (q[:, h, :] @ k[:, h // group, :].t()) * scale
            s = s.masked_fill(~allowed, float("-inf"))
            p = torch.softmax(s, dim=-1)
            out[a:b, h * D:(h + 1) * D] = (p @ v[:, h // group, :]).to(out.dtype)


def silu_mul(gate_up, out):
    I = out.shape[1]
    g = gate_up[:, :I].to(torch.float32)
    u = gate_up[:, I:].to(torch.float32)
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def linear_silu_mul(gate_up, w, out, scratch):
    from qwen_engine_b200.ops import ResidualSink
    if isinstance(out, ResidualSink):
        out = out.as_delta()
    act = scratch((gate_up.shape[0], gate_up.shape[1] // 2), gate_up.dtype)
    silu_mul(gate_up, act)
    linear(act, w, out)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def sample_row(row, temperature, top_k, u):
    """One row of the sampling rule: temperature 0 -> argmax (lowest index on a tie); else keep the
    logits >= the top_k-th largest (all when top_k is 0 or >= V), p = exp((logit - max) / temperature)
    in float32, and take the first index whose running sum (float64, index order) exceeds u * total."""
    row = row.to(torch.float32)
    best = int(torch.argmax(row))
    if not temperature > 0:
        return best
    V = row.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(row, top_k).values[-1]
        keep = row >= kth
    p = torch.exp((row - row.max()) / torch.tensor(temperature, dtype=torch.float32))
    p = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
    cum = torch.cumsum(p, dim=0)
    target = float(torch.tensor(u, dtype=torch.float32)) * float(cum[-1])
    hit = torch.nonzero(cum > target)
    return int(hit[0]) if hit.numel() else best


def sample(logits, temperature, top_k, uniform, out):
    for n in range(logits.shape[0]):
        out[n] = sample_row(logits[n].cpu(), float(temperature[n]), int(top_k[n]), float(uniform[n]))


def swiglu_small_applies(M, I, K, dtype):
    return False                 # the host-side tests take the route of separate operations


def qkv_rope_small_applies(M, N, K, dtype, head_dim, rotary_dim):
    return False                 # the host-side tests take the route of separate operations


def copy_pages(cache, pairs):
    """cache [slots, pages, ...]: page pairs[2 i] of every slot is copied to page pairs[2 i + 1]."""
    flat = pairs.tolist()
    for src, dst in zip(flat[0::2], flat[1::2]):
        cache[:, dst] = cache[:, src].clone()


_NAMES = ["copy_pages", "swiglu_small_applies", "qkv_rope_small_applies", "prepare_matrix", "embedding", "add_rmsnorm", "add_rmsnorm_rows", "linear",
          "qk_norm_rope_kv_write", "rope_neox", "rope_table", "place_tokens", "swiglu_fused_applies", "plan_attention", "paged_attention", "silu_mul", "linear_silu_mul",
          "argmax", "sample"]


def install(monkeypatch) -> None:
    """Put these functions in the place of the CUDA fronts for the length of a test."""
    import qwen_engine_b200.ops as ops
    g = globals()
    for name in _NAMES:
        monkeypatch.setattr(ops, name, g[name])
