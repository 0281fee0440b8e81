"""The parts a layer is put together from, each alone against the plain implementation; and that
parts defined outside the package (a mixer with state of its own, another position encoding), a
layer plan that names a layer twice and lets a layer read another layer's cache, and a whole toy
architecture can be registered, built and stepped without a change to the package's files."""
import math
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen3 as plain
from qwen_engine_b200 import ops
from qwen_engine_b200.cache import CacheManager, FixedStateSpec
from qwen_engine_b200.config import ModelConfig
from qwen_engine_b200.engine.runner import ModelRunner, StepEntry
from qwen_engine_b200.models.decoder import DecoderModel, LayerSpec, ModelLayout, PlanEntry
from qwen_engine_b200.parts import (FeedForward, Mixer, PartSpec, PositionEncoding, register, FEED_FORWARDS, MIXERS,
                                    POSITION_ENCODINGS)
from qwen_engine_b200.registry import ARCHITECTURES, build_model, config_from_dict, register_architecture
from qwen_engine_b200.weights import NORM, MATRIX, RandomSource, WeightSpec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _close(got, want, dtype, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all(), what
    assert err <= TOL[dtype] * scale, f"{what}: max |diff| {err:.3e} > {TOL[dtype]} * {scale:.3f}"


class DictSource:
    def __init__(self, tensors):
        self.t = tensors

    def names(self):
        return self.t.keys()

    def shape(self, n):
        return tuple(self.t[n].shape)

    def get(self, n):
        return self.t[n]


def _weights(specs, seed, std=0.1, dtype=torch.bfloat16):
    src = RandomSource(specs, seed, std, 0.2, dtype)
    return {n: src.get(n) for n in src.names()}


def _single_layer_model(block: PartSpec, hidden, vocab=50):
    """A model of one layer around a part, to run the part through the real step function."""
    layout = ModelLayout(vocab_size=vocab, hidden_size=hidden, layers=(LayerSpec(block, "L."),),
                         plan=(PlanEntry(0, 0, True),), final_norm=PartSpec("rmsnorm", dict(width=hidden, eps=1e-6)),
                         tie_head=True)
    return DecoderModel(layout)


# ---- norm -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    H, T = 72, 9
    norm = PartSpec("rmsnorm", dict(width=H, eps=3e-6)).build("norm")
    w = _weights(norm.weight_specs("n."), 1)
    norm.load("n.", DictSource(w), dtype, DEV)
    assert norm.weight.dtype == torch.float32
    g = torch.Generator().manual_seed(2)
    resid = torch.randn(T, H, generator=g)
    delta = torch.randn(T, H, generator=g).to(dtype)
    r = resid.to(DEV)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    norm.add_norm(None, r, delta.to(DEV), out)
    summed = resid + delta.float()
    _close(r, summed, torch.float32, "stream after add")
    _close(out, plain.rmsnorm(summed, w["n.weight"].float(), 3e-6), dtype, "normed")
    rows = torch.tensor([8, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    norm.add_norm_rows(None, r, None, rows, out2)
    _close(out2, plain.rmsnorm(summed[[8, 0]], w["n.weight"].float(), 3e-6), dtype, "rows")


# ---- position encoding ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,theta", [(16, 1e4), (48, 5e4), (128, 1e6)])
def test_rope_part(dtype, D, theta):
    from types import SimpleNamespace
    rope = PartSpec("rope_neox", dict(head_dim=D, theta=theta)).build("position_encoding")
    rope.load("", DictSource({}), dtype, DEV)
    T, Hq, Hkv = 7, 3, 2
    g = torch.Generator().manual_seed(3)
    q = torch.randn(T, Hq, D, generator=g).to(dtype)
    k = torch.randn(T, Hkv, D, generator=g).to(dtype)
    pos = torch.tensor([0, 1, 5, 77, 1000, 4095, 12], dtype=torch.int32)
    qd, kd = q.to(DEV), k.to(DEV)
    rope.rotate(SimpleNamespace(positions=pos.to(DEV)), qd, kd)
    cos, sin = plain.rope_angles(pos, D, theta)
    _close(qd, plain.rope_rotate(q.float(), cos, sin), dtype, "q")
    _close(kd, plain.rope_rotate(k.float(), cos, sin), dtype, "k")


# ---- mixer, feed-forward and block, through a one-layer model and the real cache ----------------------------
def _run_whole_and_cut(model, tensors, dtype, tokens, page=4):
    model.load_weights(DictSource(tensors), dtype, DEV)
    cm = CacheManager(model.cache_specs(), page, 64, 4, dtype, DEV)
    runner = ModelRunner(model, cm, DEV, dtype)
    rc = cm.open("whole")
    whole = runner.step([StepEntry(rc, tokens, list(range(len(tokens))))]).float().cpu().clone()
    cm.close(rc)
    rc = cm.open("cut")
    rows, p = [], 0
    for n in [3, 2, 5, 1, 1, 2] + [1] * 40:
        if p >= len(tokens):
            break
        n = min(n, len(tokens) - p)
        rows.append(runner.step([StepEntry(rc, tokens[p:p + n], list(range(n)))]).float().cpu().clone())
        p += n
    cm.close(rc)
    return whole, torch.cat(rows)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_mlp_and_block_parts(dtype):
    """One pre-norm block of attention and SwiGLU with odd sizes, against the plain layer."""
    H, Hq, Hkv, D, I, V = 72, 6, 2, 48, 152, 50
    rope = PartSpec("rope_neox", dict(head_dim=D, theta=5e4))
    block = PartSpec("pre_norm", dict(
        hidden_size=H, norm=PartSpec("rmsnorm", dict(width=H, eps=1e-5)),
        mixer=PartSpec("gqa_attention", dict(hidden_size=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                             scale=1 / math.sqrt(D), qk_norm_eps=1e-5, position_encoding=rope)),
        feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I))))
    model = _single_layer_model(block, H, V)
    tensors = _weights(model.weight_manifest(), 4)
    tokens = [(5 * i + 3) % V for i in range(23)]
    whole, cut = _run_whole_and_cut(model, tensors, dtype, tokens)
    # the plain layer, with the same tensors under the plain implementation's names
    w = {n.replace("L.", "model.layers.0."): t.float() for n, t in tensors.items()}
    n = dict(layers=1, hidden=H, heads=Hq, kv_heads=Hkv, head_dim=D, inter=I, vocab=V, theta=5e4, eps=1e-5,
             tied=True, scale=1 / math.sqrt(D))
    ids = torch.tensor(tokens)
    x = plain.embedding(ids, w["model.embed_tokens.weight"])
    x = plain.decoder_layer(x, torch.arange(len(tokens)), w, 0, n)
    want = plain.linear(plain.rmsnorm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"])
    _close(whole, want, dtype, "whole")
    _close(cut, want, dtype, "cut into portions")
    # the parts alone: attention and feed-forward outputs of the first branch
    blk = model.blocks[0]
    assert blk.mixer.cache_spec().num_kv_heads == Hkv and blk.mixer.attention_geometry() == (Hq, Hkv, D, 0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part_alone(dtype):
    from types import SimpleNamespace
    from qwen_engine_b200.parts import Arena
    H, I, T = 40, 56, 13
    ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I)).build("feed_forward")
    w = _weights(ffn.weight_specs("m."), 5)
    ffn.load("m.", DictSource(w), dtype, DEV)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(6)).to(dtype)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ffn.forward(SimpleNamespace(num_tokens=T, dtype=dtype, arena=Arena(DEV)), x.to(DEV), out)
    _close(out, plain.mlp_part(x.float(), {k: v.float() for k, v in w.items()}, "m."), dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_alone(dtype):
    """The attention mixer alone (the feed-forward's output projection is zero), cut into steps."""
    H, Hq, Hkv, D, V = 48, 4, 1, 32, 30
    block = PartSpec("pre_norm", dict(
        hidden_size=H, norm=PartSpec("rmsnorm", dict(width=H, eps=1e-6)),
        mixer=PartSpec("gqa_attention", dict(hidden_size=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                             scale=1 / math.sqrt(D), qk_norm_eps=1e-6,
                                             position_encoding=PartSpec("rope_neox", dict(head_dim=D, theta=1e6)))),
        feed_forward=PartSpec("swiglu", dict(hidden_size=H, intermediate_size=16))))
    model = _single_layer_model(block, H, V)
    tensors = _weights(model.weight_manifest(), 8)
    tensors["L.mlp.down_proj.weight"] = torch.zeros_like(tensors["L.mlp.down_proj.weight"])
    tokens = [(11 * i + 1) % V for i in range(17)]
    whole, cut = _run_whole_and_cut(model, tensors, dtype, tokens, page=8)
    w = {n.replace("L.", "model.layers.0."): t.float() for n, t in tensors.items()}
    n = dict(heads=Hq, kv_heads=Hkv, head_dim=D, theta=1e6, eps=1e-6, scale=1 / math.sqrt(D))
    x = plain.embedding(torch.tensor(tokens), w["model.embed_tokens.weight"])
    h = plain.rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
    x = x + plain.attention_part(h, torch.arange(len(tokens)), w, "model.layers.0.self_attn.", n)
    want = plain.linear(plain.rmsnorm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"])
    _close(whole, want, dtype, "attention whole")
    _close(cut, want, dtype, "attention cut")


# ---- parts defined here, outside the package ----------------------------------------------------------------
class DecayMixer(Mixer):
    """A toy mixer with state of fixed size: s <- a * s + x_t for each token of a request in order,
    y_t = s * w.  The state of a request lives in its slot between steps."""

    capturable = False      # it reads step data on the host: its steps are not for CUDA graphs

    def __init__(self, hidden_size: int, decay: float):
        self.hidden_size, self.decay = hidden_size, decay
        self.w = None

    def cache_spec(self):
        return FixedStateSpec((self.hidden_size,), torch.float32)

    def weight_specs(self, prefix):
        return [WeightSpec(prefix + "gain", (self.hidden_size,), NORM)]

    def load(self, prefix, source, dtype, device):
        self.w = source.get(prefix + "gain").float().to(device)

    def forward(self, ctx, x, cache, group, out, write_cache=True):
        # cache: [state slots, hidden] float32 of this layer; plain torch operations are fine in a test
        slots = ctx.slot_ids.tolist()
        cu = ctx.cu_q.tolist()
        for r, slot in enumerate(slots):
            s = cache[slot]
            for t in range(cu[r], cu[r + 1]):
                s = self.decay * s + x[t].float()
                out[t] = (s * self.w).to(out.dtype)
            cache[slot] = s


class RoutedFFN(FeedForward):
    """A toy feed-forward with routing: router logits and their softmax in float32, every token goes
    to the expert with the largest probability (a SwiGLU of its own) and its output is scaled by that
    probability.  The experts' products run through the engine's kernels on the gathered rows."""

    capturable = False      # the rows of an expert are counted on the host

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int):
        self.H, self.I, self.E = hidden_size, intermediate_size, num_experts
        self.router = None
        self.w_gu, self.w_d = [], []

    def weight_specs(self, prefix):
        specs = [WeightSpec(prefix + "router.weight", (self.E, self.H), NORM)]
        for e in range(self.E):
            specs += [WeightSpec(prefix + f"experts.{e}.gate_proj.weight", (self.I, self.H), MATRIX),
                      WeightSpec(prefix + f"experts.{e}.up_proj.weight", (self.I, self.H), MATRIX),
                      WeightSpec(prefix + f"experts.{e}.down_proj.weight", (self.H, self.I), MATRIX)]
        return specs

    def load(self, prefix, source, dtype, device):
        self.router = source.get(prefix + "router.weight").float().to(device)
        for e in range(self.E):
            g, u = (source.get(prefix + f"experts.{e}.{n}_proj.weight") for n in ("gate", "up"))
            self.w_gu.append(ops.prepare_matrix(torch.cat([g, u], dim=0).to(dtype).to(device)))
            self.w_d.append(ops.prepare_matrix(source.get(prefix + f"experts.{e}.down_proj.weight").to(dtype).to(device)))

    def forward(self, ctx, x, out):
        probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
        top_p, top_e = probs.max(dim=-1)
        for e in range(self.E):
            rows = (top_e == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows].contiguous()
            gu = torch.empty(rows.numel(), 2 * self.I, dtype=x.dtype, device=x.device)
            ops.linear(xe, self.w_gu[e], gu)
            act = torch.empty(rows.numel(), self.I, dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act)
            oe = torch.empty(rows.numel(), self.H, dtype=x.dtype, device=x.device)
            ops.linear(act, self.w_d[e], oe)
            out[rows] = (oe.float() * top_p[rows, None]).to(out.dtype)


class ShiftedRope(PositionEncoding):
    """Another position encoding: interleaved pairs (2j, 2j+1) instead of half-split ones."""

    def __init__(self, head_dim: int, theta: float):
        self.head_dim, self.theta = head_dim, theta

    def rotate(self, ctx, q, k):
        D = self.head_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=q.device) / D))
        ang = ctx.positions.float()[:, None] * inv[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for x in (q, k):
            xf = x.float().clone()
            a, b = xf[..., 0::2], xf[..., 1::2]
            x[..., 0::2] = (c * a - s * b).to(x.dtype)
            x[..., 1::2] = (s * a + c * b).to(x.dtype)


@dataclass
class ToyConfig(ModelConfig):
    architecture: ClassVar[str] = "ToyForCausalLM"
    hidden_size: int = 40
    vocab_size: int = 61
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    intermediate_size: int = 56
    decay: float = 0.7
    num_experts: int = 3
    expert_size: int = 24

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k != "architectures"})

    def validate(self):
        pass


def toy_layout(cfg: ToyConfig) -> ModelLayout:
    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", dict(width=H, eps=1e-5))
    ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size))
    attn = lambda pos: PartSpec("gqa_attention", dict(
        hidden_size=H, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
        scale=cfg.head_dim ** -0.5, qk_norm_eps=1e-5, position_encoding=pos))
    rope = PartSpec("rope_neox", dict(head_dim=cfg.head_dim, theta=1e4))
    other = PartSpec("test_interleaved_rope", dict(head_dim=cfg.head_dim, theta=1e4))
    block = lambda mixer, ff=ffn: PartSpec("pre_norm", dict(hidden_size=H, mixer=mixer, feed_forward=ff, norm=norm))
    routed = PartSpec("test_routed", dict(hidden_size=H, intermediate_size=cfg.expert_size, num_experts=cfg.num_experts))
    layers = (LayerSpec(block(attn(rope)), "layers.0."),
              LayerSpec(block(PartSpec("test_decay", dict(hidden_size=H, decay=cfg.decay)), routed), "layers.1."),
              LayerSpec(block(attn(other)), "layers.2."))
    # layer 0 runs twice (a cache slot for each run); layer 2 runs once with a cache of its own and
    # once more reading what layer 0's first run wrote (same cache description, so the same group)
    plan = (PlanEntry(0, 0, True), PlanEntry(1, 1, True), PlanEntry(0, 2, True), PlanEntry(2, 3, True),
            PlanEntry(2, 0, False))
    return ModelLayout(vocab_size=cfg.vocab_size, hidden_size=H, layers=layers, plan=plan, final_norm=norm,
                       embed_name="embed.weight", final_norm_prefix="norm.", head_name="head.weight", tie_head=False)


def _toy_plain(cfg: ToyConfig, w, tokens):
    """The toy model on whole sequences, from the plain implementation's functions."""
    T, H, D = len(tokens), cfg.hidden_size, cfg.head_dim
    pos = torch.arange(T)
    x = plain.embedding(torch.tensor(tokens), w["embed.weight"])

    def qkv(h, p):
        q = plain.rmsnorm(plain.linear(h, w[p + "q_proj.weight"]).view(T, cfg.num_heads, D), w[p + "q_norm.weight"], 1e-5)
        k = plain.rmsnorm(plain.linear(h, w[p + "k_proj.weight"]).view(T, cfg.num_kv_heads, D), w[p + "k_norm.weight"], 1e-5)
        v = plain.linear(h, w[p + "v_proj.weight"]).view(T, cfg.num_kv_heads, D)
        return q, k, v

    def interleaved(t):
        inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        ang = pos.float()[:, None] * inv[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = t[..., 0::2], t[..., 1::2]
        out = torch.empty_like(t)
        out[..., 0::2], out[..., 1::2] = c * a - s * b, s * a + c * b
        return out

    def attn_block(x, i, kind, kv=None):
        p = f"layers.{i}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
        q, k, v = qkv(h, p + "self_attn.")
        if kind == "neox":
            cos, sin = plain.rope_angles(pos, D, 1e4)
            q, k = plain.rope_rotate(q, cos, sin), plain.rope_rotate(k, cos, sin)
        else:
            q, k = interleaved(q), interleaved(k)
        keep = (k, v)
        if kv is not None:
            k, v = kv
        o = plain.causal_attention(q, k, v, D ** -0.5).reshape(T, -1)
        x = x + plain.linear(o, w[p + "self_attn.o_proj.weight"])
        h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        return x + plain.mlp_part(h, w, p + "mlp."), keep

    x, kv0 = attn_block(x, 0, "neox")
    p = "layers.1."
    h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
    s, ys = torch.zeros(H), []
    for t in range(T):
        s = cfg.decay * s + h[t]
        ys.append(s * w[p + "self_attn.gain"])
    x = x + torch.stack(ys)
    h = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
    probs = torch.softmax(h @ w[p + "mlp.router.weight"].t(), dim=-1)
    top_p, top_e = probs.max(dim=-1)
    routed = torch.stack([top_p[t] * plain.mlp_part(h[t:t + 1], w, p + f"mlp.experts.{int(top_e[t])}.")[0] for t in range(T)])
    assert len(set(top_e.tolist())) > 1, "the tokens must not all go to one expert"
    x = x + routed
    x, _ = attn_block(x, 0, "neox")
    x, _ = attn_block(x, 2, "interleaved")
    x, _ = attn_block(x, 2, "interleaved", kv=kv0)
    return plain.linear(plain.rmsnorm(x, w["norm.weight"], 1e-5), w["head.weight"])


@pytest.fixture
def toy_registered():
    register("mixer", "test_decay")(DecayMixer)
    register("position_encoding", "test_interleaved_rope")(ShiftedRope)
    register("feed_forward", "test_routed")(RoutedFFN)
    register_architecture("ToyForCausalLM", ToyConfig, toy_layout)
    yield
    del MIXERS["test_decay"], POSITION_ENCODINGS["test_interleaved_rope"], FEED_FORWARDS["test_routed"]
    del ARCHITECTURES["ToyForCausalLM"]


def test_toy_architecture_with_its_own_parts(toy_registered):
    """Registered from outside (a mixer with state of its own, a feed-forward with routing, another
    position encoding): built by the registry, loaded by the loader's checks, given cache groups of
    its own (pages for attention, state slots for the toy mixer) and stepped by the engine's step
    function, whole and in portions mixed with another request."""
    dtype = torch.float32
    cfg = config_from_dict({"architectures": ["ToyForCausalLM"], "hidden_size": 40, "decay": 0.6})
    assert isinstance(cfg, ToyConfig)
    model = build_model(cfg)
    tensors = _weights(model.weight_manifest(), 9, dtype=torch.float32)
    model.load_weights(DictSource(tensors), dtype, DEV)
    specs = model.cache_specs()
    assert len(specs) == 4 and isinstance(specs[1], FixedStateSpec)
    cm = CacheManager(specs, 4, 48, 3, dtype, DEV)
    assert [g.cache_slots for g in cm.groups] == [[0, 2, 3], [1]] and not cm.prefix_cache
    runner = ModelRunner(model, cm, DEV, dtype)
    w = {n: t.float() for n, t in tensors.items()}
    a = [(3 * i + 1) % cfg.vocab_size for i in range(19)]
    b = [(7 * i + 2) % cfg.vocab_size for i in range(11)]
    want_a, want_b = _toy_plain(cfg, w, a), _toy_plain(cfg, w, b)
    rc = cm.open("whole")
    got = runner.step([StepEntry(rc, a, list(range(len(a))))]).float().cpu().clone()
    cm.close(rc)
    _close(got, want_a, dtype, "toy whole")
    ra, rb = cm.open("a"), cm.open("b")
    pa = pb = 0
    rows_a, rows_b = [], []
    for na, nb in [(4, 2), (1, 3), (6, 1), (1, 1), (2, 4), (5, 0)]:
        na, nb = min(na, len(a) - pa), min(nb, len(b) - pb)
        entries = []
        if na:
            entries.append(StepEntry(ra, a[pa:pa + na], list(range(na))))
        if nb:
            entries.append(StepEntry(rb, b[pb:pb + nb], list(range(nb))))
        out = runner.step(entries).float().cpu().clone()
        rows_a.append(out[:na])
        rows_b.append(out[na:na + nb])
        pa, pb = pa + na, pb + nb
    assert pa == len(a) and pb == len(b)
    _close(torch.cat(rows_a), want_a, dtype, "toy a in portions")
    _close(torch.cat(rows_b), want_b, dtype, "toy b in portions")
    # the slot of an ended request is zeroed for the next one
    cm.close(ra)
    rc = cm.open("again")
    assert rc.state_slot == ra.state_slot
    got = runner.step([StepEntry(rc, a, list(range(len(a))))]).float().cpu().clone()
    _close(got, want_a, dtype, "toy reuse of a state slot")
    cm.check_invariants()


def test_plan_is_checked():
    H = 32
    norm = PartSpec("rmsnorm", dict(width=H, eps=1e-5))
    ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=48))
    attn = PartSpec("gqa_attention", dict(hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=16, scale=0.25))
    block = PartSpec("pre_norm", dict(hidden_size=H, mixer=attn, feed_forward=ffn, norm=norm))
    base = dict(vocab_size=10, hidden_size=H, layers=(LayerSpec(block, "l0."),), final_norm=norm)
    with pytest.raises(ValueError, match="exactly one"):
        DecoderModel(ModelLayout(plan=(PlanEntry(0, 0, True), PlanEntry(0, 0, True)), **base))
    with pytest.raises(ValueError, match="exactly one"):
        DecoderModel(ModelLayout(plan=(PlanEntry(0, 0, False),), **base))
    with pytest.raises(ValueError, match="names layer"):
        DecoderModel(ModelLayout(plan=(PlanEntry(3, 0, True),), **base))
    with pytest.raises(ValueError, match="unknown mixer"):
        PartSpec("no_such_mixer").build("mixer")


# ---- a windowed attention layer through the engine: pages behind the window go back while it runs -----------
@dataclass
class WindowToyConfig(ModelConfig):
    architecture: ClassVar[str] = "WindowToyForCausalLM"
    hidden_size: int = 48
    vocab_size: int = 53
    window: int = 11

    @classmethod
    def from_dict(cls, raw):
        return cls(**{k: v for k, v in raw.items() if k != "architectures"})

    def validate(self):
        pass


def window_toy_layout(cfg: WindowToyConfig) -> ModelLayout:
    H, D = cfg.hidden_size, 16
    norm = PartSpec("rmsnorm", dict(width=H, eps=1e-5))
    ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=64))
    rope = PartSpec("rope_neox", dict(head_dim=D, theta=1e4))
    attn = lambda window: PartSpec("gqa_attention", dict(hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=D, scale=D ** -0.5,
                                                         qk_norm_eps=1e-5, position_encoding=rope, window=window))
    block = lambda w: PartSpec("pre_norm", dict(hidden_size=H, mixer=attn(w), feed_forward=ffn, norm=norm))
    # one layer that sees every earlier token, one that sees a window of them: two cache groups
    return ModelLayout(vocab_size=cfg.vocab_size, hidden_size=H,
                       layers=(LayerSpec(block(None), "layers.0."), LayerSpec(block(cfg.window), "layers.1.")),
                       plan=(PlanEntry(0, 0, True), PlanEntry(1, 1, True)), final_norm=norm,
                       embed_name="embed.weight", final_norm_prefix="norm.", tie_head=True)


def _window_toy_plain(cfg, w, tokens):
    T, D = len(tokens), 16
    pos = torch.arange(T)
    x = plain.embedding(torch.tensor(tokens), w["embed.weight"])
    for i, window in ((0, None), (1, cfg.window)):
        p = f"layers.{i}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
        q = plain.rmsnorm(plain.linear(h, w[p + "self_attn.q_proj.weight"]).view(T, 4, D), w[p + "self_attn.q_norm.weight"], 1e-5)
        k = plain.rmsnorm(plain.linear(h, w[p + "self_attn.k_proj.weight"]).view(T, 2, D), w[p + "self_attn.k_norm.weight"], 1e-5)
        v = plain.linear(h, w[p + "self_attn.v_proj.weight"]).view(T, 2, D)
        cos, sin = plain.rope_angles(pos, D, 1e4)
        o = plain.causal_attention(plain.rope_rotate(q, cos, sin), plain.rope_rotate(k, cos, sin), v, D ** -0.5, window)
        x = x + plain.linear(o.reshape(T, -1), w[p + "self_attn.o_proj.weight"])
        x = x + plain.mlp_part(plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5), w, p + "mlp.")
    return plain.linear(plain.rmsnorm(x, w["norm.weight"], 1e-5), w["embed.weight"])


@pytest.mark.parametrize("dtype", DTYPES)
def test_windowed_layer_gives_pages_back_and_still_agrees(dtype):
    """A layer with a window of 11 keys beside a layer that keeps all keys: the windowed group's pages
    are handed back while the request runs (its page count stays bounded over 150 tokens), entries of
    its block table become -1, and the logits still equal the plain implementation's, through
    portions and single tokens.  The window's edge falls inside pages (page size 4)."""
    register_architecture("WindowToyForCausalLM", WindowToyConfig, window_toy_layout)
    try:
        cfg = config_from_dict({"architectures": ["WindowToyForCausalLM"], "window": 11})
        model = build_model(cfg)
        tensors = _weights(model.weight_manifest(), 21)
        model.load_weights(DictSource(tensors), dtype, DEV)
        cm = CacheManager(model.cache_specs(), 4, 48, 2, dtype, DEV, poison=True)
        assert [g.spec.window for g in cm.groups] == [None, 11] and cm.prefix_cache
        runner = ModelRunner(model, cm, DEV, dtype)
        tokens = [(13 * i + 5) % cfg.vocab_size for i in range(150)]
        want = _window_toy_plain(cfg, {n: t.float() for n, t in tensors.items()}, tokens)
        rc = cm.open("r")
        rows, p = [], 0
        for n in [9, 3, 14, 2, 1, 1, 30, 1, 1, 1, 5] + [1] * 90:
            n = min(n, len(tokens) - p)
            if n == 0:
                break
            rows.append(runner.step([StepEntry(rc, tokens[p:p + n], list(range(n)))]).float().cpu().clone())
            p += n
            held = sum(pg >= 0 for pg in rc.tables[1])
            assert held <= -(-(11 + n) // 4) + 1, "the windowed group holds more pages than its window needs"
            cm.check_invariants()
        assert p == len(tokens) and rc.tables[1][0] == -1 and all(pg >= 0 for pg in rc.tables[0])
        _close(torch.cat(rows), want, dtype, "windowed layer")
        # a second request with the same first 40 tokens shares them: every page in the group that keeps all keys, and
        # in the windowed group the pages its window still reaches (the first request gave them back long ago; they
        # are found again because nobody has taken them since)
        other = tokens[:40] + [(7 * i + 3) % cfg.vocab_size for i in range(30)]
        want2 = _window_toy_plain(cfg, {n: t.float() for n, t in tensors.items()}, other)
        rc2 = cm.open("s", known_tokens=other, max_shared_tokens=len(other) - 1)
        assert rc2.shared_tokens == 40 and rc2.tables[0] == rc.tables[0][:10]
        assert rc2.tables[1][:7] == [-1] * 7 and all(pg >= 0 for pg in rc2.tables[1][7:])
        rows, p = [], 40
        for n in [5, 1, 1, 23]:
            rows.append(runner.step([StepEntry(rc2, other[p:p + n], list(range(n)))]).float().cpu().clone())
            p += n
            cm.check_invariants()
        _close(torch.cat(rows), want2[40:], dtype, "windowed layer, shared prefix")
        cm.close(rc)
        cm.close(rc2)
        assert cm.pages_in_use() == 0
    finally:
        del ARCHITECTURES["WindowToyForCausalLM"]


# ---- the real layer sizes of the benchmark models, few layers, against the plain implementation -----------------
REAL_SIZES = {
    "qwen3-0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072),
    "qwen3-1.7b": dict(hidden_size=2048, num_attention_heads=16, num_key_value_heads=8, intermediate_size=6144),
    # groups of 4 query heads; an intermediate size above what the product that forms SiLU-mul itself takes
    "qwen3-4b": dict(hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, intermediate_size=9728),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", list(REAL_SIZES))
def test_real_layer_sizes(dtype, sizes, tmp_path):
    """Two layers with the widths of Qwen3-0.6B, 1.7B and 4B (head size 128) and a cut vocabulary: the
    kernels at the sizes they are tuned for, inside the model, through a whole prompt, portions, decoded
    tokens, and steps that mix portions of two requests with decoded tokens of two others."""
    import helpers
    from qwen_engine_b200.weights import write_model_folder
    raw = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, head_dim=128, vocab_size=2048, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096, **REAL_SIZES[sizes])
    folder = write_model_folder(config_from_dict(raw), str(tmp_path / "m"), seed=2, std=0.02, norm_std=0.1)
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    loaded = load_model(folder, dtype, DEV, 16, 64, 4, poison_cache=(3.0e4 if dtype == torch.bfloat16 else True))
    rep = TraceReplayer(folder, dtype, 1024, page_size=16, loaded=loaded)
    reqs = {"a": helpers.random_tokens(2048, 200, 31), "b": helpers.random_tokens(2048, 150, 32),
            "c": helpers.random_tokens(2048, 60, 33), "d": helpers.random_tokens(2048, 45, 34)}
    a, b, c, d = (reqs[k] for k in "abcd")
    steps = [{"entries": [{"id": "a", "tokens": a[:130], "want": [0, 64, 129]}]},
             {"entries": [{"id": "a", "tokens": a[130:170], "want": list(range(40))}]}]
    steps += [{"entries": [{"id": "a", "tokens": [t], "want": [0]}]} for t in a[170:180]]
    # mixed: a and c decode, b and d bring portions (b's long enough for the attention kernel of prompt portions)
    steps += [{"entries": [{"id": "c", "tokens": c[:50], "want": [49]}]},
              {"entries": [{"id": "a", "tokens": a[180:181], "want": [0]}, {"id": "b", "tokens": b[:100], "want": [0, 99]},
                           {"id": "c", "tokens": c[50:51], "want": [0]}, {"id": "d", "tokens": d[:21], "want": [20]}]},
              {"entries": [{"id": "a", "tokens": a[181:182], "want": [0]}, {"id": "b", "tokens": b[100:], "want": [0, 49]},
                           {"id": "c", "tokens": c[51:52], "want": [0]}, {"id": "d", "tokens": d[21:], "want": [0, 23]}]}]
    # all four decode (some tens of rows would need more requests; four rows here), then the rest of a and c
    steps += [{"entries": [{"id": "a", "tokens": [a[182 + i]], "want": [0]}, {"id": "c", "tokens": [c[52 + i]], "want": [0]}]}
              for i in range(8)]
    steps += [{"entries": [{"id": "a", "tokens": a[190:], "want": [9]}]}]
    got = helpers.run_steps(rep, steps)
    helpers.check_requests(got, folder, reqs, dtype, f"real layer sizes {sizes}")
    if dtype == torch.bfloat16:
        assert ops.tcgen05_status() == 0 and ops.tc_attention_status() == 0


@pytest.mark.parametrize("sizes", ["qwen3-1.7b", "qwen3-4b"])
def test_real_layer_sizes_some_tens_of_rows(sizes, tmp_path):
    """Decode steps of 24 and 40 requests at the widths of Qwen3-1.7B and 4B in bfloat16: the products for some
    tens of rows (weights on the wide side of the tensor-core instruction, K shared within a cluster where weight
    rows are few) and the attention kernel for decoded tokens with groups of 2 and 4 query heads."""
    import helpers
    from qwen_engine_b200.weights import write_model_folder
    raw = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, head_dim=128, vocab_size=2048, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096, **REAL_SIZES[sizes])
    folder = write_model_folder(config_from_dict(raw), str(tmp_path / "m"), seed=3, std=0.02, norm_std=0.1)
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    n_req = 40
    loaded = load_model(folder, torch.bfloat16, DEV, 16, n_req * 4, n_req, poison_cache=3.0e4)
    rep = TraceReplayer(folder, torch.bfloat16, n_req * 64, page_size=16, loaded=loaded)
    reqs = {f"r{i}": helpers.random_tokens(2048, 20 + (7 * i) % 30, 50 + i) for i in range(n_req)}
    items = list(reqs.items())
    steps = [{"entries": [{"id": rid, "tokens": t[:-2], "want": []} for rid, t in items[k:k + 8]]} for k in range(0, n_req, 8)]
    steps.append({"entries": [{"id": rid, "tokens": [t[-2]], "want": [0]} for rid, t in items[:24]]})              # 24 rows
    steps.append({"entries": [{"id": rid, "tokens": [t[-1] if i < 24 else t[-2]], "want": [0]}
                              for i, (rid, t) in enumerate(items)]})                                              # 40 rows
    steps.append({"entries": [{"id": rid, "tokens": [t[-1]], "want": [0]} for rid, t in items[24:]]})              # 16 rows
    with helpers.LaunchSpy() as spy:
        got = helpers.run_steps(rep, steps)
    assert spy.count("qe_linear_tcgen05_swap") > 0 and spy.count("qe_linear_tcgen05_splitk") > 0, sorted(spy.counts)
    assert spy.count("qe_decode_attention_mma") > 0
    assert all(sorted(got[rid]) == [len(t) - 2, len(t) - 1] for rid, t in items)
    helpers.check_requests(got, folder, reqs, torch.bfloat16, f"some tens of rows {sizes}")
    assert ops.tcgen05_status() == 0
