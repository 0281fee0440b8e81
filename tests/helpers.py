"""Shared by the tests: the tiny configurations, model folders, tolerances, traces."""
from __future__ import annotations

import random

import torch

import plain_qwen3
from qwen_engine_b200.registry import config_from_dict
from qwen_engine_b200.weights import write_model_folder

# Tiny configurations that differ in every size and option.  tiny-a and tiny-b are the two of
# the benchmark description; tiny-c has a head size that is no power of two and three groups; tiny-d
# has the head size of the real models (128), which the kernels that the benchmark times are made for.
TINY = {
    "tiny-a": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                            tie_word_embeddings=True, max_position_embeddings=512),
                   seed=0, std=0.02, norm_std=0.1, page=4),
    "tiny-b": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=80,
                            num_attention_heads=4, num_key_value_heads=1, head_dim=32,
                            intermediate_size=224, vocab_size=389, rope_parameters={"rope_theta": 1000000.0},
                            rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=640),
                   seed=1, std=0.05, norm_std=0.2, page=8),
    "tiny-c": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=1, hidden_size=72,
                            num_attention_heads=6, num_key_value_heads=2, head_dim=48,
                            intermediate_size=152, vocab_size=301, rope_theta=50000.0, rms_norm_eps=3e-6,
                            tie_word_embeddings=True, max_position_embeddings=1024),
                   seed=7, std=0.08, norm_std=0.3, page=16),
    "tiny-d": dict(cfg=dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=256,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                            intermediate_size=640, vocab_size=997, rope_theta=1000000.0, rms_norm_eps=1e-6,
                            tie_word_embeddings=True, max_position_embeddings=2048),
                   seed=11, std=0.05, norm_std=0.1, page=16),
}


def make_folder(path: str, name: str, store_dtype=torch.bfloat16, **overrides) -> str:
    spec = TINY[name]
    raw = dict(spec["cfg"], **overrides)
    cfg = config_from_dict(raw)
    write_model_folder(cfg, path, spec["seed"], spec["std"], spec["norm_std"], store_dtype)
    return path


_plain_cache: dict = {}


def plain_logits(folder: str, tokens) -> torch.Tensor:
    """float32 logits [T, vocab] of the plain implementation for one whole request."""
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        if folder not in _plain_cache:
            _plain_cache[folder] = plain_qwen3.read_model_folder(folder)
        cfg, w = _plain_cache[folder]
        _plain_cache[key] = plain_qwen3.forward_logits(cfg, w, list(tokens))
    return _plain_cache[key]


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def vocab_of(name: str) -> int:
    return TINY[name]["cfg"]["vocab_size"]


# ---- tolerances ------------------------------------------------------------------------------
# float32: the engine and the plain implementation differ by the order of float32 sums only.
# bfloat16: activations between kernels are rounded to 8 bits of mantissa; the bound is relative
# to the largest logit of the compared rows.  Both are fixed here once and not widened per test.
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}


def assert_close_logits(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float32)
    want = want.to(torch.float32)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: max |diff| {err:.3e} > {TOL[dtype]} * {scale:.3f}"


# ---- replay helpers ----------------------------------------------------------------------------
MIXED_LENS = [40, 64, 23, 90, 128, 17, 55, 64, 101, 33, 128, 72]


def make_replayer(folder, name, dtype, max_tokens, prefix_cache=True, poison=False, device="cuda:0"):
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.trace import TraceReplayer
    page = TINY[name]["page"]
    unit = max(64, page)
    num_pages = -(-max_tokens // unit) * (unit // page)
    loaded = load_model(folder, dtype, device, page, num_pages, 8, enable_prefix_cache=prefix_cache,
                        poison_cache=poison, check_device=(device != "cpu"))
    return TraceReplayer(folder, dtype, max_tokens, page_size=page, loaded=loaded)


def run_steps(rep, steps):
    """Run steps; returns {request id: {position: logits row}}."""
    got: dict = {}
    pos: dict = {}
    for i, st in enumerate(steps):
        st = dict(st, step=i)
        logits = rep.run_step(st)
        row = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[base + w] = logits[row].float().cpu().clone()
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert (logits is None and row == 0) or logits.shape[0] == row
        rep.cache.check_invariants()
    return got


def check_requests(got, folder, requests, dtype, what):
    for rid, toks in requests.items():
        want = plain_logits(folder, toks)
        rows = got[rid]
        idx = sorted(rows)
        assert_close_logits(torch.stack([rows[i] for i in idx]), want[idx], dtype, f"{what} {rid}")



def mixed_steps(reqs, seed, sizes=(2, 3, 5, 8, 13, 21)):
    """Up to four live requests; each step gives some a portion (of one of ``sizes`` tokens), some a
    single token, and leaves some out; a finished request ends and a new one takes its place (and
    its pages)."""
    import random
    rng = random.Random(seed)
    order = list(reqs)
    live, done, pos = [], [], {}
    steps = []
    while len(done) < len(reqs):
        while len(live) < 4 and order:
            rid = order.pop(0)
            live.append(rid)
            pos[rid] = 0
        entries, end = [], []
        for rid in list(live):
            left = len(reqs[rid]) - pos[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue                                   # left out of this step
            mode = rng.random()
            n = 1 if (mode < 0.4 and pos[rid] > 0) else min(left, rng.choice(list(sizes)))
            n = min(n, left)
            want = sorted(rng.sample(range(n), k=min(n, rng.choice([1, 2, n]))))
            entries.append({"id": rid, "tokens": reqs[rid][pos[rid]:pos[rid] + n], "want": want})
            pos[rid] += n
            if pos[rid] == len(reqs[rid]):
                end.append(rid)
                live.remove(rid)
                done.append(rid)
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps




def live_tokens_needed(steps, unit=64) -> int:
    """The most tokens that the live requests of a trace hold at any time, each request's count
    rounded up to ``unit``: the smallest ``max_tokens`` the trace can be replayed with."""
    held, most = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // unit) * unit for n in held.values()))
        for rid in st.get("end", []):
            held.pop(rid, None)
    return most


class LaunchSpy:
    """Counts the calls into the compiled library by entry point while it is active, so that a test
    can say which kernels served it (``with LaunchSpy() as spy: ...; spy.count("qe_...")``)."""

    class _Proxy:
        def __init__(self, real, counts):
            object.__setattr__(self, "_real", real)
            object.__setattr__(self, "_counts", counts)

        def __getattr__(self, name):
            if name.startswith("qe_"):
                self._counts[name] = self._counts.get(name, 0) + 1
            return getattr(self._real, name)

    def __enter__(self):
        from qwen_engine_b200 import ops
        self.counts: dict = {}
        self._ops, self._real = ops, ops.lib()
        ops._lib = LaunchSpy._Proxy(self._real, self.counts)
        return self

    def __exit__(self, *exc):
        self._ops._lib = self._real
        return False

    def count(self, name: str) -> int:
        return self.counts.get(name, 0)


# ---- generation helpers ------------------------------------------------------------------------
def make_engine(folder, name, dtype, device="cuda:0", **engine_kwargs):
    """An LLMEngine over a model folder; on the CPU the caller has put the plain operations in
    the place of the kernels."""
    from qwen_engine_b200.config import EngineConfig
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    kw = dict(dtype=dtype, device=device, block_size=TINY[name]["page"], max_model_len=128, max_num_seqs=4,
              max_num_batched_tokens=64)
    kw.update(engine_kwargs)
    poison = kw.pop("poison_cache", False)
    ec = EngineConfig(**kw)
    loaded = load_model(folder, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(), ec.max_num_seqs,
                        ec.enable_prefix_cache, poison_cache=poison, check_device=(device != "cpu"))
    return LLMEngine(loaded, ec)


def plain_sampled_generate(folder, prompt, steps, temperature, top_k, seed, request_index):
    """Generation by the plain implementation with the engine's sampling rule and the same
    uniform numbers: recompute the whole sequence at every step."""
    import ref_ops
    from qwen_engine_b200.sampling import uniform_for
    tokens, out = list(prompt), []
    for i in range(steps):
        row = plain_logits(folder, tokens)[-1]
        nxt = ref_ops.sample_row(row, temperature, top_k, uniform_for(seed, request_index, i))
        out.append(nxt)
        tokens.append(nxt)
    return out
