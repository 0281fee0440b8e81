"""Benchmark of the engine on one B200: decode tokens a second at a fixed batch and context,
prefill tokens a second at 2,048 tokens, for Qwen3-0.6B-shaped random weights.

    python bench.py --gpus 1 --steps K --warmup W        # prints ONE JSON line

A step is one decode step of the whole batch.  ``value`` is timed on the device over the step
function (tokens already on the host side of the step function, no sampling read-back);
``e2e`` is the same through the Python entry point (LLMEngine.step: host tokens in, sampled
tokens out, every step).  ``prefill`` is one 2,048-token prompt to its last logits;
``roofline`` is the decode step's bytes (every weight once, the cache of the live requests)
over its time; ``points`` holds batch 1 and 64.  The step's inputs (1.2 GB of weights plus the
cache) are larger than L2, so successive steps do not find them there.

``--impl reference`` would run kzw3933/Qwen-Engine itself from baseline/_ref; see
``reference_arm``.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(raw)
            peaks = dict(FALLBACK_PEAKS)
            for k in FALLBACK_PEAKS:
                if k in flat:
                    peaks[k] = flat[k]
            return peaks, "measured"
        except Exception:       # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def config_record(model, layers, layers_of_config, hidden, heads, kv_heads, head_dim, intermediate, vocab, batch, context,
                  page_size, prefill_tokens) -> dict:
    """The ``config`` of the JSON line: every size, flat, the same keys for both arms."""
    return {"model": model, "layers": layers, "layers_of_config": layers_of_config, "hidden": hidden, "heads": heads,
            "kv_heads": kv_heads, "head_dim": head_dim, "intermediate": intermediate, "vocab": vocab,
            "global_batch": batch, "seq_len": context, "page_size": page_size, "prefill_tokens": prefill_tokens,
            "l2": "inputs larger than L2", "parallelism": "single GPU"}


class ClockSampler:
    """nvidia-smi in the background during the timed regions (read-only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, spans: list[tuple[int, int]]) -> dict:
        rows = [r for a, b in spans for r in self.rows[a:b]] or self.rows
        sm = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(rows)}


def reference_arm(args) -> int:
    """The reference arm: the unmodified kzw3933/Qwen-Engine as installed into baseline/_ref
    (pip install --no-deps --target), through its own classes and stock code path in
    ``mode="triton"``: Qwen3Config defaults (Qwen3-0.6B) -> Qwen3ForCausalLM with its own random
    initialisation -> KVCachePool -> ModelExecutor.run_prefill / run_decode_step -> its argmax
    sampler, i.e. the body of its LLMEngine.serving loop (src/engine/llm_engine.py:101-145) with
    the step count under the benchmark's control.  Token ids stand in for its tokenizer, which needs
    the network.  Nothing of this repository's engine is imported."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "engine")) or not os.path.isdir(os.path.join(ref, "models")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref does not hold the reference's engine and models packages (not installed)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference is single-GPU"}))
        return 0
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, ref)
        from engine import KVCachePool                       # the reference's own packages
        from engine.executor import ModelExecutor
        from engine.sequence import Sequence
        from models import Qwen3Config, Qwen3ForCausalLM
        args.warmup = max(args.warmup, 3)
        rng = random.Random(0)
        cfg = Qwen3Config()
        dev = torch.device("cuda:0")
        torch.manual_seed(2)
        t0 = time.time()
        model = Qwen3ForCausalLM(**cfg.to_model_kwargs(), dtype=torch.bfloat16).to(dev).eval()
        print(f"[bench reference] model ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
        V, block = cfg.vocab_size, 16
        extra = args.warmup + args.steps + 4
        big = args.batch if args.no_points else max(args.batch, 64)
        blocks = big * (-(-(args.context + 3 * extra) // block) + 1) + args.prefill_tokens // block + 8
        pool = KVCachePool(num_layers=cfg.num_hidden_layers, num_blocks=blocks, block_size=block,
                           num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, dtype=torch.bfloat16, device=dev)
        ex = ModelExecutor(model, pool, dev, mode="triton")
        sid = [0]

        def new_seq(n):
            sid[0] += 1
            return Sequence(sid[0], "", [rng.randrange(V) for _ in range(n)])

        def decode_step(seqs):
            logits = ex.run_decode_step(seqs)                 # llm_engine.py:132-143
            toks = ex.sample_next_tokens(logits)
            for s, t in zip(seqs, toks):
                s.output_token_ids.append(t)
                s.num_computed_tokens += 1
                s.num_kv_tokens += 1
            ex.register_shared_blocks(seqs)

        clocks = ClockSampler()
        clocks.start()
        spans = []
        with torch.no_grad():
            # prefill of one 2,048-token prompt (its executor computes logits for every row)
            def prefill_once():
                s = new_seq(args.prefill_tokens)
                logits, ctx = ex.run_prefill([s])
                ex.sample_next_tokens(ex.gather_prefill_last_logits(logits, ctx.cu_seqlens))
                ex.release_sequence(s)
            for _ in range(2):
                prefill_once()
            torch.cuda.synchronize()
            m0 = clocks.mark()
            t0 = time.perf_counter()
            for _ in range(3):
                prefill_once()
            torch.cuda.synchronize()
            prefill_ms = (time.perf_counter() - t0) / 3 * 1e3
            spans.append((m0, clocks.mark()))

            def decode_rate(batch, steps, warmup):
                seqs = [new_seq(args.context) for _ in range(batch)]
                for i in range(0, batch, 8):
                    group = seqs[i:i + 8]
                    logits, ctx = ex.run_prefill(group)
                    toks = ex.sample_next_tokens(ex.gather_prefill_last_logits(logits, ctx.cu_seqlens))
                    for s, t in zip(group, toks):                # llm_engine.py:115-119
                        s.output_token_ids.append(t)
                        s.num_computed_tokens = s.num_kv_tokens = s.prompt_len
                for _ in range(warmup):
                    decode_step(seqs)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                m = clocks.mark()
                t0 = time.perf_counter()
                a.record()
                for _ in range(steps):
                    decode_step(seqs)
                b.record()
                torch.cuda.synchronize()
                wall = time.perf_counter() - t0
                spans.append((m, clocks.mark()))
                for s in seqs:
                    ex.release_sequence(s)
                return batch * steps / (a.elapsed_time(b) / 1e3), a.elapsed_time(b) / steps, batch * steps / wall
            value, ms_per_step, e2e_value = decode_rate(args.batch, args.steps, args.warmup)
            points = {}
            if not args.no_points:
                points["decode_b1"] = round(decode_rate(1, args.steps, 3)[0], 1)
                points["decode_b64"] = round(decode_rate(64, max(3, args.steps // 4), 2)[0], 1)
        clocks.stop()
        print(json.dumps({
            "metric": "decode tok/s (Qwen3-0.6B, batch 8, context 1024)", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic: uniform random token ids, the reference's own random initialisation",
            "config": config_record("qwen3-0.6b", cfg.num_hidden_layers, cfg.num_hidden_layers, cfg.hidden_size,
                                    cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size,
                                    cfg.vocab_size, args.batch, args.context, block, args.prefill_tokens),
            "mode": "triton",
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s"},
            "prefill": {"value": round(args.prefill_tokens / (prefill_ms / 1e3), 1), "tokens": args.prefill_tokens,
                        "ms": round(prefill_ms, 3)},
            "points": points, "clocks": clocks.summary(spans)}))
        return 0
    except Exception as e:          # noqa: BLE001 - the arm reports instead of failing the round
        msg = f"{type(e).__name__}: {e}".replace("\n", " ")[:300]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference did not run here: {msg}"}))
        return 0



def capture_context(runner, entries):
    """Run one step eagerly and hand back the StepContext the model saw (index data, block tables and the
    attention work lists on the device), for timing single kernels on a real step's data."""
    seen = []
    real = runner.model.forward
    graphs = runner.use_cuda_graphs
    runner.use_cuda_graphs = False
    runner.model.forward = lambda ctx, cache: (seen.append(ctx), real(ctx, cache))[1]
    try:
        runner.step(entries)
    finally:
        runner.model.forward = real
        runner.use_cuda_graphs = graphs
    return seen[0]


def kernel_chains(loaded, cfg, peaks, tag, ctx, torch, ops, out) -> None:
    """Each kernel class of the step alone: one launch per layer, back to back over the layers' own weights and
    caches (more bytes than L2 holds, as in the step), timed with CUDA events; microseconds a launch and the
    launch's bytes (decode: weights or keys and values read once) or flops (prompt portions) over the measured
    peak.  ``tag`` "decode": the classes of a decode step at the benchmark's batch; "prefill": those of its prompt.
    ``ctx`` must be the context of the step that ran last (its index data lives in the step function's buffer)."""
    model, cache = loaded.model, loaded.cache
    blocks = model.blocks
    L = len(blocks)
    H, Hq, Hkv, D, I = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    dev = "cuda:0"
    bf = torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def chain(fn, reps=5):
        """us a launch of the chain's L launches, replayed from a CUDA graph (so that the host's launch rate,
        a few microseconds a call from Python, does not show)."""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / reps / L

    def record(name, us, nbytes=None, flops=None):
        e = {"us": round(us, 2)}
        if nbytes is not None:
            e["gbs"] = round(nbytes / us / 1e3, 1)
            e["frac"] = round(nbytes / (us * 1e-6) / hbm, 3)
        if flops is not None:
            e["tflops"] = round(flops / us / 1e6, 1)
            e["frac"] = round(flops / (us * 1e-6) / tflops, 3)
        out[name] = e

    T = ctx.num_tokens
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.5).to(bf)      # noqa: E731
    x, attn, act = rnd(T, H), rnd(T, Hq * D), rnd(T, I)
    qkv, gate_up = rnd(T, (Hq + 2 * Hkv) * D), rnd(T, 2 * I)
    y_qkv, y_h, y_gu = torch.empty_like(qkv), torch.empty(T, H, dtype=bf, device=dev), torch.empty_like(gate_up)
    resid = torch.zeros(T, H, dtype=torch.float32, device=dev)
    a_out = torch.empty(T, Hq * D, dtype=bf, device=dev)
    dec = tag == "decode"
    tokens_kv = sum(ctx.ctx_lens_host) + T
    view = ctx.groups[cache.group_of_slot[0][0]]
    mixers = [b.mixer for b in blocks]
    ffns = [b.ffn for b in blocks]
    ctx.arena.reset()

    def products(name, ws, xin, yout, N, K):
        us = chain(lambda: [ops.linear(xin, w, yout) for w in ws])
        record(f"{tag}_{name}", us, nbytes=N * K * 2 if dec else None, flops=None if dec else 2.0 * T * N * K)
    rot0 = mixers[0].pos.half_split_rotation()
    if not dec and ops.qkv_rope_fused_applies(T, qkv.shape[1], H, bf, D, rot0.rotary_dim):
        # as the step runs it: per-head norm, rotation and cache write in the product's epilogue
        table = torch.empty(T, D // 2, 2, dtype=torch.float32, device=dev)
        ops.rope_table(ctx.positions, rot0.inv_freq, table)
        us = chain(lambda: [ops.linear_qkv_rope(x, m.w_qkv, y_qkv, m.q_norm_w, m.k_norm_w, cfg.rms_norm_eps, table,
                                                cache.layer_view(i), view.slot_mapping, Hq, Hkv) for i, m in enumerate(mixers)])
        record(f"{tag}_qkv_rope", us, flops=2.0 * T * (Hq + 2 * Hkv) * D * H)
    else:
        products("qkv", [m.w_qkv for m in mixers], x, y_qkv, (Hq + 2 * Hkv) * D, H)
    products("o", [m.w_o for m in mixers], attn, y_h, H, Hq * D)
    if not dec and ops.swiglu_fused_applies(T, I, H, bf):
        us = chain(lambda: [ops.linear_swiglu(x, f.w_gate_up, act) for f in ffns])
        record(f"{tag}_gate_up_swiglu", us, flops=2.0 * T * 2 * I * H)
    elif dec and ops.swiglu_small_applies(T, I, H, bf):
        us = chain(lambda: [ops.linear_swiglu_small(x, f.w_gate_up, act) for f in ffns])
        record(f"{tag}_gate_up_swiglu", us, nbytes=2 * I * H * 2)
    else:
        products("gate_up", [f.w_gate_up for f in ffns], x, y_gu, 2 * I, H)
    products("down", [f.w_down for f in ffns], act, y_h, H, I)

    def attention():
        for i, m in enumerate(mixers):
            mark = ctx.arena.mark()
            ops.paged_attention(qkv, cache.layer_view(i), view.block_tables, ctx, a_out, m.scale, 0, Hq, Hkv, D)
            ctx.arena.release(mark)
    us = chain(attention)
    kv_bytes = tokens_kv * 2 * Hkv * D * 2
    if dec:
        record("decode_attention", us, nbytes=kv_bytes)
    else:
        flops = sum(4.0 * Hq * D * n * (c + (n + 1) / 2) for n, c in zip(ctx.q_lens_host, ctx.ctx_lens_host))
        record("prefill_attention", us, flops=flops)
    out[f"{tag}_attention"]["kernel"] = ops.last_attention_kernel

    w_norm = blocks[0].norm1.weight
    us = chain(lambda: [ops.add_rmsnorm(resid, y_h, b.norm1.weight, cfg.rms_norm_eps, x) for b in blocks])
    record(f"{tag}_add_rmsnorm", us, nbytes=T * H * (4 + 4 + 2 + 2))
    del w_norm

    def rotary():
        for i, m in enumerate(mixers):
            rot = m.pos.half_split_rotation()
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, m.q_norm_w, m.k_norm_w, cfg.rms_norm_eps, rot.inv_freq, rot.rotary_dim,
                                      cache.layer_view(i), view.slot_mapping, Hq, Hkv, D)
    us = chain(rotary)
    record(f"{tag}_qk_norm_rope_kv_write", us, nbytes=T * (Hq + 2 * Hkv) * D * 2 * 2)
    if tag == "decode":
        # the output head on the wanted rows, alone (one launch: the matrix is larger than L2 by itself)
        N = ctx.num_logit_rows
        normed = torch.randn(N, H, device=dev).to(bf)
        logits = torch.empty(N, cfg.vocab_size, dtype=torch.float32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        times = []
        for _ in range(4):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            ops.linear(normed, model.head, logits)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        us = sorted(times[1:])[1]
        out["decode_lm_head"] = {"us": round(us, 2), "gbs": round(cfg.vocab_size * H * 2 / us / 1e3, 1),
                                 "frac": round(cfg.vocab_size * H * 2 / (us * 1e-6) / hbm, 3)}


def run_workload(name: str, torch, peaks) -> dict:
    """A scheduler workload at the sizes of a larger model, end to end through ``LLMEngine.serving`` with random
    weights: generated tokens a second (wall clock from the first step to the last), prompt tokens found in shared
    pages, preemptions, and steps, tokens and device time by kind of step."""
    from qwen_engine_b200.config import EngineConfig, preset_config_dict, preset_init
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.sampling import SamplingParams
    rng = random.Random(11)
    if name == "mixed-1.7b":
        preset, n_req, new_tokens, chunk, max_len = "qwen3-1.7b", 32, 256, 512, 2048 + 256 + 16
        lens = [rng.randint(128, 2048) for _ in range(n_req)]
        shared = 0
    elif name == "shared-prefix-4b":
        preset, n_req, new_tokens, chunk, max_len = "qwen3-4b", 16, 512, 2048, 4096
        lens = [1024 + 256] * n_req
        shared = 1024
    else:
        raise ValueError(f"unknown workload {name!r}")
    cfg = config_from_dict(preset_config_dict(preset))
    init = preset_init(preset)
    page = init["block_size"]
    V = cfg.vocab_size
    common = [rng.randrange(V) for _ in range(shared)]
    prompts = [common + [rng.randrange(V) for _ in range(n - shared)] for n in lens]
    pages = sum(-(-(n + new_tokens) // page) + 1 for n in lens) + 64
    t0 = time.time()
    loaded = load_model(None, torch.bfloat16, "cuda:0", page, pages, n_req, enable_prefix_cache=True, config=cfg,
                        random_seed=init["seed"], random_std=init["std"], random_norm_std=init["norm_std"])
    print(f"[bench] {name}: model ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
    ec = EngineConfig(dtype=torch.bfloat16, device="cuda:0", block_size=page, num_blocks=pages, max_model_len=max_len,
                      max_num_seqs=n_req, max_num_batched_tokens=chunk + n_req, prefill_chunk_size=chunk,
                      enable_prefix_cache=True, profile=True)
    eng = LLMEngine(loaded, ec)
    sp = SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)
    # warm-up outside the timed run: one short request through prompt and decoding (kernels loaded, arena sized)
    eng.add_request(prompts[0][:64] if not shared else [rng.randrange(V) for _ in range(64)], SamplingParams(max_new_tokens=4, ignore_eos=True))
    eng.serving()
    eng.stats.__init__()
    hit0, pre0 = eng.scheduler.prefix_hit_tokens, eng.scheduler.num_preemptions
    for p in prompts:
        eng.add_request(p, sp)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.serving()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    generated = sum(len(o.output_token_ids) for o in outs)
    st = eng.stats
    rec = {"model": preset, "layers": cfg.num_hidden_layers, "requests": n_req, "prompt_tokens": sum(lens),
           "new_tokens_each": new_tokens, "prefill_chunk": chunk, "value": round(generated / wall, 1), "unit": "generated tokens/s",
           "seconds": round(wall, 3), "generated_tokens": generated, "steps": st.steps,
           "prefix_hit_tokens": eng.scheduler.prefix_hit_tokens - hit0, "preemptions": eng.scheduler.num_preemptions - pre0,
           "graph_replays": loaded.runner.num_graph_replays, "graph_captures": loaded.runner.num_graph_captures,
           "capture_seconds": round(loaded.runner.graph_capture_seconds, 3),
           "by_kind": {k: {"steps": v["steps"], "tokens": v["tokens"], "device_ms": round(v["device_ms"], 1)}
                       for k, v in (st.profile or {}).items()}}
    del eng, loaded
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="qwen3-0.6b")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--workload", choices=["mixed-1.7b", "shared-prefix-4b"], default=None,
                    help="run only this scheduler workload (32 requests with prompts of 128..2048 tokens and 256 new tokens at "
                         "Qwen3-1.7B sizes in portions of 512; 16 requests sharing 1,024 of 1,280 prompt tokens with 512 new "
                         "tokens at Qwen3-4B sizes) and print its record as one JSON line")
    ap.add_argument("--no-workloads", action="store_true", help="skip the two scheduler workloads at the end of the default run")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel-class timings")
    ap.add_argument("--profile", choices=["decode", "prefill"], default=None,
                    help="bracket that timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from qwen_engine_b200 import ops
    if args.workload:
        peaks, _ = load_peaks()
        print(json.dumps({"metric": f"generated tok/s, workload {args.workload}", "impl": "ours", "n_gpus": 1,
                          **run_workload(args.workload, torch, peaks)}))
        return 0
    from qwen_engine_b200.config import EngineConfig, parse_dtype, preset_config_dict, preset_init
    from qwen_engine_b200.engine.llm import LLMEngine
    from qwen_engine_b200.engine.loading import load_model
    from qwen_engine_b200.engine.runner import StepEntry
    from qwen_engine_b200.registry import config_from_dict
    from qwen_engine_b200.sampling import SamplingParams

    peaks, peaks_src = load_peaks()
    dtype = parse_dtype(args.dtype)
    raw = preset_config_dict(args.preset)
    layers_of_config = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    init = preset_init(args.preset)
    page = init["block_size"]
    big_batch = args.batch if args.no_points else max(args.batch, 64)
    extra = args.warmup + args.steps + 8
    per_req = -(-(args.context + 3 * extra) // page) + 1
    pages = big_batch * per_req + -(-args.prefill_tokens // page) + 8
    t_load = time.time()
    loaded = load_model(None, dtype, "cuda:0", page, pages, big_batch + 2, enable_prefix_cache=False, config=cfg,
                        random_seed=init["seed"], random_std=init["std"], random_norm_std=init["norm_std"])
    print(f"[bench] model ready in {time.time() - t_load:.1f}s", file=sys.stderr, flush=True)
    runner, cache, model = loaded.runner, loaded.cache, loaded.model
    rng = random.Random(0)
    V = cfg.vocab_size

    def tokens(n):
        return [rng.randrange(V) for _ in range(n)]

    def timed(fn, n_iter, what=None):
        if what is not None and what == args.profile:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            try:
                return timed(fn, n_iter)
            finally:
                torch.cuda.profiler.stop()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_iter):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n_iter

    clocks = ClockSampler()
    clocks.start()
    spans = []

    # ---- prefill: one prompt of 2,048 tokens to its last logits ----------------------------------
    P = args.prefill_tokens
    prompt = tokens(P)

    def prefill_once():
        rc = cache.open("prefill")
        runner.step([StepEntry(rc, prompt, [P - 1])])
        cache.close(rc)
    for _ in range(args.warmup):
        prefill_once()
    m0 = clocks.mark()
    prefill_ms = timed(prefill_once, 5 if args.profile is None else 1, "prefill")
    spans.append((m0, clocks.mark()))
    # the first, eager run of a prompt length that has not come before (recurring shapes are replayed from a graph)
    def prefill_eager(n):
        rc = cache.open("prefill")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        runner.step([StepEntry(rc, prompt[:n], [n - 1])])
        torch.cuda.synchronize()
        cache.close(rc)
        return (time.perf_counter() - t0) * 1e3
    eager_ms = min(prefill_eager(P - 16 * k) for k in (1, 2, 3)) if args.profile is None else None
    c = cfg
    gemm_params = c.num_hidden_layers * (c.hidden_size * (c.q_width + 2 * c.kv_width) + c.q_width * c.hidden_size
                                         + 3 * c.hidden_size * c.intermediate_size)
    prefill_flops = 2.0 * P * gemm_params + c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * P * P / 2 \
        + 2.0 * c.vocab_size * c.hidden_size
    prefill = {"value": round(P / (prefill_ms / 1e3), 1), "tokens": P, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
               "first_run_ms": None if eager_ms is None else round(eager_ms, 3)}

    # ---- decode at batch 64, 8, 1 over real, scattered pages ----------------------------------------
    reqs = [cache.open(f"d{i}") for i in range(big_batch)]
    per_step = max(1, 4096 // args.context)
    for i in range(0, big_batch, per_step):
        runner.step([StepEntry(rc, tokens(args.context), []) for rc in reqs[i:i + per_step]])
    torch.cuda.synchronize()
    weight_bytes = model.weight_bytes()
    kv_bytes_per_token = sum(g.tensor[:, 0].numel() // g.tensor.shape[4] * g.tensor.element_size()
                             for g in cache.paged_groups)      # all layers, K and V, one token

    def decode_rate(batch, steps, warmup, record=None, what=None):
        live = reqs[:batch]

        def one():
            runner.step([StepEntry(rc, [rng.randrange(V)], [0]) for rc in live])
        for _ in range(warmup):
            one()
        l0, m = ops.launch_count, clocks.mark()
        ms = timed(one, steps, what)
        if record is not None:
            record["launches"] = ops.launch_count - l0
            spans.append((m, clocks.mark()))
        return batch * 1e3 / ms, ms

    points = {}
    points_detail = {}

    def point(name, batch, steps):
        rate, ms = decode_rate(batch, steps, 3)
        nbytes = weight_bytes + batch * reqs[0].num_tokens * kv_bytes_per_token
        points[name] = round(rate, 1)
        points_detail[name] = {"ms": round(ms, 4), "context": reqs[0].num_tokens, "gbs": round(nbytes / ms / 1e6, 1),
                               "frac": round(nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
    if not args.no_points and big_batch >= 64:
        point("decode_b64", 64, max(5, args.steps // 2))
    rec = {}
    value, ms_per_step = decode_rate(args.batch, args.steps, args.warmup, rec, "decode")
    ctx_now = reqs[0].num_tokens
    step_bytes = weight_bytes + args.batch * ctx_now * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    if not args.no_points:
        point("decode_b1", 1, args.steps)
    kernels = {}
    if not args.no_kernels and args.profile is None and dtype == torch.bfloat16:
        dctx = capture_context(runner, [StepEntry(rc, [rng.randrange(V)], [0]) for rc in reqs[:args.batch]])
        kernel_chains(loaded, cfg, peaks, "decode", dctx, torch, ops, kernels)
        rc = cache.open("prefill")
        pctx = capture_context(runner, [StepEntry(rc, prompt, [P - 1])])
        kernel_chains(loaded, cfg, peaks, "prefill", pctx, torch, ops, kernels)
        cache.close(rc)
    for rc in reqs:
        cache.close(rc)

    # ---- end to end through the Python entry point ----------------------------------------------------
    ec = EngineConfig(dtype=dtype, device="cuda:0", block_size=page, num_blocks=pages, max_model_len=args.context + 4 * extra,
                      max_num_seqs=args.batch, max_num_batched_tokens=4096, enable_prefix_cache=False)
    eng = LLMEngine(loaded, ec)
    # (at least 5 untimed decode steps: a step launched ahead is a shape of its own, run eagerly at first sight
    # and captured in a CUDA graph at the second, after the one decode step that is not launched ahead)
    e2e_warmup = max(args.warmup, 5)
    sp = SamplingParams(max_new_tokens=e2e_warmup + args.steps + 8, ignore_eos=True)    # (the requests' ends lie outside the timed steps)
    for _ in range(args.batch):
        eng.add_request(tokens(args.context), sp)
    while eng.stats.decode_tokens < args.batch * e2e_warmup:      # prompts, then the warm-up decode steps
        eng.step()
    torch.cuda.synchronize()
    import gc
    gc.collect()
    gc.disable()                 # (a collection of the benchmark's own heap in mid-loop would stall the host for longer than a step)
    m0 = clocks.mark()
    t0 = time.perf_counter()
    call_s = []
    for _ in range(args.steps):
        t1 = time.perf_counter()
        eng.step()                                                  # host tokens in, sampled tokens out
        call_s.append(time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    gc.enable()
    print(f"[bench] end to end: {e2e_s / args.steps * 1e3:.3f} ms a step; calls (ms): " + " ".join(f"{c * 1e3:.2f}" for c in call_s), file=sys.stderr)
    spans.append((m0, clocks.mark()))
    e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.last_h2d_bytes, "d2h_bytes_per_step": 4 * args.batch}
    while eng.has_work():
        eng.step()
    eng.check_device()               # no bounded wait inside a kernel ran out during any of the above
    workloads = {}
    if not args.no_workloads and args.profile is None and dtype == torch.bfloat16 and args.preset == "qwen3-0.6b" and not args.layers:
        del eng, reqs, runner, cache, model
        loaded.runner = loaded.cache = loaded.model = None
        import gc as _gc
        _gc.collect()
        torch.cuda.empty_cache()
        for w in ("mixed-1.7b", "shared-prefix-4b"):
            try:
                workloads[w] = run_workload(w, torch, peaks)
            except Exception as e:      # noqa: BLE001 - the headline stands without them
                workloads[w] = {"failed": f"{type(e).__name__}: {e}"[:200]}
    clocks.stop()

    line = {
        "metric": "decode tok/s (Qwen3-0.6B, batch 8, context 1024)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "fp32",
        "data": "synthetic: uniform random token ids, random weights N(0, 0.02) seed 2", "impl": "ours",
        "config": config_record(args.preset, cfg.num_hidden_layers, layers_of_config, c.hidden_size, c.num_attention_heads,
                                c.num_key_value_heads, c.head_dim, c.intermediate_size, c.vocab_size, args.batch,
                                args.context, page, P),
        "context_at_timing": ctx_now, "peaks": peaks_src,
        "e2e": e2e, "gpu_launches": rec.get("launches", 0),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points, "points_detail": points_detail,
        "kernels": kernels, "workloads": workloads,
        "clocks": clocks.summary(spans),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
