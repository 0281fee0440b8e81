"""The Python entry point: ``LLM.generate`` and, in the reference's manner,
``LLMEngine.submit`` / ``LLMEngine.serving`` (src/engine/llm_engine.py:75-152).

Host tokens go in, host tokens come out; everything between runs through the
scheduler, the step function and the sampler on the device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Optional, Sequence as Seq, Union

from ..cache.manager import UNKNOWN_TOKEN
from ..config import EngineConfig, ModelConfig, parse_dtype
from ..sampling.params import SamplingParams
from ..sampling.sampler import SampledTokens, Sampler, uniform_for
from .loading import LoadedModel, load_model
from .runner import StepEntry
from .scheduler import Scheduler, SchedulerOutput
from .sequence import Sequence, SequenceStatus


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    finish_reason: Optional[str]
    text: Optional[str] = None
    prompt_text: Optional[str] = None
    num_preemptions: int = 0
    shared_prefix_len: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    prefix_hit_tokens: int = 0
    preemptions: int = 0
    peak_pages_used: int = 0
    pages_in_use: int = 0
    step_seconds: float = 0.0
    # with EngineConfig.profile: steps, tokens and device time (ms, CUDA events around the step and its
    # sampling) by kind of step: "decode" (single decoded tokens only), "prefill" (prompt portions only), "mixed"
    profile: Optional[dict] = None

    def profile_table(self) -> str:
        if not self.profile:
            return "no profile (EngineConfig.profile is off, or no step ran on a CUDA device)"
        lines = [f"{'kind':8s} {'steps':>7s} {'tokens':>9s} {'device ms':>10s} {'ms/step':>8s} {'tokens/s':>10s}"]
        for kind, p in self.profile.items():
            ms = p["device_ms"]
            lines.append(f"{kind:8s} {p['steps']:7d} {p['tokens']:9d} {ms:10.2f} {ms / max(1, p['steps']):8.3f} "
                         f"{p['tokens'] / ms * 1e3 if ms > 0 else 0.0:10.0f}")
        return "\n".join(lines)


@dataclass
class _Flight:
    """A step that is launched and whose sampled tokens the host has not read yet."""

    out: SchedulerOutput
    wanting: list                       # the scheduled requests that get a token, in the order of the logits' rows
    tokens: Optional[SampledTokens]     # None: the step samples nothing (prompt portions only)
    decode_tokens: int = 0
    prefill_tokens: int = 0
    events: Optional[tuple] = None      # profile: CUDA events before and after the step's launches


class LLMEngine:
    """The engine: a loaded model, its cache, a scheduler and a sampler.

    ``submit`` queues requests, ``step`` runs one scheduled batch, ``serving``
    runs until every queued request has ended (the reference's loop,
    llm_engine.py:101-152).

    With ``EngineConfig.run_ahead`` a step is scheduled and launched before the host has read the tokens
    of the step before it, so that the host's work on a step (scheduling, the work lists, the launches)
    overlaps the device's work on the one before: the token ids that decoding requests need stay on the
    device, the requests' outputs hold a place for them (``UNKNOWN_TOKEN``), and ``step`` returns what
    the older of the two steps produced.  Prompt portions and admissions need no token of the step in
    flight and go into the step launched ahead as into any other.  A request that turns out to have
    ended (a stop token) while the step launched ahead carried it loses that step's token; one that
    ends by a count is known beforehand and is not carried.  A step launched ahead never preempts: a
    request that finds no pages sits it out, and when nothing can run the next step is scheduled with
    the tokens read, preemption allowed."""

    def __init__(self, loaded: LoadedModel, engine_config: EngineConfig, tokenizer=None):
        self.loaded = loaded
        self.config = engine_config
        self.tokenizer = tokenizer
        self.model_config = loaded.config
        self.cache = loaded.cache
        self.runner = loaded.runner
        self.sampler = Sampler(loaded.runner.device)
        limit = loaded.runner.max_positions
        if limit is not None and engine_config.max_model_len > limit:
            # found here, not in the middle of serving, where the step function would refuse the position
            raise ValueError(f"max_model_len = {engine_config.max_model_len} is beyond the model's "
                             f"max_position_embeddings = {limit}")
        eos = getattr(loaded.config, "eos_token_ids", None) or getattr(loaded.config, "eos_token_id", None)
        self.scheduler = Scheduler(
            self.cache, engine_config.max_num_seqs, engine_config.max_num_batched_tokens,
            engine_config.prefill_chunk_size, engine_config.max_model_len, eos_token_id=eos)
        self._next_seq_id = 0
        self._flight: Optional[_Flight] = None
        self._checks_device = loaded.runner.device.type == "cuda"
        self.stats = EngineStats()

    # ---- intake -------------------------------------------------------------------------
    def _encode(self, prompt: Union[str, Seq[int]]) -> tuple[list[int], Optional[str]]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass token ids, or a model folder "
                                 "that holds tokenizer files")
            # as the reference does (llm_engine.py:52-55)
            ids = self.tokenizer(prompt, return_tensors="pt").input_ids[0].tolist()
            return ids, prompt
        return [int(t) for t in prompt], None

    def add_request(self, prompt: Union[str, Seq[int]], sampling: Optional[SamplingParams] = None) -> int:
        ids, text = self._encode(prompt)
        vocab = self.loaded.model.layout.vocab_size
        for t in ids:
            if not (0 <= t < vocab):
                raise ValueError(f"token id {t} is outside the vocabulary (0..{vocab - 1})")
        seq = Sequence(self._next_seq_id, ids, sampling or SamplingParams(), prompt_text=text)
        self.scheduler.add(seq)
        self._next_seq_id += 1
        return seq.seq_id

    def submit(self, prompt_texts, max_new_tokens: int = 16, sampling: Optional[SamplingParams] = None) -> list[int]:
        """Queue prompts (texts or token-id lists), as llm_engine.py:75-80."""
        if isinstance(prompt_texts, str) or (prompt_texts and isinstance(prompt_texts[0], int)):
            prompt_texts = [prompt_texts]
        ids = []
        for p in prompt_texts:
            sp = sampling or SamplingParams(max_new_tokens=max_new_tokens)
            ids.append(self.add_request(p, sp))
        return ids

    # ---- one step ---------------------------------------------------------------------
    def _launch(self, out: SchedulerOutput, before: Optional[_Flight]) -> Optional[_Flight]:
        """Run and sample the scheduled batch without waiting for the device.  ``before``: the step
        whose tokens are still on the device; requests whose newest token is a place for one of them
        take it from there."""
        if not out.scheduled:
            return None
        source = {sch.seq.seq_id: i for i, sch in enumerate(before.wanting)} if before is not None else {}
        entries = []
        flight = _Flight(out, [s for s in out.scheduled if s.wants_logits], None)
        for sch in out.scheduled:
            toks = sch.seq.get_tokens(sch.start, sch.num_tokens)
            src = None
            if toks and toks[-1] == UNKNOWN_TOKEN:
                if len(toks) != 1 or sch.seq.seq_id not in source:
                    raise RuntimeError(f"request {sch.seq.seq_id}: a token that is not known yet can only be run alone")
                src = source[sch.seq.seq_id]
            entries.append(StepEntry(sch.seq.cache, toks, [sch.num_tokens - 1] if sch.wants_logits else [], src))
            if sch.num_tokens == 1 and sch.seq.output_len > 0:
                flight.decode_tokens += 1
            else:
                flight.prefill_tokens += sch.num_tokens
        device_tokens = before.tokens.device if (before is not None and before.tokens is not None) else None
        timed = self.config.profile and self.runner.device.type == "cuda"
        if timed:
            import torch
            flight.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            flight.events[0].record()
        logits = self.runner.step(entries, device_tokens=device_tokens)
        if flight.wanting:
            params = [s.seq.sampling for s in flight.wanting]
            uniforms = [uniform_for(p.seed if p.seed is not None else self.config.seed, s.seq.seq_id,
                                    s.seq.output_len) for p, s in zip(params, flight.wanting)]
            flight.tokens = self.sampler.sample_async(logits, params, uniforms)
        if timed:
            flight.events[1].record()
        return flight

    def _account(self, cur: _Flight) -> None:
        """Profile: the device time of a step whose results the host has (or waits for here)."""
        if cur.events is None:
            return
        cur.events[1].synchronize()
        kind = "decode" if cur.prefill_tokens == 0 else ("prefill" if cur.decode_tokens == 0 else "mixed")
        if self.stats.profile is None:
            self.stats.profile = {}
        p = self.stats.profile.setdefault(kind, {"steps": 0, "tokens": 0, "device_ms": 0.0})
        p["steps"] += 1
        p["tokens"] += cur.decode_tokens + cur.prefill_tokens
        p["device_ms"] += float(cur.events[0].elapsed_time(cur.events[1]))

    def _can_run_ahead(self, cur: _Flight) -> bool:
        """Whether the next step may be scheduled and launched before the tokens of ``cur`` are read: the
        requests that get a token from it are all still running (their next token's id is then taken
        from the device)."""
        if not self.config.run_ahead:
            return False
        return all(s.seq.status is SequenceStatus.RUNNING and s.seq.cache is not None for s in cur.wanting)

    def step(self) -> list[Sequence]:
        """Schedule, run and sample one batch; returns the requests that ended in the step whose
        tokens were read (with ``run_ahead``, the step before the one just launched)."""
        t0 = time.perf_counter()
        if self._flight is None:
            out: SchedulerOutput = self.scheduler.schedule()
            if not out.scheduled:
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler found nothing to run although requests are pending")
                return []
            self._flight = self._launch(out, None)
        cur, self._flight = self._flight, None
        placed: Optional[dict[int, int]] = None
        if self._can_run_ahead(cur):
            placed = {}
            for sch in cur.wanting:
                seq = sch.seq
                seq.hold = self.scheduler.ends_by_length_after(seq, 1)
                placed[seq.seq_id] = seq.output_len
                seq.output_token_ids.append(UNKNOWN_TOKEN)
            ahead = self.scheduler.schedule(may_preempt=False)
            if ahead.preempted:
                raise RuntimeError("a step launched ahead must not preempt")
            self._flight = self._launch(ahead, cur)
        sampled: dict[int, int] = {}
        if cur.tokens is not None:
            sampled = {s.seq.seq_id: t for s, t in zip(cur.wanting, cur.tokens.read())}
        self.stats.decode_tokens += cur.decode_tokens
        self.stats.prefill_tokens += cur.prefill_tokens
        self._account(cur)
        ended = self.scheduler.update(cur.out, sampled, placed)
        st = self.stats
        st.steps += 1
        st.generated_tokens += sum(1 for s in cur.wanting if s.seq.seq_id in sampled)
        st.prefix_hit_tokens = self.scheduler.prefix_hit_tokens
        st.preemptions = self.scheduler.num_preemptions
        st.peak_pages_used = self.cache.peak_pages_used
        st.pages_in_use = self.cache.pages_in_use()
        st.step_seconds += time.perf_counter() - t0
        return ended

    def has_work(self) -> bool:
        return self._flight is not None or self.scheduler.has_work()

    def check_device(self) -> None:
        """Every wait inside the kernels is bounded; one that runs out makes its kernel return without its
        output and leaves a code in a status word.  This reads the words (it synchronises the device, so it
        is called where the engine has nothing in flight: at the end of ``serving``, and by callers of
        ``step`` when they see fit) and raises ``ops.DeviceWaitTimeout`` if any is set."""
        if self._checks_device:
            from .. import ops
            ops.check_device_status()

    def _output_of(self, seq: Sequence) -> RequestOutput:
        text = None
        if self.tokenizer is not None:
            # the reference decodes prompt and output together (llm_engine.py:67-73)
            text = self.tokenizer.decode(seq.prompt_token_ids + seq.output_token_ids, skip_special_tokens=True)
        return RequestOutput(seq.seq_id, list(seq.prompt_token_ids), list(seq.output_token_ids),
                             seq.finish_reason, text, seq.prompt_text, seq.num_preemptions,
                             seq.shared_prefix_len)

    def serving(self, print_func: Optional[Callable] = None) -> list[RequestOutput]:
        """Run until every queued request has ended; ``print_func(prompt_text, output_text)`` is
        called for each, as in llm_engine.py:101-152."""
        done: list[Sequence] = []
        while self.has_work():
            done.extend(self.step())
        self.check_device()
        done.sort(key=lambda s: s.seq_id)
        outs = [self._output_of(s) for s in done]
        if print_func is not None:
            for o in outs:
                shown = o.text if o.text is not None else " ".join(str(t) for t in o.output_token_ids)
                prompt = o.prompt_text if o.prompt_text is not None else " ".join(str(t) for t in o.prompt_token_ids)
                print_func(prompt, shown)
        return outs


def _load_tokenizer(model_dir: Optional[str]):
    """A tokenizer only if the model folder carries one; the token-id interface needs none."""
    import os
    if model_dir is None or not any(os.path.isfile(os.path.join(model_dir, f))
                                    for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_dir)
    except Exception:                                     # noqa: BLE001 - text prompts are then refused
        return None


class LLM:
    """``LLM(model=folder).generate(prompts, sampling_params)``.

    ``model`` is a folder with config.json and model.safetensors, or a model
    configuration (then ``seed`` draws random weights).  Keyword arguments are
    the fields of ``EngineConfig`` (dtype, block_size, num_blocks,
    max_model_len, max_num_seqs, max_num_batched_tokens, prefill_chunk_size,
    enable_prefix_cache, seed, device, run_ahead, profile)."""

    def __init__(self, model: Union[str, ModelConfig], tokenizer=None, weights_seed: Optional[int] = None,
                 weights_std: float = 0.02, weights_norm_std: float = 0.1, **engine_kwargs):
        if "dtype" in engine_kwargs:
            engine_kwargs["dtype"] = parse_dtype(engine_kwargs["dtype"])
        self.engine_config = EngineConfig(**engine_kwargs)
        ec = self.engine_config
        if isinstance(model, str):
            loaded = load_model(model, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(),
                                ec.max_num_seqs, ec.enable_prefix_cache, use_cuda_graphs=ec.use_cuda_graphs,
                                gpu_memory_fraction=ec.gpu_memory_fraction)
            tokenizer = tokenizer or _load_tokenizer(model)
        else:
            loaded = load_model(None, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(),
                                ec.max_num_seqs, ec.enable_prefix_cache, config=model,
                                random_seed=ec.seed if weights_seed is None else weights_seed,
                                random_std=weights_std, random_norm_std=weights_norm_std,
                                use_cuda_graphs=ec.use_cuda_graphs, gpu_memory_fraction=ec.gpu_memory_fraction)
        self.engine = LLMEngine(loaded, ec, tokenizer)

    def generate(self, prompts, sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None
                 ) -> list[RequestOutput]:
        if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.engine.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        outs = {o.request_id: o for o in self.engine.serving()}
        return [outs[i] for i in ids]

    def add_request(self, prompt, sampling: Optional[SamplingParams] = None) -> int:
        return self.engine.add_request(prompt, sampling)

    def step(self) -> list[RequestOutput]:
        return [self.engine._output_of(s) for s in self.engine.step()]

    def stats(self) -> EngineStats:
        return self.engine.stats
