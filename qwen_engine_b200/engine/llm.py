"""The Python entry point: ``LLM.generate`` and, in the reference's manner,
``LLMEngine.submit`` / ``LLMEngine.serving`` (src/engine/llm_engine.py:75-152).

Host tokens go in, host tokens come out; everything between runs through the
scheduler, the step function and the sampler on the device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence as Seq, Union

import torch

from ..config import EngineConfig, ModelConfig, parse_dtype
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, uniform_for
from .loading import LoadedModel, load_model
from .runner import StepEntry
from .scheduler import Scheduler, SchedulerOutput
from .sequence import Sequence


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


class LLMEngine:
    """The engine: a loaded model, its cache, a scheduler and a sampler.

    ``submit`` queues requests, ``step`` runs one scheduled batch, ``serving``
    runs until every queued request has ended (the reference's loop,
    llm_engine.py:101-152)."""

    def __init__(self, loaded: LoadedModel, engine_config: EngineConfig, tokenizer=None):
        self.loaded = loaded
        self.config = engine_config
        self.tokenizer = tokenizer
        self.model_config = loaded.config
        self.cache = loaded.cache
        self.runner = loaded.runner
        self.sampler = Sampler(loaded.runner.device)
        self.scheduler = Scheduler(
            self.cache, engine_config.max_num_seqs, engine_config.max_num_batched_tokens,
            engine_config.prefill_chunk_size, engine_config.max_model_len,
            eos_token_id=getattr(loaded.config, "eos_token_id", None))
        self._next_seq_id = 0
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
    def step(self) -> list[Sequence]:
        """Schedule, run and sample one batch; returns the requests that ended in it."""
        t0 = time.perf_counter()
        out: SchedulerOutput = self.scheduler.schedule()
        if not out.scheduled:
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler found nothing to run although requests are pending")
            return []
        entries = []
        for sch in out.scheduled:
            toks = sch.seq.get_tokens(sch.start, sch.num_tokens)
            entries.append(StepEntry(sch.seq.cache, toks, [sch.num_tokens - 1] if sch.wants_logits else []))
        logits = self.runner.step(entries)
        sampled: dict[int, int] = {}
        wanting = [s for s in out.scheduled if s.wants_logits]
        if wanting:
            params = [s.seq.sampling for s in wanting]
            uniforms = [uniform_for(p.seed if p.seed is not None else self.config.seed, s.seq.seq_id,
                                    s.seq.output_len) for p, s in zip(params, wanting)]
            tokens = self.sampler.sample(logits, params, uniforms)
            sampled = {s.seq.seq_id: t for s, t in zip(wanting, tokens)}
        for sch in out.scheduled:
            if sch.num_tokens == 1 and sch.seq.output_len > 0:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += sch.num_tokens
        ended = self.scheduler.update(out, sampled)
        st = self.stats
        st.steps += 1
        st.generated_tokens += len(sampled)
        st.prefix_hit_tokens = self.scheduler.prefix_hit_tokens
        st.preemptions = self.scheduler.num_preemptions
        st.peak_pages_used = self.cache.peak_pages_used
        st.pages_in_use = self.cache.pages_in_use()
        st.step_seconds += time.perf_counter() - t0
        return ended

    def has_work(self) -> bool:
        return self.scheduler.has_work()

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
    enable_prefix_cache, seed, device)."""

    def __init__(self, model: Union[str, ModelConfig], tokenizer=None, weights_seed: Optional[int] = None,
                 weights_std: float = 0.02, weights_norm_std: float = 0.1, **engine_kwargs):
        if "dtype" in engine_kwargs:
            engine_kwargs["dtype"] = parse_dtype(engine_kwargs["dtype"])
        self.engine_config = EngineConfig(**engine_kwargs)
        ec = self.engine_config
        if isinstance(model, str):
            loaded = load_model(model, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(),
                                ec.max_num_seqs, ec.enable_prefix_cache, use_cuda_graphs=ec.use_cuda_graphs)
            tokenizer = tokenizer or _load_tokenizer(model)
        else:
            loaded = load_model(None, ec.dtype, ec.device, ec.block_size, ec.resolved_num_blocks(),
                                ec.max_num_seqs, ec.enable_prefix_cache, config=model,
                                random_seed=ec.seed if weights_seed is None else weights_seed,
                                random_std=weights_std, random_norm_std=weights_norm_std,
                                use_cuda_graphs=ec.use_cuda_graphs)
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
