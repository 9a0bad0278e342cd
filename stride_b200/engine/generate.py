"""The Python entry point: token ids in, token ids out.

    from stride_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)
    outs[0].tokens

arhaamatiq/stride has no Python entry; this one wraps the same Engine and Scheduler that
the command line drives (tools/stride_cli.cpp:124-251), with its names for the options.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..sampling.sampler import SamplingParams
from .engine import Engine, EngineOptions
from .scheduler import GenRequest, Scheduler, SchedulerOptions


@dataclass
class GenerationResult:
    tokens: list = field(default_factory=list)
    values: list = field(default_factory=list)       # the logit of every chosen token
    finish_reason: str = ""
    fingerprint: int = 0
    logits: list = field(default_factory=list)       # rows of logits, if asked for


class LLM:
    def __init__(self, model=None, *, dtype: str = "bfloat16", engine: Optional[Engine] = None, concurrency: int = 256,
                 max_rows: int = 256, prefill_chunk: int = 64, row_shuffle_seed: int = 0, **engine_options):
        """`model`: a folder with config.json and model.safetensors. Further keyword arguments are
        fields of `EngineOptions` (kv_bytes, kv_pages, page_size, max_context, max_slots, ...)."""
        if engine is None:
            opts = EngineOptions(dtype=dtype, max_rows=max_rows,
                                 max_full_rows=engine_options.pop("max_full_rows", min(max_rows, max(concurrency, 1))),
                                 **engine_options)
            engine = Engine(model, opts)
        self.engine = engine
        self.scheduler_options = SchedulerOptions(max_seqs=concurrency, max_rows=min(max_rows, engine.options.max_rows),
                                                  prefill_chunk=prefill_chunk, row_shuffle_seed=row_shuffle_seed)
        self.last_stats = None

    def generate(self, prompts: list, max_new_tokens: int = 16, sampling: Optional[SamplingParams] = None, *,
                 temperature: float = 0.0, top_p: float = 1.0, top_k: int = 0, seed: int = 0, stop_tokens=(),
                 use_eos: bool = False, full_logits: bool = False) -> list:
        """Generate for every prompt (a list of token ids). Request i samples with seed + i."""
        base = sampling or SamplingParams(temperature, top_p, top_k, seed)
        stops = tuple(stop_tokens) + (tuple(self.engine.spec.eos_token_ids) if use_eos else ())
        sched = Scheduler(self.engine, self.scheduler_options)
        results = [GenerationResult() for _ in prompts]

        def make_callback(r: GenerationResult):
            def on_token(ev, logits):
                if ev.token >= 0:
                    r.tokens.append(ev.token)
                    r.values.append(ev.value)
                    r.fingerprint = ev.fingerprint
                    if logits is not None:
                        r.logits.append(logits.copy())
                if ev.finished:
                    r.finish_reason = ev.finish_reason or ""
            return on_token

        for i, p in enumerate(prompts):
            sp = SamplingParams(base.temperature, base.top_p, base.top_k, base.seed + i)
            sched.submit(GenRequest(prompt=list(p), max_new_tokens=max_new_tokens, sampling=sp, stop_tokens=stops,
                                    full_logits=full_logits, on_token=make_callback(results[i])))
        sched.run()
        self.last_stats = sched.stats
        return results


def generate(model, prompts: list, max_new_tokens: int = 16, *, dtype: str = "bfloat16", **kwargs) -> list:
    """One-shot form of `LLM(model, ...).generate(prompts, ...)`; returns the lists of new tokens."""
    gen_keys = ("sampling", "temperature", "top_p", "top_k", "seed", "stop_tokens", "use_eos", "full_logits")
    gen_args = {k: kwargs.pop(k) for k in gen_keys if k in kwargs}
    llm = LLM(model, dtype=dtype, **kwargs)
    return [r.tokens for r in llm.generate(prompts, max_new_tokens, **gen_args)]
