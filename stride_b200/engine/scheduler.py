"""Continuous batching above the step function.

Each `step()`: drop cancelled requests; admit waiting requests while slots and pages
allow; plan the batch under the token budget (every request with exactly one unprocessed
token first, one row each; then portions of prompts, at most `prefill_chunk` tokens per
request, in running order); if the plan needs more pages than are free, preempt the
youngest running request (its slot and pages go back, it returns to the FRONT of the
waiting queue and is later recomputed from its first token, prompt and generated tokens
alike) and plan again; run the batch through `Engine.step`; choose a token for every
request whose last known token was in the batch; finish on a stop token ("stop") or on
max_new_tokens ("length") and give slot and pages back.

The decisions (the admission rule, the plan under the budget, the page arithmetic and the
choice of what to do when pages are short) are taken by the native planner in
`csrc/runtime.cpp`, on the books of the native page pool; this module keeps the requests,
their tokens and callbacks, and drives the engine and the sampler.

This restates arhaamatiq/stride's Scheduler (src/scheduler.cpp:72-304) including its
admission rule (free pages >= pages of the prompt + one page of growth per running request
+ one, unless nothing is running) and its failure when a single running request does not
fit ("KV arena too small for one sequence"). Requests longer than the context capacity, or
empty, finish at intake with "context_length" / "empty_prompt" (src/scheduler.cpp:82-89).
"""
from __future__ import annotations

import ctypes
import threading
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

from ..sampling.sampler import Sampler, SamplingParams, splitmix64
from .engine import Engine, EngineError, StepEntry

_FNV_OFFSET = 14695981039346656037
_FNV_PRIME = 1099511628211
_MASK = (1 << 64) - 1


def _fnv_mix(h: int, v: int) -> int:
    for i in range(4):
        h ^= (v >> (i * 8)) & 0xFF
        h = (h * _FNV_PRIME) & _MASK
    return h


def _float_bits(v: float) -> int:
    return int(np.float32(v).view(np.uint32))


@dataclass
class TokenEvent:
    token: int = -1
    value: float = 0.0
    index: int = 0                 # 0-based index among the generated tokens
    finished: bool = False
    finish_reason: Optional[str] = None
    fingerprint: int = 0           # FNV-1a over (token, bits of its logit) of all tokens so far


@dataclass
class GenRequest:
    prompt: list
    max_new_tokens: int = 16
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_tokens: tuple = ()
    full_logits: bool = False      # pass the logits row to on_token at every generated token
    on_token: Optional[Callable] = None    # on_token(event, logits or None)
    cancelled: Optional[threading.Event] = None


@dataclass
class SchedulerOptions:
    max_seqs: int = 256            # most requests running at once
    max_rows: int = 256            # token budget of one step
    prefill_chunk: int = 64        # most prompt tokens of one request in one step
    row_shuffle_seed: int = 0      # tests: shuffle the order of the requests inside a batch


@dataclass
class SchedulerStats:
    steps: int = 0
    rows: int = 0
    generated: int = 0
    preemptions: int = 0
    replayed_rows: int = 0
    peak_seqs: int = 0
    peak_blocks: int = 0


class _Seq:
    __slots__ = ("req", "tokens", "prompt_len", "next_pos", "generated", "slot", "arrival", "fingerprint", "done",
                 "inflight", "launched", "closing")

    def __init__(self, req: GenRequest, arrival: int):
        self.req = req
        self.tokens = list(req.prompt)
        self.prompt_len = len(self.tokens)
        self.next_pos = 0
        self.generated = 0
        self.slot = -1
        self.arrival = arrival
        self.fingerprint = _FNV_OFFSET
        self.done = False
        self.inflight = 0       # pipelined mode: steps launched for this request whose tokens the host has not read yet
        self.launched = 0       # tokens whose sampling has been launched (>= generated)
        self.closing = False    # no further step is to be launched for it (it finishes with a token already launched)


_DRAIN = object()      # plan(): the steps in flight have to be read back before a decision can be taken
_PLAN_RUN, _PLAN_NOTHING, _PLAN_DRAIN, _PLAN_TOO_SMALL, _PLAN_PREEMPT = range(5)    # results of sb_sched_plan
_I32P, _U8P, _I64P = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_int64)


class _PlanBuffers:
    """Arrays the native planner reads (one row per running request) and writes (the plan)."""
    FIELDS = (("slot", np.int32, _I32P), ("next_pos", np.int32, _I32P), ("total", np.int32, _I32P), ("closing", np.uint8, _U8P),
              ("inflight", np.uint8, _U8P), ("arrival", np.int64, _I64P), ("out_index", np.int32, _I32P), ("out_count", np.int32, _I32P))

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.out_n = ctypes.c_int32(0)
        for name, dtype, ptr in self.FIELDS:
            arr = np.zeros(capacity, dtype=dtype)
            setattr(self, name, arr)
            setattr(self, name + "_p", arr.ctypes.data_as(ptr))


class Scheduler:
    def __init__(self, engine: Engine, options: Optional[SchedulerOptions] = None, sampler=None):
        self.engine = engine
        self.opts = options or SchedulerOptions()
        if self.opts.max_rows > engine.options.max_rows:
            raise EngineError(f"scheduler max_rows {self.opts.max_rows} exceeds the engine's {engine.options.max_rows}")
        self.stats = SchedulerStats()
        self._mu = threading.Lock()
        self._incoming: deque = deque()
        self._waiting: deque = deque()
        self._running: list = []
        self._arrival = 0
        self._rng_state = self.opts.row_shuffle_seed
        self._sampler = sampler or Sampler(engine.device, engine.env.max_logit_rows)
        lib = self._lib = engine.cache._lib
        if not getattr(lib, "_sb_sched_typed", False):
            lib.sb_sched_may_admit.restype, lib.sb_sched_may_admit.argtypes = ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
            lib.sb_sched_plan.restype = ctypes.c_int
            lib.sb_sched_plan.argtypes = [ctypes.c_void_p, ctypes.c_int, _I32P, _I32P, _I32P, _U8P, _U8P, _I64P, ctypes.c_int, ctypes.c_int,
                                          _I32P, _I32P, ctypes.POINTER(ctypes.c_int32)]
            lib._sb_sched_typed = True
        self._buf = _PlanBuffers(max(self.opts.max_seqs, 1))

    # ------------------------------------------------------------------ intake
    def submit(self, request: GenRequest) -> None:
        """Thread-safe."""
        with self._mu:
            self._incoming.append(request)

    def idle(self) -> bool:
        with self._mu:
            return not (self._incoming or self._waiting or self._running)

    def _finish(self, seq: _Seq) -> None:
        seq.done = True
        if seq.slot >= 0:
            self.engine.cache.release_slot(seq.slot)
            seq.slot = -1

    def _admit(self) -> None:
        cache = self.engine.cache
        capacity = self.engine.max_context
        with self._mu:
            while self._incoming:
                seq = _Seq(self._incoming.popleft(), self._arrival)
                self._arrival += 1
                room = capacity - seq.prompt_len
                if room <= 0 or seq.prompt_len == 0:
                    if seq.req.on_token:
                        seq.req.on_token(TokenEvent(finished=True, finish_reason="empty_prompt" if seq.prompt_len == 0
                                                    else "context_length"), None)
                    continue
                seq.req.max_new_tokens = min(seq.req.max_new_tokens, room)
                self._waiting.append(seq)
        while self._waiting and len(self._running) < self.opts.max_seqs:
            nxt = self._waiting[0]
            if nxt.req.cancelled is not None and nxt.req.cancelled.is_set():
                self._waiting.popleft()
                continue
            # Room for its tokens and one page of growth per running request, and a free slot.
            if not self._lib.sb_sched_may_admit(cache._pool, len(self._running), len(nxt.tokens)):
                break
            slot = cache.acquire_slot()
            if slot < 0:
                break
            nxt.slot = slot
            nxt.next_pos = 0        # (re)computed from the first token: its pages were given back on preemption
            self._running.append(self._waiting.popleft())
        self.stats.peak_seqs = max(self.stats.peak_seqs, len(self._running))

    def _preempt(self, victim: _Seq) -> None:
        self.engine.cache.release_slot(victim.slot)
        victim.slot = -1
        self.stats.preemptions += 1
        self.stats.replayed_rows += victim.next_pos
        self._running.remove(victim)
        self._waiting.appendleft(victim)

    def _check_kernels(self, tokens) -> None:
        """The step's tokens are on the host. The sampling kernels report -1 - code instead of a token when a wait
        inside one of the step's tensor-core kernels gave up: that is an error, not a token."""
        worst = min((int(t) for t in tokens), default=0)
        if worst < 0:
            self.engine.check_kernels(-1 - worst)
            raise EngineError(f"the sampler returned {worst} instead of a token")

    # ------------------------------------------------------------------ planning
    def plan(self):
        """[(sequence, tokens to run)] for the next step, pages ensured; None if nothing is to run."""
        cache, buf = self.engine.cache, self._buf
        while True:
            n = len(self._running)
            if n == 0:
                return None
            run = self._running
            buf.slot[:n], buf.next_pos[:n], buf.total[:n] = [s.slot for s in run], [s.next_pos for s in run], [len(s.tokens) for s in run]
            buf.closing[:n], buf.inflight[:n] = [s.closing for s in run], [s.inflight > 0 for s in run]
            buf.arrival[:n] = [s.arrival for s in run]
            result = self._lib.sb_sched_plan(cache._pool, n, buf.slot_p, buf.next_pos_p, buf.total_p, buf.closing_p, buf.inflight_p,
                                             buf.arrival_p, self.opts.max_rows, self.opts.prefill_chunk, buf.out_index_p,
                                             buf.out_count_p, ctypes.byref(buf.out_n))
            if result == _PLAN_NOTHING:
                return None
            if result == _PLAN_DRAIN:
                return _DRAIN           # pages of a request with a step in flight cannot be taken away yet
            if result == _PLAN_TOO_SMALL:
                raise EngineError("the cache pool is too small for one sequence")
            if result == _PLAN_PREEMPT:
                self._preempt(self._running[int(buf.out_index[0])])     # the youngest; then plan again
                continue
            if result != _PLAN_RUN:
                raise EngineError(self._lib.sb_last_error().decode())
            m = buf.out_n.value
            plan = [(self._running[i], c) for i, c in zip(buf.out_index[:m].tolist(), buf.out_count[:m].tolist())]
            if self.opts.row_shuffle_seed:
                for i in range(len(plan) - 1, 0, -1):
                    self._rng_state = splitmix64(self._rng_state)
                    j = self._rng_state % (i + 1)
                    plan[i], plan[j] = plan[j], plan[i]
            return plan

    # ------------------------------------------------------------------ one step
    def step(self) -> bool:
        """Run one engine step. False when nothing is queued or running."""
        cache = self.engine.cache
        for s in list(self._running):
            if s.req.cancelled is not None and s.req.cancelled.is_set():
                cache.release_slot(s.slot)
                self._running.remove(s)
        self._admit()
        plan = self.plan()
        if plan is None:
            return False
        entries, wanted = [], []
        for s, count in plan:
            a = s.next_pos
            last = a + count == len(s.tokens)
            entries.append(StepEntry(slot=s.slot, first_pos=a, tokens=s.tokens[a:a + count], want=[count - 1] if last else []))
            if last:
                wanted.append(s)
            s.next_pos += count
        logits = self.engine.step(entries)
        self.stats.steps += 1
        self.stats.rows += sum(c for _, c in plan)
        used = max((t - f for t, f in zip(cache.total_pages(), cache.free_pages())), default=0)
        self.stats.peak_blocks = max(self.stats.peak_blocks, used)
        if wanted:
            tokens, values = self._sampler.choose(logits, [s.req.sampling for s in wanted], [len(s.tokens) for s in wanted])
            self._check_kernels(tokens)
            full = None
            if any(s.req.full_logits and s.req.on_token for s in wanted):
                full = logits.to("cpu").numpy()
            for i, s in enumerate(wanted):
                tok, val = int(tokens[i]), float(values[i])
                s.fingerprint = _fnv_mix(_fnv_mix(s.fingerprint, tok & 0xFFFFFFFF), _float_bits(val))
                s.tokens.append(tok)
                s.generated += 1
                self.stats.generated += 1
                ev = TokenEvent(token=tok, value=val, index=s.generated - 1, fingerprint=s.fingerprint)
                if tok in s.req.stop_tokens:
                    ev.finished, ev.finish_reason = True, "stop"
                elif s.generated >= s.req.max_new_tokens:
                    ev.finished, ev.finish_reason = True, "length"
                if s.req.on_token:
                    s.req.on_token(ev, full[i] if (full is not None and s.req.full_logits) else None)
                if ev.finished:
                    self._finish(s)
        for s in self._running:
            if not s.done:
                cache.trim(s.slot)
        self._running = [s for s in self._running if not s.done]
        return True

    # ------------------------------------------------------------------ pipelined running
    def _can_pipeline(self) -> bool:
        """Pipelining needs a sampler with `launch` / `collect` that leaves every row's token where the next step's
        embedding finds it (it says so with `pipelined = True`), and an engine that keeps such a table."""
        return bool(getattr(self._sampler, "pipelined", False)) and getattr(self.engine, "sampled", None) is not None

    def _launch(self):
        """Queue one step on the GPU without waiting for its tokens: rows whose input token is not known yet (it is
        being sampled by the step before) carry -1 and read it on the device. Returns a record for `_collect`, None
        when there is nothing to run, or _DRAIN when the steps in flight have to be read back first."""
        cache = self.engine.cache
        for s in list(self._running):
            if s.req.cancelled is not None and s.req.cancelled.is_set():
                if s.inflight:
                    return _DRAIN
                cache.release_slot(s.slot)
                self._running.remove(s)
        self._admit()
        plan = self.plan()
        if plan is None or plan is _DRAIN:
            return plan
        entries, wanted, ends = [], [], []
        for s, count in plan:
            a = s.next_pos
            last = a + count == len(s.tokens)
            entries.append(StepEntry(slot=s.slot, first_pos=a, tokens=s.tokens[a:a + count], want=[count - 1] if last else []))
            if last:
                wanted.append(s)
            s.next_pos += count
            ends.append((s, s.next_pos))
        pipelined = all(Sampler.on_device(s.req.sampling) and not s.req.full_logits for s in wanted)
        logits = self.engine.step(entries)
        self.stats.steps += 1
        self.stats.rows += sum(c for _, c in plan)
        used = max((t - f for t, f in zip(cache.total_pages(), cache.free_pages())), default=0)
        self.stats.peak_blocks = max(self.stats.peak_blocks, used)
        ticket, full = None, None
        if wanted:
            ticket = self._sampler.launch(logits, [s.req.sampling for s in wanted], [len(s.tokens) for s in wanted],
                                          self.engine.logit_slots, self.engine.sampled)
            if any(s.req.full_logits and s.req.on_token for s in wanted):
                full = logits.to("cpu").numpy()             # synchronises: such a step is not pipelined
            for s in wanted:
                s.tokens.append(-1)                          # stands for the token being sampled
                s.inflight += 1
                s.launched += 1
                if s.launched >= s.req.max_new_tokens:
                    s.closing = True                         # that token is its last ("length")
        return (wanted, ticket, full, ends, pipelined)

    def _collect(self, record) -> None:
        """Read back the tokens of a launched step and do the bookkeeping `step()` does after sampling."""
        wanted, ticket, full, ends, _ = record
        cache = self.engine.cache
        if ticket is not None:
            tokens, values = self._sampler.collect(ticket)
            self._check_kernels(tokens)
            for i, s in enumerate(wanted):
                s.inflight -= 1
                if s.done:                                   # finished by a stop token a step ago: this row was surplus
                    if s.inflight == 0 and s.slot >= 0:
                        self._finish(s)
                    continue
                tok, val = int(tokens[i]), float(values[i])
                s.fingerprint = _fnv_mix(_fnv_mix(s.fingerprint, tok & 0xFFFFFFFF), _float_bits(val))
                s.tokens[s.prompt_len + s.generated] = tok   # the oldest placeholder
                s.generated += 1
                self.stats.generated += 1
                ev = TokenEvent(token=tok, value=val, index=s.generated - 1, fingerprint=s.fingerprint)
                if tok in s.req.stop_tokens:
                    ev.finished, ev.finish_reason = True, "stop"
                elif s.generated >= s.req.max_new_tokens:
                    ev.finished, ev.finish_reason = True, "length"
                if s.req.on_token:
                    s.req.on_token(ev, full[i] if (full is not None and s.req.full_logits) else None)
                if ev.finished:
                    s.done = s.closing = True
                    if s.inflight == 0:
                        self._finish(s)                      # else its slot is given back when the surplus step is read
        windowed = any(g.window > 0 for g in cache.groups)
        if ticket is None and windowed and getattr(self.engine, "device", None) is not None and str(self.engine.device) != "cpu":
            import torch
            torch.cuda.current_stream().synchronize()      # pages are only given back once the step has run
        if windowed:
            for s, end in ends:
                if s.slot >= 0 and not s.done:
                    cache.trim(s.slot, end)
        self._running = [s for s in self._running if not (s.done and s.slot < 0)]

    def run(self, steps: Optional[int] = None) -> int:
        """Run until nothing is queued or running, or for `steps` engine steps. With a GPU engine the next step is
        queued before the tokens of the current one are read (see `_launch`), so the host's work per step overlaps
        the GPU's. Returns the number of steps run."""
        if not self._can_pipeline():
            n = 0
            while (steps is None or n < steps) and self.step():
                n += 1
            return n
        n, pending = 0, None
        while True:
            launched = None
            if steps is None or n < steps:
                launched = self._launch()
                if launched is _DRAIN:
                    if pending is None:
                        raise EngineError("the scheduler asked to drain an empty pipeline")
                    self._collect(pending)
                    pending = None
                    continue
            if launched is None and pending is None:
                return n
            if launched is not None:
                n += 1
                if not launched[4]:                          # a step that needs its logits on the host: no overlap
                    if pending is not None:
                        self._collect(pending)
                        pending = None
                    self._collect(launched)
                    continue
            if pending is not None:
                self._collect(pending)
            pending = launched
