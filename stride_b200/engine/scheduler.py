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

The requests' tokens and state, admission, the plan under the budget with its page
arithmetic and preemption, and what a chosen token means for its request (stop token, length,
fingerprint) live in the native `Sched` of `csrc/runtime.cpp`, on the books of the native page
pool; this module keeps what cannot live there (callbacks, sampling parameters, cancellation
flags) and drives the engine and the sampler, one step ahead of the tokens where it can.

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

from ..sampling.sampler import Sampler, SamplingParams
from .engine import Engine, EngineError, StepEntry

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


_DRAIN = object()      # the steps in flight have to be read back before a decision can be taken
_PLAN_RUN, _PLAN_NOTHING, _PLAN_DRAIN, _PLAN_TOO_SMALL, _PLAN_PREEMPT = range(5)    # results of the native planner
_I32P, _U8P, _I64P = ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_int64)
_U64P, _F32P = ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_float)
_FINISH = {2: "stop", 3: "length"}


class _Buffers:
    """Named numpy arrays with their ctypes pointers (`name_p`)."""
    POINTERS = {np.int32: _I32P, np.uint8: _U8P, np.int64: _I64P, np.uint64: _U64P, np.float32: _F32P}

    def __init__(self, capacity: int, fields):
        self.capacity = capacity
        for name, dtype in fields:
            arr = np.zeros(capacity, dtype=dtype)
            setattr(self, name, arr)
            setattr(self, name + "_p", arr.ctypes.data_as(self.POINTERS[dtype]))


class _PlanBuffers(_Buffers):
    """Arrays the native planner `sb_sched_plan` reads (one row per running request) and writes (the plan)."""

    def __init__(self, capacity: int):
        super().__init__(capacity, (("slot", np.int32), ("next_pos", np.int32), ("total", np.int32), ("closing", np.uint8),
                                    ("inflight", np.uint8), ("arrival", np.int64), ("out_index", np.int32), ("out_count", np.int32)))
        self.out_n = ctypes.c_int32(0)


def native_scheduler(lib):
    """The runtime library with the scheduler's functions typed."""
    if not getattr(lib, "_sb_sched_typed", False):
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.sb_sched_may_admit.restype, lib.sb_sched_may_admit.argtypes = ci, [vp, ci, ci]
        lib.sb_sched_plan.restype = ci
        lib.sb_sched_plan.argtypes = [vp, ci, _I32P, _I32P, _I32P, _U8P, _U8P, _I64P, ci, ci, _I32P, _I32P, ctypes.POINTER(ctypes.c_int32)]
        lib.sb_sched_create.restype, lib.sb_sched_create.argtypes = vp, [vp, ci, ci, ci, ci, ctypes.c_uint64]
        lib.sb_sched_destroy.restype, lib.sb_sched_destroy.argtypes = None, [vp]
        lib.sb_sched_add.restype, lib.sb_sched_add.argtypes = ci, [vp, _I32P, ci, ci, _I32P, ci]
        lib.sb_sched_cancel.restype, lib.sb_sched_cancel.argtypes = None, [vp, ci]
        lib.sb_sched_counts.restype, lib.sb_sched_counts.argtypes = None, [vp, _I32P]
        lib.sb_sched_queue.restype, lib.sb_sched_queue.argtypes = ci, [vp, ci, _I32P, ci]
        lib.sb_sched_stats.restype, lib.sb_sched_stats.argtypes = None, [vp, _I64P]
        lib.sb_sched_begin_step.restype = ci
        lib.sb_sched_begin_step.argtypes = [vp, _I32P, _I32P, _I32P, _I32P, _U8P, _I32P, ctypes.POINTER(ctypes.c_int32)]
        lib.sb_sched_launched.restype, lib.sb_sched_launched.argtypes = None, [vp, _I32P, ci]
        lib.sb_sched_commit.restype = None
        lib.sb_sched_commit.argtypes = [vp, ci, _I32P, _I32P, _F32P, ci, _U8P, _I32P, _U64P]
        lib.sb_sched_end_step.restype, lib.sb_sched_end_step.argtypes = None, [vp, _I32P, _I32P, ci]
        lib.sb_sched_abort.restype, lib.sb_sched_abort.argtypes = None, [vp]
        lib._sb_sched_typed = True
    return lib


class Scheduler:
    def __init__(self, engine: Engine, options: Optional[SchedulerOptions] = None, sampler=None):
        self.engine = engine
        self.opts = options or SchedulerOptions()
        if self.opts.max_rows > engine.options.max_rows:
            raise EngineError(f"scheduler max_rows {self.opts.max_rows} exceeds the engine's {engine.options.max_rows}")
        self._mu = threading.Lock()
        self._incoming: deque = deque()
        self._requests: dict = {}          # native id -> GenRequest of every request that waits or runs
        self._sampler = sampler or Sampler(engine.device, engine.env.max_logit_rows)
        self._lib = native_scheduler(engine.cache._lib)
        self._sched = self._lib.sb_sched_create(engine.cache._pool, self.opts.max_seqs, self.opts.max_rows, self.opts.prefill_chunk,
                                                engine.max_context, self.opts.row_shuffle_seed)
        if not self._sched:
            raise EngineError(self._lib.sb_last_error().decode())
        rows = max(self.opts.max_rows, 1)
        self._plan = _Buffers(rows, (("id", np.int32), ("slot", np.int32), ("first", np.int32), ("count", np.int32), ("last", np.uint8),
                                     ("tokens", np.int32), ("n_want", np.int32), ("want", np.int32)))
        self._plan_n = ctypes.c_int32(0)
        self._rows = _Buffers(rows, (("id", np.int32), ("token", np.int32), ("value", np.float32), ("kind", np.uint8), ("index", np.int32),
                                     ("fingerprint", np.uint64), ("end", np.int32)))
        self._counts = np.zeros(2, dtype=np.int32)
        self._stats = np.zeros(7, dtype=np.int64)

    def __del__(self):
        sched, self._sched = getattr(self, "_sched", None), None
        if sched:
            self._lib.sb_sched_destroy(sched)

    # ------------------------------------------------------------------ intake and views
    def submit(self, request: GenRequest) -> None:
        """Thread-safe."""
        with self._mu:
            self._incoming.append(request)

    def idle(self) -> bool:
        with self._mu:
            if self._incoming:
                return False
        self._lib.sb_sched_counts(self._sched, self._counts.ctypes.data_as(_I32P))
        return not self._counts.any()

    @property
    def stats(self) -> SchedulerStats:
        self._lib.sb_sched_stats(self._sched, self._stats.ctypes.data_as(_I64P))
        return SchedulerStats(*(int(v) for v in self._stats))

    def _queue(self, which: int) -> list:
        buf = np.zeros(self.opts.max_seqs + len(self._requests) + 1, dtype=np.int32)
        n = self._lib.sb_sched_queue(self._sched, which, buf.ctypes.data_as(_I32P), buf.size)
        return buf[:n].tolist()

    @property
    def _waiting(self) -> list:
        """Ids of the requests that wait, the next to be admitted first."""
        return self._queue(0)

    @property
    def _running(self) -> list:
        """Ids of the requests that run, in the order of admission."""
        return self._queue(1)

    def _intake(self) -> None:
        """Hands new requests to the native scheduler and tells it which requests were cancelled."""
        with self._mu:
            incoming, self._incoming = list(self._incoming), deque()
        for req in incoming:
            prompt = np.asarray(req.prompt, dtype=np.int32).reshape(-1)
            stops = np.asarray(tuple(req.stop_tokens), dtype=np.int32).reshape(-1)
            rid = self._lib.sb_sched_add(self._sched, prompt.ctypes.data_as(_I32P), prompt.size, int(req.max_new_tokens),
                                         stops.ctypes.data_as(_I32P), stops.size)
            if rid < 0:
                if req.on_token:
                    req.on_token(TokenEvent(finished=True, finish_reason="empty_prompt" if rid == -1 else "context_length"), None)
                continue
            self._requests[rid] = req
        for rid, req in list(self._requests.items()):
            if req.cancelled is not None and req.cancelled.is_set():
                self._lib.sb_sched_cancel(self._sched, rid)
                del self._requests[rid]

    # ------------------------------------------------------------------ the parts of a step
    def _begin(self):
        """The next step, or None (nothing to run) or _DRAIN: (a call that runs it on the engine and returns its logits,
        ids of the requests a token is to be chosen for, the tokens each of those has before the new one, (ids, positions
        reached) of all requests in the step)."""
        self._intake()
        p = self._plan
        result = self._lib.sb_sched_begin_step(self._sched, p.id_p, p.slot_p, p.first_p, p.count_p, p.last_p, p.tokens_p,
                                               ctypes.byref(self._plan_n))
        if result == _PLAN_NOTHING:
            return None
        if result == _PLAN_DRAIN:
            return _DRAIN
        if result == _PLAN_TOO_SMALL:
            raise EngineError("the cache pool is too small for one sequence")
        if result != _PLAN_RUN:
            raise EngineError(self._lib.sb_last_error().decode())
        m = self._plan_n.value
        ids, firsts, counts, lasts = (a[:m].tolist() for a in (p.id, p.first, p.count, p.last))
        wanted = [rid for rid, last in zip(ids, lasts) if last]
        lengths = [f + c for f, c, last in zip(firsts, counts, lasts) if last]     # tokens each has before the new one
        ends = (ids, [f + c for f, c in zip(firsts, counts)])
        if hasattr(self.engine, "step_arrays"):
            # the plan goes to the engine as the arrays it is: the native stager reads them
            p.n_want[:m] = p.last[:m]
            k = len(wanted)
            p.want[:k] = (p.count[:m] - 1)[p.last[:m] != 0]
            return (lambda: self.engine.step_arrays(m, p.slot, p.first, p.count, p.tokens, p.n_want, p.want)), wanted, lengths, ends
        slots, tokens = p.slot[:m].tolist(), p.tokens[:sum(counts)].tolist()
        entries, at = [], 0
        for slot, first, count, last in zip(slots, firsts, counts, lasts):
            entries.append(StepEntry(slot=slot, first_pos=first, tokens=tokens[at:at + count], want=[count - 1] if last else []))
            at += count
        return (lambda: self.engine.step(entries)), wanted, lengths, ends

    def _commit(self, ahead: bool, wanted: list, tokens, values, full) -> None:
        """Hands the chosen tokens to the native scheduler and tells the requests what it made of them."""
        n = len(wanted)
        worst = min((int(t) for t in tokens), default=0)
        if worst < 0:
            # the sampling kernels report -1 - code instead of a token when a wait inside one of the step's tensor-core
            # kernels gave up: that is an error, not a token
            self.engine.check_kernels(-1 - worst)
            raise EngineError(f"the sampler returned {worst} instead of a token")
        r = self._rows
        r.id[:n], r.token[:n], r.value[:n] = wanted, tokens, values
        self._lib.sb_sched_commit(self._sched, 1 if ahead else 0, r.id_p, r.token_p, r.value_p, n, r.kind_p, r.index_p, r.fingerprint_p)
        kinds, indices, prints = r.kind[:n].tolist(), r.index[:n].tolist(), r.fingerprint[:n].tolist()
        for i, rid in enumerate(wanted):
            kind = kinds[i]
            req = self._requests.get(rid)
            if kind == 0 or req is None:          # a surplus row, or a request that was cancelled meanwhile
                continue
            if kind >= 2:
                del self._requests[rid]
            if req.on_token:
                ev = TokenEvent(token=int(tokens[i]), value=float(values[i]), index=indices[i], fingerprint=prints[i],
                                finished=kind >= 2, finish_reason=_FINISH.get(kind))
                req.on_token(ev, full[i] if (full is not None and req.full_logits) else None)

    def _end(self, ends, whole: bool) -> None:
        ids, positions = ends
        n = len(ids)
        r = self._rows
        r.id[:n] = ids
        r.end[:n] = -1 if whole else positions
        self._lib.sb_sched_end_step(self._sched, r.id_p, r.end_p, n)

    def _full_logits(self, wanted: list, logits):
        if any(self._requests[rid].full_logits and self._requests[rid].on_token for rid in wanted if rid in self._requests):
            return logits.to("cpu").numpy()
        return None

    # ------------------------------------------------------------------ one step
    def step(self) -> bool:
        """Run one engine step and wait for its tokens. False when nothing is queued or running."""
        begun = self._begin()
        if begun is None:
            return False
        if begun is _DRAIN:
            raise EngineError("the scheduler asked to drain an empty pipeline")
        run_step, wanted, lengths, ends = begun
        logits = run_step()
        if wanted:
            reqs = [self._requests[rid] for rid in wanted]
            tokens, values = self._sampler.choose(logits, [q.sampling for q in reqs], lengths)
            self._commit(False, wanted, tokens, values, self._full_logits(wanted, logits))
        self._end(ends, whole=True)
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
        begun = self._begin()
        if begun is None or begun is _DRAIN:
            return begun
        run_step, wanted, lengths, ends = begun
        logits = run_step()
        ticket, full, pipelined = None, None, True
        if wanted:
            reqs = [self._requests[rid] for rid in wanted]
            pipelined = all(Sampler.on_device(q.sampling) and not q.full_logits for q in reqs)
            ticket = self._sampler.launch(logits, [q.sampling for q in reqs], lengths, self.engine.logit_slots, self.engine.sampled)
            full = self._full_logits(wanted, logits)             # synchronises: such a step is not pipelined
            ids = np.asarray(wanted, dtype=np.int32)
            self._lib.sb_sched_launched(self._sched, ids.ctypes.data_as(_I32P), ids.size)
        return (wanted, ticket, full, ends, pipelined)

    def _collect(self, record) -> None:
        """Read back the tokens of a launched step and do the bookkeeping `step()` does after sampling."""
        wanted, ticket, full, ends, _ = record
        if ticket is not None:
            tokens, values = self._sampler.collect(ticket)
            self._commit(True, wanted, tokens, values, full)
        elif any(g.window > 0 for g in self.engine.cache.groups) and str(getattr(self.engine, "device", "cpu")) != "cpu":
            import torch
            torch.cuda.current_stream().synchronize()      # pages are only given back once the step has run
        self._end(ends, whole=False)

    def abort(self) -> None:
        """Give up every request (no callbacks): slots and pages go back to the cache, the queues are empty. Waits for
        the GPU first, since steps may still be running on pages that are about to be handed out again."""
        if str(getattr(self.engine, "device", "cpu")) != "cpu":
            import torch
            try:
                torch.cuda.synchronize()
            except RuntimeError:
                pass
        with self._mu:
            self._incoming.clear()
        self._requests.clear()
        self._lib.sb_sched_abort(self._sched)

    def run(self, steps: Optional[int] = None) -> int:
        """Run until nothing is queued or running, or for `steps` engine steps. With a GPU engine the next step is
        queued before the tokens of the current one are read (see `_launch`), so the host's work per step overlaps
        the GPU's. Returns the number of steps run. An error on the way (from the engine, the sampler or a callback)
        aborts all requests before it is passed on, so that the engine's cache is left as it was found."""
        try:
            return self._run(steps)
        except BaseException:
            self.abort()
            raise

    def _run(self, steps: Optional[int]) -> int:
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
