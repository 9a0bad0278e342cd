"""The scheduler's decisions on the CPU, against a fake engine whose "model" is a hash of the tokens a
slot has been fed: any token fed twice, skipped, or at a wrong position changes what is generated."""
from __future__ import annotations

import ctypes
import hashlib
import threading
from types import SimpleNamespace

import pytest
import torch

from stride_b200.cache.manager import CacheManager
from stride_b200.engine.engine import EngineError
from stride_b200.engine.scheduler import GenRequest, Scheduler, SchedulerOptions
from stride_b200.parts import CacheNeed
from stride_b200.sampling.sampler import SamplingParams

VOCAB = 97


class FakeEngine:
    def __init__(self, pages=64, page_size=4, max_slots=8, max_rows=16, max_context=64):
        need = CacheNeed("pages", kv_heads=1, head_dim=2, dtype=torch.float32)
        self.cache = CacheManager([need], device="cpu", max_slots=max_slots, max_context=max_context, page_size=page_size, num_pages=pages)
        self.options = SimpleNamespace(max_rows=max_rows)
        self.env = SimpleNamespace(max_logit_rows=max_rows)
        self.spec = SimpleNamespace(eos_token_ids=(), vocab_size=VOCAB)
        self.max_context = max_context
        self.device = "cpu"
        self.fed = {}              # slot -> tokens fed so far
        self.batches = []          # per step: [(slot, first_pos, n tokens, wants logits)]

    def step(self, entries):
        assert sum(len(e.tokens) for e in entries) <= self.options.max_rows
        out = []
        self.batches.append([(e.slot, e.first_pos, len(e.tokens), bool(e.want)) for e in entries])
        for e in entries:
            seq = self.fed.setdefault(e.slot, [])
            if e.first_pos == 0:
                seq.clear()                       # a (re)started request
            assert e.first_pos == len(seq), "tokens must continue the slot's sequence"
            assert self.cache.length[e.slot] >= e.first_pos + len(e.tokens), "pages must be ensured"
            seq.extend(e.tokens)
            for j in e.want:
                assert j == len(e.tokens) - 1
                out.append(list(seq))
        return out or None


class HashSampler:
    def choose(self, logits, params, lengths):
        toks = []
        for seq, n in zip(logits, lengths):
            assert len(seq) == n
            toks.append(int.from_bytes(hashlib.sha256(repr(seq).encode()).digest()[:4], "little") % VOCAB)
        return toks, [float(t) for t in toks]


def _run(engine, prompts, max_new=12, opts=None, stops=()):
    sched = Scheduler(engine, opts or SchedulerOptions(max_seqs=8, max_rows=16, prefill_chunk=5), sampler=HashSampler())
    outs = [dict(tokens=[], finish=None) for _ in prompts]

    def cb(i):
        def on_token(ev, logits):
            if ev.token >= 0:
                assert ev.index == len(outs[i]["tokens"])
                outs[i]["tokens"].append(ev.token)
            if ev.finished:
                outs[i]["finish"] = ev.finish_reason
        return on_token
    for i, p in enumerate(prompts):
        sched.submit(GenRequest(prompt=p, max_new_tokens=max_new, stop_tokens=stops, on_token=cb(i)))
    sched.run()
    assert sched.idle()
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()
    return outs, sched


PROMPTS = [[1, 2, 3, 4, 5, 6, 7], [9], [11, 12, 13], list(range(20, 33)), [40, 41], [50, 51, 52, 53, 54, 55]]


def _solo():
    return [_run(FakeEngine(), [p])[0][0] for p in PROMPTS]


def test_batches_obey_budget_order_and_chunking():
    eng = FakeEngine()
    outs, sched = _run(eng, PROMPTS)
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in _solo()]
    assert all(o["finish"] == "length" and len(o["tokens"]) == 12 for o in outs)
    for batch in eng.batches:
        assert sum(n for _, _, n, _ in batch) <= 16
        kinds = [n == 1 and want for _, _, n, want in batch]
        # decode rows come first, portions after them, none longer than prefill_chunk
        assert kinds == sorted(kinds, reverse=True) or all(n <= 5 for _, _, n, _ in batch)
        assert all(n <= 5 for _, _, n, _ in batch)
    # the 13-token prompt was cut into 5 + 5 + 3 and only the last portion asked for logits
    slot13 = [b for batch in eng.batches for b in batch if b[1] in (0, 5, 10) and b[2] in (5, 3)]
    assert sched.stats.generated == 72 and sched.stats.preemptions == 0 and sched.stats.peak_seqs == 6
    assert sched.stats.rows == sum(n for batch in eng.batches for _, _, n, _ in batch)


def test_running_out_of_pages_preempts_the_youngest_and_replays():
    solo = _solo()
    eng = FakeEngine(pages=9, page_size=4)              # 36 tokens of cache for requests that grow to 7+12, 13+12, ...
    outs, sched = _run(eng, PROMPTS, opts=SchedulerOptions(max_seqs=6, max_rows=16, prefill_chunk=5))
    assert sched.stats.preemptions > 0 and sched.stats.replayed_rows > 0
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in solo]
    assert sched.stats.peak_blocks <= 9
    # a restarted request begins again at position 0 with a portion, never in the middle
    restarts = [b for batch in eng.batches for b in batch if b[1] == 0]
    # (a request preempted before it ever ran restarts nothing)
    assert len(PROMPTS) < len(restarts) <= len(PROMPTS) + sched.stats.preemptions


def test_a_single_request_that_cannot_fit_raises():
    eng = FakeEngine(pages=3, page_size=4)
    sched = Scheduler(eng, SchedulerOptions(max_seqs=2, max_rows=16, prefill_chunk=16), sampler=HashSampler())
    sched.submit(GenRequest(prompt=list(range(10)), max_new_tokens=20))
    with pytest.raises(EngineError, match="too small for one sequence"):
        sched.run()


def test_admission_keeps_room_for_growth():
    eng = FakeEngine(pages=8, page_size=4, max_rows=32)
    sched = Scheduler(eng, SchedulerOptions(max_seqs=8, max_rows=32, prefill_chunk=16), sampler=HashSampler())
    for p in ([1] * 12, [2] * 8):
        sched.submit(GenRequest(prompt=p, max_new_tokens=3))
    sched.step()                                  # both admitted and prefilled: 3 + 2 pages held, 3 free
    assert len(sched._running) == 2 and eng.cache.free_pages() == [3]
    sched.submit(GenRequest(prompt=[3] * 4, max_new_tokens=3))
    sched.step()
    # the third needs 1 page + one page of growth for each of the 2 running + 1 = 4 > 3 free: it waits
    assert len(sched._running) == 2 and len(sched._waiting) == 1
    sched.run()
    assert sched.stats.generated == 9 and sched.stats.preemptions == 0


def test_stop_tokens_limits_and_cancellation():
    solo = _solo()
    stop = solo[0]["tokens"][4]
    outs, _ = _run(FakeEngine(), [PROMPTS[0]], stops=(stop,))
    k = solo[0]["tokens"].index(stop)
    assert outs[0]["tokens"] == solo[0]["tokens"][:k + 1] and outs[0]["finish"] == "stop"
    eng = FakeEngine(max_context=16)
    outs, _ = _run(eng, [[], list(range(16)), list(range(10))], max_new=50)
    assert (outs[0]["finish"], outs[1]["finish"]) == ("empty_prompt", "context_length")
    assert outs[2]["finish"] == "length" and len(outs[2]["tokens"]) == 6          # clamped to the room left
    eng = FakeEngine()
    sched = Scheduler(eng, SchedulerOptions(max_seqs=4, max_rows=16, prefill_chunk=8), sampler=HashSampler())
    flag = threading.Event()
    got = []
    sched.submit(GenRequest(prompt=[1, 2, 3], max_new_tokens=100, cancelled=flag, on_token=lambda ev, l: got.append(ev.token)))
    sched.submit(GenRequest(prompt=[4, 5], max_new_tokens=5))
    for _ in range(4):
        sched.step()
    flag.set()
    sched.run()
    assert 0 < len(got) < 100 and sched.idle()
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_batch_order_shuffle_changes_nothing():
    solo = _solo()
    outs, _ = _run(FakeEngine(), PROMPTS, opts=SchedulerOptions(max_seqs=4, max_rows=9, prefill_chunk=3, row_shuffle_seed=5))
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in solo]


@pytest.mark.parametrize("seed", range(8))
def test_native_planner_decisions_under_random_states(seed):
    """The planner in csrc/runtime.cpp against its rules restated here, over random sets of running requests: decoded
    tokens first, then portions in running order, under the budget; pages ensured when it says run; the youngest named
    when pages are short; drain while a step is in flight; too small when one request alone does not fit."""
    import ctypes
    import random

    import numpy as np
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    eng = FakeEngine(pages=rng.choice([6, 12, 40]), page_size=page, max_slots=8, max_rows=64, max_context=64)
    sched = Scheduler(eng, SchedulerOptions(max_seqs=8, max_rows=rng.choice([4, 9, 32]), prefill_chunk=rng.choice([2, 5, 16])),
                      sampler=HashSampler())
    from stride_b200.engine.scheduler import _PlanBuffers
    cache, lib, buf = eng.cache, sched._lib, _PlanBuffers(8)
    for _ in range(60):
        while cache.live_slots:
            cache.release_slot(next(iter(cache.live_slots)))
        n = rng.randint(1, 6)
        slots = [cache.acquire_slot() for _ in range(n)]
        total = [rng.randint(1, 40) for _ in range(n)]
        nxt = []
        for s, t in zip(slots, total):
            done = rng.choice([0, 0, t - 1, rng.randint(0, t - 1)])
            if not cache.ensure(s, done):
                done = 0
            nxt.append(done)
        closing = [rng.random() < 0.15 for _ in range(n)]
        inflight = [rng.random() < 0.1 for _ in range(n)]
        arrival = rng.sample(range(100), n)
        buf.slot[:n], buf.next_pos[:n], buf.total[:n] = slots, nxt, total
        buf.closing[:n], buf.inflight[:n], buf.arrival[:n] = closing, inflight, arrival
        free_before = cache.free_pages()[0]
        held = {i: -(-int(cache.length[slots[i]]) // page) for i in range(n)}      # pages each request has
        result = lib.sb_sched_plan(cache._pool, n, buf.slot_p, buf.next_pos_p, buf.total_p, buf.closing_p, buf.inflight_p,
                                   buf.arrival_p, sched.opts.max_rows, sched.opts.prefill_chunk, buf.out_index_p,
                                   buf.out_count_p, ctypes.byref(buf.out_n))
        # the rules, restated
        budget, want = sched.opts.max_rows, []
        for i in range(n):
            if total[i] - nxt[i] == 1 and not closing[i] and budget > 0:
                want.append((i, 1))
                budget -= 1
        for i in range(n):
            rem = total[i] - nxt[i]
            if rem > 1 and not closing[i] and budget > 0:
                c = min(rem, sched.opts.prefill_chunk, budget)
                want.append((i, c))
                budget -= c
        need = sum(max(0, -(-(nxt[i] + c) // page) - held[i]) for i, c in want)
        if not want:
            assert result == 1
        elif need > free_before:
            if any(inflight):
                assert result == 2
            elif n <= 1:
                assert result == 3
            else:
                assert result == 4 and int(buf.out_index[0]) == max(range(n), key=lambda i: arrival[i])
            assert cache.free_pages()[0] == free_before          # nothing was taken
        else:
            m = buf.out_n.value
            assert result == 0 and list(zip(buf.out_index[:m].tolist(), buf.out_count[:m].tolist())) == want
            assert cache.free_pages()[0] == free_before - need
            assert all(cache.length[slots[i]] >= nxt[i] + c for i, c in want)
        cache.check()


# ---------------------------------------------------------------------------- one step ahead
class PipeEngine(FakeEngine):
    """The fake engine with what running a step ahead needs: a table of every slot's last chosen token, which a row
    whose token is still being chosen (-1) reads, as the embedding kernel does on the device."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.sampled = {}
        self.logit_slots = []
        self.placeholders = 0

    def step(self, entries):
        fixed = []
        for e in entries:
            tokens = list(e.tokens)
            if tokens == [-1]:
                tokens = [self.sampled[e.slot]]
                self.placeholders += 1
            assert all(t >= 0 for t in tokens), "only a single decoded token may be a placeholder"
            fixed.append(SimpleNamespace(slot=e.slot, first_pos=e.first_pos, tokens=tokens, want=e.want))
        self.logit_slots = [e.slot for e in fixed for _ in e.want]
        return super().step(fixed)


class PipeSampler(HashSampler):
    pipelined = True

    def launch(self, logits, params, lengths, scatter_index=None, scatter=None):
        tokens, values = self.choose(logits, params, lengths)
        if scatter is not None:
            for slot, t in zip(scatter_index, tokens):
                scatter[slot] = t
        return tokens, values

    def collect(self, ticket):
        return ticket


def _run_ahead(engine, prompts, max_new=12, opts=None, stops=()):
    sched = Scheduler(engine, opts or SchedulerOptions(max_seqs=8, max_rows=16, prefill_chunk=5), sampler=PipeSampler())
    assert sched._can_pipeline()
    outs = [dict(tokens=[], finish=None) for _ in prompts]

    def cb(i):
        def on_token(ev, logits):
            if ev.token >= 0:
                assert ev.index == len(outs[i]["tokens"])
                outs[i]["tokens"].append(ev.token)
            if ev.finished:
                assert outs[i]["finish"] is None
                outs[i]["finish"] = ev.finish_reason
        return on_token
    for i, p in enumerate(prompts):
        sched.submit(GenRequest(prompt=p, max_new_tokens=max_new, stop_tokens=stops, on_token=cb(i)))
    sched.run()
    assert sched.idle()
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()
    return outs, sched


def test_a_step_ahead_gives_the_same_tokens():
    """The scheduler queues step N + 1 before it has read step N's tokens (rows carry -1 and read the token from the
    engine's table): same tokens, same finishes, every slot and page given back."""
    solo = _solo()
    eng = PipeEngine()
    outs, sched = _run_ahead(eng, PROMPTS)
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in solo]
    assert all(o["finish"] == "length" for o in outs) and eng.placeholders > 0
    assert sched.stats.generated == 72
    outs, _ = _run_ahead(PipeEngine(), PROMPTS, opts=SchedulerOptions(max_seqs=4, max_rows=9, prefill_chunk=3, row_shuffle_seed=5))
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in solo]


def test_a_step_ahead_with_stop_tokens_and_short_pools():
    solo = _solo()
    # a stop token ends a request whose next row is already queued: that surplus row changes nothing
    for which in (0, 3, 5):
        stop = solo[which]["tokens"][4]
        outs, _ = _run_ahead(PipeEngine(), PROMPTS, stops=(stop,))
        for o, s in zip(outs, solo):
            want = s["tokens"][:s["tokens"].index(stop) + 1] if stop in s["tokens"] else s["tokens"]
            assert o["tokens"] == want and o["finish"] == ("stop" if stop in s["tokens"] else "length")
    # pages run out: steps in flight are read back first, then the youngest is preempted and replayed
    eng = PipeEngine(pages=9, page_size=4)
    outs, sched = _run_ahead(eng, PROMPTS, opts=SchedulerOptions(max_seqs=6, max_rows=16, prefill_chunk=5))
    assert sched.stats.preemptions > 0
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in solo]
    with pytest.raises(EngineError, match="too small for one sequence"):
        _run_ahead(PipeEngine(pages=3, page_size=4), [list(range(10))], max_new=20, opts=SchedulerOptions(max_seqs=2, max_rows=16, prefill_chunk=16))


def test_a_step_ahead_with_cancellation():
    eng = PipeEngine()
    sched = Scheduler(eng, SchedulerOptions(max_seqs=4, max_rows=16, prefill_chunk=8), sampler=PipeSampler())
    flag = threading.Event()
    got, other = [], []
    sched.submit(GenRequest(prompt=[1, 2, 3], max_new_tokens=100, cancelled=flag, on_token=lambda ev, l: got.append(ev.token)))
    sched.submit(GenRequest(prompt=[4, 5], max_new_tokens=30, on_token=lambda ev, l: other.append(ev.token)))
    sched.run(steps=6)
    flag.set()
    sched.run()
    assert 0 < len(got) < 100 and len(other) == 30 and sched.idle()
    assert other == _run(FakeEngine(), [[4, 5]], max_new=30)[0][0]["tokens"]
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_fingerprints_are_fnv1a_over_tokens_and_logit_bits():
    """arhaamatiq/stride's request fingerprint (src/scheduler.cpp:26-31): FNV-1a over the four bytes of every chosen
    token and the four bytes of its float32 logit, in order."""
    import struct
    seen = []
    sched = Scheduler(FakeEngine(), SchedulerOptions(max_seqs=2, max_rows=16, prefill_chunk=8), sampler=HashSampler())
    sched.submit(GenRequest(prompt=[3, 1, 4, 1, 5], max_new_tokens=6, on_token=lambda ev, l: seen.append(ev)))
    sched.run()
    h = 14695981039346656037
    for ev in seen:
        for word in (ev.token & 0xFFFFFFFF, struct.unpack("<I", struct.pack("<f", ev.value))[0]):
            for i in range(4):
                h = ((h ^ ((word >> (8 * i)) & 0xFF)) * 1099511628211) & ((1 << 64) - 1)
        assert ev.fingerprint == h
    assert [ev.index for ev in seen] == list(range(6)) and seen[-1].finished and seen[-1].finish_reason == "length"


def test_request_ids_are_used_again_and_waiting_requests_can_be_cancelled():
    """Many more requests than ever run at once go through two slots; a request cancelled while it waits never runs;
    the native table of requests is as large as the most requests known at once, however many are served."""
    eng = FakeEngine(max_slots=2)
    sched = Scheduler(eng, SchedulerOptions(max_seqs=2, max_rows=8, prefill_chunk=4), sampler=HashSampler())
    done, flags = {}, {}
    for i in range(40):
        flags[i] = threading.Event()
        sched.submit(GenRequest(prompt=[i + 1, 2, 3], max_new_tokens=3, cancelled=flags[i],
                                on_token=lambda ev, l, i=i: done.setdefault(i, []).append(ev.token)))
    for i in (5, 6, 39):
        flags[i].set()                       # they still wait: cancelled before they ever run
    sched.run()
    assert sched.idle() and not sched._requests
    assert sorted(done) == [i for i in range(40) if i not in (5, 6, 39)] and all(len(v) == 3 for v in done.values())
    assert max(sched._lib.sb_sched_add(sched._sched, None, 0, 1, None, 0) for _ in range(1)) == -1     # an empty prompt is refused
    for i, toks in done.items():
        assert toks == _run(FakeEngine(), [[i + 1, 2, 3]], max_new=3)[0][0]["tokens"]
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages() and len(eng.cache.free_slots) == 2
    # forty requests were known at once, so forty ids exist; whoever comes later gets one of them again
    later = [sched._lib.sb_sched_add(sched._sched, (ctypes.c_int32 * 2)(7, 8), 2, 1, None, 0) for _ in range(40)]
    assert sorted(later) == list(range(40))


@pytest.mark.parametrize("ahead", [False, True])
def test_windowed_groups_give_pages_back_while_requests_run(ahead):
    """With a window of 8 keys a request of 5 + 40 tokens never holds more than a few pages of 4, waited for or a step
    ahead; the tokens are those of a pool without a window (the fake model does not look at the cache)."""
    class Windowed(PipeEngine if ahead else FakeEngine):
        def __init__(self):
            super().__init__(pages=12, page_size=4)
            need = CacheNeed("pages", kv_heads=1, head_dim=2, window=8, dtype=torch.float32)
            self.cache = CacheManager([need], device="cpu", max_slots=8, max_context=64, page_size=4, num_pages=12)
            self.most = 0

        def step(self, entries):
            out = super().step(entries)
            self.most = max(self.most, 12 - self.cache.free_pages()[0])
            return out
    eng = Windowed()
    prompts = [[1, 2, 3, 4, 5], [9, 8, 7]]
    outs, sched = (_run_ahead if ahead else _run)(eng, prompts, max_new=40, opts=SchedulerOptions(max_seqs=2, max_rows=8, prefill_chunk=4))
    want = [_run(FakeEngine(), [p], max_new=40)[0][0]["tokens"] for p in prompts]
    assert [o["tokens"] for o in outs] == want
    # two requests of up to 45 tokens would hold 23 pages without the window; 12 exist and no request was preempted
    assert sched.stats.preemptions == 0 and eng.most <= 10


@pytest.mark.parametrize("seed", range(10))
def test_every_step_is_the_plain_schedulers_step(seed):
    """Random workloads (prompts of 1 to 30 tokens, limits, stop tokens, pools from roomy to tight, requests that arrive
    while others run): the engine's scheduler runs, step for step, the batch that the plain restatement of the policy
    (tests/plain_scheduler.py) runs: the same requests in the same order, the same positions and tokens, a new token
    wanted for the same ones; it ends the same requests for the same reasons and preempts as often."""
    import random

    from plain_scheduler import PlainScheduler
    rng = random.Random(seed)
    page, pages = rng.choice([2, 4, 8]), rng.choice([10, 16, 64])
    sizes = dict(max_seqs=rng.choice([2, 4, 8]), max_rows=rng.choice([4, 9, 16]), prefill_chunk=rng.choice([2, 5, 16]))
    eng = FakeEngine(pages=pages, page_size=page, max_slots=8, max_rows=16, max_context=48)
    sched = Scheduler(eng, SchedulerOptions(**sizes), sampler=HashSampler())
    plain = PlainScheduler(pages=pages, page_size=page, max_slots=8, max_context=48, **sizes)
    finishes, slot_name = {}, {}

    def submit(name):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.choice([0, 1, 2, 5, 9, 17, 30, 48]))]
        limit, stops = rng.choice([1, 3, 8, 40]), tuple(rng.sample(range(VOCAB), rng.choice([0, 0, 6])))
        # (a pool of 10 pages of 2 cannot hold the longest: keep those workloads to what one request can hold)
        if len(prompt) + limit > pages * page - page:
            prompt = prompt[:max(0, pages * page - page - limit)]

        def on_token(ev, logits, name=name):
            if ev.finished:
                finishes[name] = ev.finish_reason
        sched.submit(GenRequest(prompt=prompt, max_new_tokens=limit, stop_tokens=stops, on_token=on_token))
        early = plain.submit(name, prompt, limit, stops)
        return early

    expect = {}
    names = iter(range(1000))
    for _ in range(rng.randint(1, 6)):
        n = next(names)
        expect[n] = submit(n)
    for _ in range(400):
        want = plain.plan()
        before = len(eng.batches)
        ran = sched.step()
        assert ran == (want is not None)
        if want is None:
            if rng.random() < 0.5:      # idle: stop here, or wait for somebody to arrive
                break
        else:
            got = eng.batches[before]
            assert [(f, c, w) for _, f, c, w in got] == [(f, len(t), w) for _, f, t, w in want]
            for (slot, first, count, wants), (name, _, tokens, _) in zip(got, want):
                if first == 0:
                    slot_name[slot] = name
                assert slot_name[slot] == name and eng.fed[slot][first:first + count] == tokens
                if wants:
                    token = HashSampler().choose([list(eng.fed[slot])], None, [first + count])[0][0]
                    reason = plain.chosen(name, token)
                    if reason:
                        expect[name] = reason
        if rng.random() < 0.15:
            n = next(names)
            expect[n] = submit(n)
    while sched.step():
        want = plain.plan()
        assert want is not None
        for (slot, first, count, wants), (name, _, tokens, _) in zip(eng.batches[-1], want):
            if first == 0:
                slot_name[slot] = name
            if wants:
                reason = plain.chosen(name, HashSampler().choose([list(eng.fed[slot])], None, [first + count])[0][0])
                if reason:
                    expect[name] = reason
    assert plain.plan() is None
    assert finishes == {k: v for k, v in expect.items() if v is not None}
    assert sched.stats.preemptions == plain.preemptions
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages()
    _PLAIN_RUNS.append((sched.stats.preemptions, sorted(set(finishes.values()))))


_PLAIN_RUNS = []


def test_the_random_workloads_met_every_case():
    """(runs after the comparison above) Between them the workloads preempted, stopped on stop tokens, reached limits and
    refused prompts, so the comparison has seen every rule."""
    if len(_PLAIN_RUNS) < 10:
        pytest.skip("the comparison did not run in this session")
    assert any(p > 0 for p, _ in _PLAIN_RUNS)
    assert {"stop", "length", "empty_prompt", "context_length"} <= {r for _, reasons in _PLAIN_RUNS for r in reasons}


@pytest.mark.parametrize("ahead", [False, True])
def test_an_error_in_the_middle_of_a_run_leaves_the_cache_as_it_was(ahead):
    """The engine fails at its seventh step: the error reaches the caller, every slot and page is back, and the same
    engine serves the next run as if nothing had happened."""
    class Failing(PipeEngine if ahead else FakeEngine):
        fail_at = 7

        def step(self, entries):
            if len(self.batches) + 1 == self.fail_at:
                self.fail_at = -1
                raise EngineError("the seventh step fails")
            return super().step(entries)
    eng = Failing()
    run = _run_ahead if ahead else _run
    with pytest.raises(EngineError, match="seventh"):
        run(eng, PROMPTS)
    eng.cache.check()
    assert eng.cache.free_pages() == eng.cache.total_pages() and len(eng.cache.free_slots) == 8
    outs, _ = run(eng, PROMPTS)
    assert [o["tokens"] for o in outs] == [o["tokens"] for o in _solo()]
