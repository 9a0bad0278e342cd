"""The native stager on the CPU: a step's entries become the one integer array that goes to the device (tokens,
positions, slots, wanted rows, entry records, the wanted rows' slots), as restated here; steps that do not agree with
the cache's books are refused with a reason."""
from __future__ import annotations

import ctypes
import random

import numpy as np
import pytest
import torch

from stride_b200.cache.manager import CacheManager
from stride_b200.engine.engine import _native_stager
from stride_b200.parts import CacheNeed

R, VOCAB = 48, 100
_I32P = ctypes.POINTER(ctypes.c_int32)


def _cache(slots=6):
    need = CacheNeed("pages", kv_heads=1, head_dim=2, dtype=torch.float32)
    return CacheManager([need], device="cpu", max_slots=slots, max_context=64, page_size=4, num_pages=64)


def _stage(cache, entries, max_logit_rows=16):
    """entries: (slot, first, tokens, want). Returns (rc, message, staging, rows, wanted rows)."""
    lib = _native_stager(cache._lib)
    arr = lambda values: np.asarray(list(values) + [0], dtype=np.int32)     # never empty
    slot, first = arr(e[0] for e in entries), arr(e[1] for e in entries)
    count, n_want = arr(len(e[2]) for e in entries), arr(len(e[3]) for e in entries)
    tokens, want = arr(t for e in entries for t in e[2]), arr(j for e in entries for j in e[3])
    staging = np.full(9 * R, -7, dtype=np.int32)
    out = np.zeros(2, dtype=np.int32)
    p = lambda a: a.ctypes.data_as(_I32P)
    rc = lib.sb_stage_step(cache._pool, len(entries), p(slot), p(first), p(count), p(tokens), p(n_want), p(want), VOCAB, R, max_logit_rows,
                           p(staging), p(out))
    return rc, lib.sb_last_error().decode(), staging, int(out[0]), int(out[1])


@pytest.mark.parametrize("seed", range(5))
def test_staging_matches_its_restatement(seed):
    rng = random.Random(seed)
    cache = _cache()
    slots = [cache.acquire_slot() for _ in range(5)]
    entries, budget = [], R
    for s in rng.sample(slots, rng.randint(1, 5)):
        first = rng.randint(0, 20)
        L = rng.randint(1, min(9, budget - (5 - len(entries))))
        budget -= L
        assert cache.ensure(s, first + L)
        tokens = [-1] if (L == 1 and rng.random() < 0.3) else [rng.randrange(VOCAB) for _ in range(L)]
        want = sorted(rng.sample(range(L), rng.randint(0, min(L, 2))))
        entries.append((s, first, tokens, want))
    rc, msg, got, rows, wanted = _stage(cache, entries)
    assert rc == 0, msg
    ref = np.full(9 * R, -7, dtype=np.int32)
    at = w = 0
    for i, (s, first, tokens, want) in enumerate(entries):
        L = len(tokens)
        ref[at:at + L] = tokens
        ref[R + at:R + at + L] = np.arange(first, first + L)
        ref[2 * R + at:2 * R + at + L] = s
        for j in want:
            ref[3 * R + w], ref[8 * R + w] = at + j, s
            w += 1
        ref[4 * R + i], ref[5 * R + i], ref[6 * R + i], ref[7 * R + i] = s, at, L, first
        at += L
    assert (rows, wanted) == (at, w) and np.array_equal(got, ref)


def test_steps_that_disagree_with_the_books_are_refused():
    cache = _cache()
    a, b = cache.acquire_slot(), cache.acquire_slot()
    assert cache.ensure(a, 10) and cache.ensure(b, 4)
    ok = (a, 0, [1, 2, 3], [2])
    for entries, reason in (
            ([ok, (a, 3, [4], [0])], "appears twice"),
            ([(5, 0, [1], [])], "not held by a request"),
            ([(b, 2, [1, 2, 3], [])], "have no pages"),
            ([(a, -1, [1], [])], "have no pages"),
            ([(a, 0, [1, VOCAB], [])], "out of range"),
            ([(a, 0, [1, -1], [])], "out of range"),          # a placeholder only as a single decoded token
            ([(a, 0, [1, 2], [2])], "outside the entry"),
            ([(a, 0, [], [])], "without tokens"),
            ([(a, 0, list(range(10)), list(range(10))), (b, 0, [1, 2, 3, 4], [0, 1, 2, 3])], "exceed max_full_rows")):
        rc, msg, _, _, _ = _stage(cache, entries, max_logit_rows=12)
        assert rc < 0 and reason in msg, (entries, msg)
    cache2 = _cache()
    s = cache2.acquire_slot()
    assert cache2.ensure(s, 60)
    rc, msg, _, _, _ = _stage(cache2, [(s, 0, [1] * (R + 1), [])])
    assert rc < 0 and "exceeds max_rows" in msg
    assert _stage(cache, [ok, (b, 3, [-1], [0])])[0] == 0


def test_decode_steps_are_padded_for_their_graph():
    cache = _cache()
    lib = _native_stager(cache._lib)
    slots = [cache.acquire_slot() for _ in range(3)]
    firsts = [7, 0, 19]
    for s, f in zip(slots, firsts):
        assert cache.ensure(s, f + 1)
    p = lambda a: a.ctypes.data_as(_I32P)
    slot, first, token = (np.asarray(v, dtype=np.int32) for v in (slots, firsts, [5, -1, 99]))
    staging = np.full(9 * R, -7, dtype=np.int32)
    assert lib.sb_stage_decode(cache._pool, 3, 4, cache.pad_slot, p(slot), p(first), p(token), VOCAB, R, p(staging)) == 0
    pad = cache.pad_slot
    assert staging[0:4].tolist() == [5, -1, 99, 0] and staging[R:R + 4].tolist() == [7, 0, 19, 0]
    assert staging[2 * R:2 * R + 4].tolist() == slots + [pad] and staging[3 * R:3 * R + 4].tolist() == [0, 1, 2, 3]
    assert staging[8 * R:8 * R + 4].tolist() == slots + [pad]
    meta = staging[4 * R:8 * R].reshape(4, R)[:, :4]
    assert meta.tolist() == [slots + [pad], [0, 1, 2, 3], [1, 1, 1, 1], [7, 0, 19, 0]]
    for bad, reason in (((np.asarray([slots[0], slots[0], slots[2]], dtype=np.int32), first, token), "appears twice"),
                        ((slot, np.asarray([8, 0, 19], dtype=np.int32), token), "has no page"),
                        ((slot, first, np.asarray([5, VOCAB, 1], dtype=np.int32)), "out of range")):
        assert lib.sb_stage_decode(cache._pool, 3, 4, pad, p(bad[0]), p(bad[1]), p(bad[2]), VOCAB, R, p(staging)) < 0
        assert reason in lib.sb_last_error().decode()
