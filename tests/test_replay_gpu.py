"""Trace replay against the plain implementation, in 32-bit and in bfloat16: every
request whole; most of it in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; and mixed, up to four live requests with portions of
some beside decoded tokens of others, in a pool so small that pages are used again."""
from __future__ import annotations

import pytest
import torch

import plain_llama as plain
from conftest import TINY, TraceRun, bf16_noise, check_mean_deviation, logit_tolerance, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 100, 45, 120, 33], "B": [150, 41, 97, 200, 64], "C": [48, 130, 17, 99, 64],
           "D": [300, 65, 530, 129, 40], "U": [520, 257, 64, 300, 31]}


def _requests(name):
    vocab = TINY[name][0]["vocab_size"]
    return [random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[name])]


def _plain_logits(model_dir, requests, dtype):
    """Per request: (logits of the plain implementation, bfloat16 rounding noise of the request or None)."""
    cfg, w = plain.load_plain(model_dir)
    if dtype == "float32":
        return [(plain.forward(cfg, w, r, torch.float32, None), None) for r in requests]
    return [(plain.forward(cfg, w, r, torch.float32, torch.bfloat16), bf16_noise(cfg, w, r)) for r in requests]


def _compare(got, want, dtype, what, noise=None):
    if want is None:        # this configuration and precision is held to bit-equality between the replays alone
        return
    tol = logit_tolerance(dtype, want, noise)
    diff = (got - want).abs()
    worst = int(diff.max(dim=1).values.argmax())
    assert diff.max() <= tol, f"{what}: max |diff| {diff.max():.3e} > {tol:.3e}, first bad place {int((diff.max(dim=1).values > tol).nonzero()[0])}, worst {worst}"


def _cut(logits, a, b):
    return None if logits is None else logits[a:b]


class _Bits:
    """Keeps the logits of the first replay of every request and checks that later replays, cut and batched in other
    ways and lying in other pages, give the same bits: in both precisions every kernel adds in an order that depends
    on the token's own position alone."""

    def __init__(self):
        self.first = {}

    def check(self, i, a, got, what):
        for k in range(got.shape[0]):
            ref = self.first.setdefault((i, a + k), got[k].clone())
            assert torch.equal(ref, got[k]), f"{what}: position {a + k} differs in bits from its first replay (max {(ref - got[k]).abs().max():.3e})"


def _portions(n, sizes):
    """Cut range(n) into portions of the given sizes (cycled), the last one may be shorter but never 1 token
    unless n forces it."""
    out, at, i = [], 0, 0
    while at < n:
        s = min(sizes[i % len(sizes)], n - at)
        out.append((at, at + s))
        at += s
        i += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "U"])
def test_replay_modes(name, dtype, model_dirs, tmp_path):
    cfg, _, page = TINY[name]
    vocab = cfg["vocab_size"]
    reqs = _requests(name)
    if name == "U" and dtype == "bfloat16":
        # U makes every key carry weight 1/T; losing one moves logits by ~1e-3, which float32 shows and bfloat16 cannot
        # resolve: no comparison with the plain implementation here, but the four replays still have to agree in bits
        want = [(None, None)] * len(reqs)
    else:
        want = _plain_logits(model_dirs[name], reqs, dtype)
    # The pool holds the two longest requests plus one page: mixed replay must reuse pages.
    per = lambda n: -(-n // page) * page
    longest = sorted((per(len(r)) for r in reqs), reverse=True)
    pool = max(longest[0] + longest[1] + page, 4 * page)
    tr = TraceRun(model_dirs[name], dtype, tmp_path, pool, page, extra=("--kv-shuffle", "7"))
    bits = _Bits()
    try:
        # 1. each request alone and whole, logits at every place
        for i, r in enumerate(reqs):
            s = tr.run([(f"w{i}", r, range(len(r)))], end=[f"w{i}"])
            _compare(tr.logits(s, vocab), want[i][0], dtype, f"{name} whole request {i}", want[i][1])
            if want[i][1] is not None:
                check_mean_deviation(tr.logits(s, vocab), want[i][0], want[i][1], f"{name} whole request {i}")
            bits.check(i, 0, tr.logits(s, vocab), f"{name} whole request {i}")
        # 2. all but the last 32 tokens in one step, then one by one
        for i, r in enumerate(reqs):
            cut = max(1, len(r) - 32)
            s = tr.run([(f"d{i}", r[:cut], [cut - 1])])
            _compare(tr.logits(s, vocab), _cut(want[i][0], cut - 1, cut), dtype, f"{name} request {i} prefill end", want[i][1])
            bits.check(i, cut - 1, tr.logits(s, vocab), f"{name} request {i} prefill end")
            for p in range(cut, len(r)):
                s = tr.run([(f"d{i}", r[p:p + 1], [0])], end=[f"d{i}"] if p == len(r) - 1 else [])
                _compare(tr.logits(s, vocab), _cut(want[i][0], p, p + 1), dtype, f"{name} request {i} decode at {p}", want[i][1])
                bits.check(i, p, tr.logits(s, vocab), f"{name} request {i} decode at {p}")
        # 3. portions of changing size, down to two tokens
        for i, r in enumerate(reqs):
            cuts = _portions(len(r), [7, 2, 19, 3, 2, 31, 5])
            for j, (a, b) in enumerate(cuts):
                s = tr.run([(f"p{i}", r[a:b], range(b - a))], end=[f"p{i}"] if j == len(cuts) - 1 else [])
                _compare(tr.logits(s, vocab), _cut(want[i][0], a, b), dtype, f"{name} request {i} portion {a}:{b}", want[i][1])
                bits.check(i, a, tr.logits(s, vocab), f"{name} request {i} portion {a}:{b}")
        # 4. mixed: requests start at different steps, portions beside single tokens, pages reused
        fed = [0] * len(reqs)
        sizes = [[9, 1, 1, 4, 1], [2, 13, 1, 1, 1, 6], [5, 1, 1, 1], [17, 1, 2, 1, 1], [3, 1, 8, 1]]
        live, waiting, turn = [], list(range(len(reqs))), [0] * len(reqs)
        steps = 0
        while live or waiting:
            per_live = lambda: sum(per(len(reqs[i])) for i in live)
            while waiting and len(live) < 4 and per_live() + per(len(reqs[waiting[0]])) <= pool:
                live.append(waiting.pop(0))
            entries, ends, spans = [], [], []
            for k, i in enumerate(list(live)):
                if (steps + k) % 5 == 4 and len(live) > 1:
                    continue            # this request sits the step out and goes on later
                n = min(sizes[i][turn[i] % len(sizes[i])], len(reqs[i]) - fed[i])
                turn[i] += 1
                a, b = fed[i], fed[i] + n
                entries.append((f"m{i}", reqs[i][a:b], range(n)))
                spans.append((i, a, b))
                fed[i] = b
                if b == len(reqs[i]):
                    ends.append(f"m{i}")
                    live.remove(i)
            s = tr.run(entries, end=ends)
            got = tr.logits(s, vocab)
            at = 0
            for i, a, b in spans:
                _compare(got[at:at + b - a], _cut(want[i][0], a, b), dtype, f"{name} mixed step {steps} request {i} {a}:{b}", want[i][1])
                bits.check(i, a, got[at:at + b - a], f"{name} mixed step {steps} request {i} {a}:{b}")
                at += b - a
            steps += 1
    finally:
        tr.close()
