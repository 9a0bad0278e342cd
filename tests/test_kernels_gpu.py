"""Each CUDA kernel alone against a plain torch reference of the same operation, at sizes other
than the engine's test configurations."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("n,M,K", [(1, 128, 64), (5, 200, 72), (16, 256, 512), (33, 384, 2048), (64, 1000, 136),
                                   (128, 128, 8192), (200, 333, 264), (777, 520, 1024)])
def test_gemm_tc_store_and_add(n, M, K):
    from stride_b200.kernels import ops
    x = _rand(n, K, seed=1, dtype=torch.bfloat16)
    w = _rand(M, K, seed=2, scale=0.05, dtype=torch.bfloat16)
    ref = x.float() @ w.float().T
    tol = 2e-3 * float(ref.abs().max()) + 1e-5      # float32 accumulation in another order
    out = torch.full((n, M), float("nan"), device=DEV)
    ops.gemm_tc(x, w, out, ops.STORE)
    assert ops.gemm_tc_status() == 0
    assert (out - ref).abs().max() <= tol
    base = _rand(n, M, seed=3)
    acc = base.clone()
    ops.gemm_tc(x, w, acc, ops.ADD)
    assert ops.gemm_tc_status() == 0
    assert (acc - (base + ref)).abs().max() <= tol
    splits = ops.gemm_tc_splits(M, K)
    if splits > 1 and n <= ops.gemm_tc_partial_tokens():
        parts = torch.full((splits, n, M), float("nan"), device=DEV)
        ops.gemm_tc(x, w, parts, ops.STORE, splits=splits)
        assert ops.gemm_tc_status() == 0
        assert (parts.sum(0) - ref).abs().max() <= tol
    elif splits > 1:    # the kernel adds the ranges itself
        out = torch.full((n, M), float("nan"), device=DEV)
        ops.gemm_tc(x, w, out, ops.STORE, splits=splits)
        assert ops.gemm_tc_status() == 0
        assert (out - ref).abs().max() <= tol


def test_gemm_tc_one_hot_positions():
    """x rows that are unit vectors pick single columns of W: any wrong swizzle, descriptor step or
    tile offset shows as a wrong element, not as a small numeric difference."""
    from stride_b200.kernels import ops
    n, M, K = 96, 256, 256
    w = _rand(M, K, seed=4, dtype=torch.bfloat16)
    idx = torch.arange(n) * 37 % K
    x = torch.zeros(n, K, dtype=torch.bfloat16, device=DEV)
    x[torch.arange(n), idx] = 1.0
    out = torch.zeros(n, M, device=DEV)
    ops.gemm_tc(x, w, out, ops.STORE)
    assert ops.gemm_tc_status() == 0
    assert torch.equal(out, w.float()[:, idx.to(DEV)].T.contiguous())


@pytest.mark.parametrize("n,I,K", [(3, 64, 64), (40, 200, 136), (130, 320, 192), (300, 1024, 512)])
def test_gemm_tc_swiglu(n, I, K):
    from stride_b200.kernels import ops
    x = _rand(n, K, seed=5, dtype=torch.bfloat16)
    w = _rand(2 * I, K, seed=6, scale=0.1, dtype=torch.bfloat16)
    g = x.float() @ w[:I].float().T
    u = x.float() @ w[I:].float().T
    ref = (g / (1 + torch.exp(-g))) * u
    out = torch.full((n, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, out, ops.SWIGLU, half_rows=I)
    assert ops.gemm_tc_status() == 0
    assert (out.float() - ref).abs().max() <= 1e-2 * float(ref.abs().max()) + 1e-4


@pytest.mark.parametrize("M,K", [(384, 1024), (2048, 2048), (200, 8192), (1000, 136)])
def test_gemm_tc_does_not_depend_on_the_batch(M, K):
    """A token's result has the same bits alone and among 7 to 700 other tokens (token tiles of 16 to 256), wherever it stands among
    them: with K in one range, and with the weight's K ranges added by the caller (few tokens) or by the kernel (many)."""
    from stride_b200.kernels import ops
    w = _rand(M, K, seed=7, scale=0.05, dtype=torch.bfloat16)
    x = _rand(700, K, seed=8, dtype=torch.bfloat16)
    S, few = ops.gemm_tc_splits(M, K), ops.gemm_tc_partial_tokens()
    one, ranged = [], []
    for n, at in ((1, 0), (8, 5), (100, 77), (200, 130), (256, 255), (333, 1), (700, 699)):
        xs = x[:n].clone()
        xs[at] = x[0]
        out = torch.zeros(n, M, device=DEV)
        ops.gemm_tc(xs, w, out, ops.STORE)
        one.append(out[at].clone())
        if S > 1:
            if n <= few:
                parts = torch.zeros(S, n, M, device=DEV)
                ops.gemm_tc(xs, w, parts, ops.STORE, splits=S)
                total = parts[0, at].clone()
                for s in range(1, S):
                    total += parts[s, at]
            else:
                out = torch.zeros(n, M, device=DEV)
                ops.gemm_tc(xs, w, out, ops.STORE, splits=S)
                total = out[at].clone()
            ranged.append(total)
    assert ops.gemm_tc_status() == 0
    for group in (one, ranged):
        for other in group[1:]:
            assert torch.equal(group[0], other)


# ---------------------------------------------------------------------------- attention
def _paged_case(lengths_new, lengths_old, Hq, Hkv, D, page, dtype, seed=0, peak=None):
    """A step with one entry per request: request i has lengths_old[i] cached tokens and brings
    lengths_new[i] new ones. Returns the tensors the attention kernels take plus per-request q, k, v."""
    g = torch.Generator().manual_seed(seed)
    E = len(lengths_new)
    total = [a + b for a, b in zip(lengths_old, lengths_new)]
    max_pages = max(-(-t // page) for t in total) + 1
    n_pages = sum(-(-t // page) for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.zeros(n_pages, 2, Hkv, page, D, dtype=dtype)
    table = torch.full((E, max_pages), -1, dtype=torch.int32)
    ks, vs, qs = [], [], []
    rows_q, positions, slots = [], [], []
    meta = torch.zeros(4, E, dtype=torch.int32)
    at = 0
    for i in range(E):
        T = total[i]
        k = torch.randn(T, Hkv, D, generator=g).to(dtype)
        v = torch.randn(T, Hkv, D, generator=g).to(dtype)
        q = torch.randn(lengths_new[i], Hq, D, generator=g).to(dtype)
        if peak is not None and i == peak[0]:
            # one far key stands out for the last query of this request: a kernel that skips it is far off
            key = peak[1]
            k[key] = 0
            k[key, :, 0] = 8.0
            q[-1] = 0
            q[-1, :, 0] = 8.0
            v[key] = 5.0
        for t in range(T):
            pi = t // page
            if table[i, pi] < 0:
                table[i, pi] = perm.pop()
            cache[table[i, pi], 0, :, t % page] = k[t]
            cache[table[i, pi], 1, :, t % page] = v[t]
        ks.append(k), vs.append(v), qs.append(q)
        meta[:, i] = torch.tensor([i, at, lengths_new[i], lengths_old[i]])
        positions += list(range(lengths_old[i], T))
        slots += [i] * lengths_new[i]
        at += lengths_new[i]
    q_all = torch.cat(qs).reshape(at, Hq * D)
    dev = lambda t: t.to(DEV)
    return dict(q=dev(q_all), cache=dev(cache), table=dev(table), meta=dev(meta), positions=dev(torch.tensor(positions, dtype=torch.int32)),
                slots=dev(torch.tensor(slots, dtype=torch.int32)), qs=qs, ks=ks, vs=vs, old=lengths_old, new=lengths_new)


def _attention_reference(case, Hq, Hkv, D, window=0):
    import plain_llama as plain
    outs = []
    scale_fix = 1.0
    for q, k, v, old, new in zip(case["qs"], case["ks"], case["vs"], case["old"], case["new"]):
        T = old + new
        qq = torch.zeros(T, Hq, D)
        qq[old:] = q.float()
        o = plain.attention(qq, k.float(), v.float(), torch.arange(T), window)
        outs.append(o[old:])
    return torch.cat(outs)


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 16, 0), (128, 6, 2, 64, 0), (64, 4, 4, 8, 0), (64, 12, 4, 32, 100),
                                                  (128, 16, 1, 128, 0)])
def test_attention_tc_against_plain(D, Hq, Hkv, page, window):
    """Portions and decoded tokens in one step, keys spread over shuffled pages, sequences that cross the
    256-key chunk and 64-key tile edges."""
    from stride_b200.kernels import ops
    new = [1, 77, 1, 3, 200, 1, 2, 64]
    old = [300, 0, 255, 256, 100, 0, 510, 63]
    case = _paged_case(new, old, Hq, Hkv, D, page, torch.bfloat16, seed=D + page, peak=(0, 3))
    G = Hq // Hkv
    ppt, short = 64 // G, 16 // G
    tiles, items, last = [], [], 0
    for e, (L, p0) in enumerate(zip(new, old)):
        if L <= short:
            items.append(e)
            last = max(last, p0 + L - 1)
        else:
            for t in range(-(-L // ppt)):
                tiles += [e, t]
    work = torch.tensor(tiles + items, dtype=torch.int32, device=DEV)
    chunks = last // 256 + 1
    scratch = torch.zeros(ops.attention_tc_scratch(len(items), Hkv, chunks, D), device=DEV)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    ops.attention_tc(case["q"], out, case["cache"], case["table"], case["meta"], work, len(tiles) // 2, len(items), chunks,
                     scratch, Hq, Hkv, D, window, scale)
    ref = _attention_reference(case, Hq, Hkv, D, window)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    # bfloat16 probabilities and output: 2^-8 relative on values of order 1
    assert (got - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
    # the decode kernel folding its own chunks (counters) gives the same bits as the separate combine kernel
    counters = torch.zeros(len(items) * Hkv, dtype=torch.int32, device=DEV)
    out3 = torch.full_like(case["q"], float("nan"))
    for _ in range(2):       # twice: the counters must be back at zero after a launch
        ops.attention_tc(case["q"], out3, case["cache"], case["table"], case["meta"], work, len(tiles) // 2, len(items), chunks,
                         scratch, Hq, Hkv, D, window, scale, counters=counters)
        assert torch.equal(out3, out) and int(counters.abs().sum()) == 0
    # the generic kernel on the same case
    out2 = torch.full_like(case["q"], float("nan"))
    ops.attention_generic(case["q"], out2, case["cache"], case["table"], case["positions"], case["slots"], Hq, Hkv, D, window, scale)
    assert (out2.float().cpu() - ref).abs().max() <= 1e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 16, 0), (64, 32, 8, 64, 0), (64, 6, 2, 8, 150), (128, 8, 2, 32, 0),
                                                  (128, 6, 2, 64, 300), (64, 5, 5, 16, 0)])
def test_attention_kernels_agree_in_bits(D, Hq, Hkv, page, window):
    """The last 150 positions of a request of 700 tokens, computed as one prompt portion by the mma.sync kernel, as one
    portion by the tcgen05 kernel, as portions of two positions and as single positions by the decode
    kernel: every row has the same bits each way. This also pins that tcgen05.mma and mma.sync accumulate alike."""
    from stride_b200.kernels import ops
    T, R = 700, 150
    case = _paged_case([R], [T - R], Hq, Hkv, D, page, torch.bfloat16, seed=3 * D + page, peak=(0, 5))
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    q, cache, table = case["q"], case["cache"], case["table"]

    def run(entries, tc5):
        """entries: (first row, length) of each entry; its first position is T - R + first row."""
        E = len(entries)
        meta = torch.zeros(4, E, dtype=torch.int32)
        for e, (row, L) in enumerate(entries):
            meta[:, e] = torch.tensor([0, row, L, T - R + row])
        meta = meta.to(DEV)
        out = torch.full_like(q, float("nan"))
        short = 16 // G
        if tc5:
            tiles = [x for e, (row, L) in enumerate(entries) for t in range(-(-L // (128 // G))) for x in (e, t)]
            ops.attention_tc5(q, out, cache, table, meta, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 2,
                              Hq, Hkv, D, window, scale)
            assert ops.attention_tc5_status() == 0
            return out
        tiles, items = [], []
        for e, (row, L) in enumerate(entries):
            if L <= short:
                items.append(e)
            else:
                tiles += [x for t in range(-(-L // (64 // G))) for x in (e, t)]
        chunks = (T - 1) // 256 + 1
        scratch = torch.zeros(max(1, ops.attention_tc_scratch(len(items), Hkv, chunks, D)), device=DEV)
        counters = torch.zeros(max(1, len(items)) * Hkv, dtype=torch.int32, device=DEV)
        ops.attention_tc(q, out, cache, table, meta, torch.tensor(tiles + items, dtype=torch.int32, device=DEV), len(tiles) // 2,
                         len(items), chunks, scratch, Hq, Hkv, D, window, scale, counters=counters)
        return out

    whole = run([(0, R)], False)
    ref = _attention_reference(case, Hq, Hkv, D, window)
    assert (whole.float().cpu() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
    singles = run([(r, 1) for r in range(R)], False)
    assert torch.equal(whole, singles)
    if 2 * G <= 16:
        pairs = run([(r, 2) for r in range(0, R, 2)], False)
        assert torch.equal(whole, pairs)
    uneven = run([(0, 37), (37, 1), (38, 70), (108, 42)], False)
    assert torch.equal(whole, uneven)
    if ops.attention_tc5_supported(Hq, Hkv, D, page):
        assert torch.equal(whole, run([(0, R)], True))
        assert torch.equal(whole, run([(0, 37), (37, 1), (38, 70), (108, 42)], True))


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 64, 0), (64, 32, 8, 128, 0), (64, 6, 2, 8, 700), (128, 8, 2, 64, 0),
                                                  (128, 6, 2, 48, 1100), (64, 5, 5, 16, 0), (64, 24, 2, 64, 0)])
def test_decode_attention_over_long_contexts(D, Hq, Hkv, page, window):
    """Decoded tokens (and one entry of two positions) over contexts of 1 to 2,300 keys, pages of 8 to 128 keys (one
    lookup per tile, or one per key), 1 to 12 query heads per key/value head (rows 8 to 15 of a tile in use or not),
    one far key that stands out: the decode kernel agrees with the float64 reference and leaves its counters ready."""
    from stride_b200.kernels import ops
    G = Hq // Hkv
    news = [1, 1, min(2, 16 // G), 1, 1, 1]
    olds = [2299, 0, 1279, 255, 256, 1800]
    case = _paged_case(news, olds, Hq, Hkv, D, page, torch.bfloat16, seed=5 * D + page, peak=(0, 3))
    q, cache, table, meta = case["q"], case["cache"], case["table"], case["meta"]
    scale = 1.0 / math.sqrt(D)
    E = len(news)
    items = torch.arange(E, dtype=torch.int32, device=DEV)
    chunks = max(a + b - 1 for a, b in zip(news, olds)) // 256 + 1
    out = torch.full_like(q, float("nan"))
    scratch = torch.zeros(ops.attention_tc_scratch(E, Hkv, chunks, D), device=DEV)
    counters = torch.zeros(E * Hkv, dtype=torch.int32, device=DEV)
    ops.attention_tc(q, out, cache, table, meta, items, 0, E, chunks, scratch, Hq, Hkv, D, window, scale, counters=counters)
    torch.cuda.synchronize()
    assert int(counters.abs().sum()) == 0
    ref = _attention_reference(case, Hq, Hkv, D, window)
    assert (out.float().cpu() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
    # the same entries again, in another order in the batch: the same bits
    order = torch.tensor([3, 0, 5, 1, 4, 2], dtype=torch.int32, device=DEV)
    again = torch.full_like(q, float("nan"))
    ops.attention_tc(q, again, cache, table, meta, order, 0, E, chunks, scratch, Hq, Hkv, D, window, scale, counters=counters)
    assert torch.equal(out, again)


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 64, 0), (128, 6, 2, 32, 0), (64, 4, 4, 16, 300)])
@pytest.mark.parametrize("olds", [[255, 3], [256, 100, 0], [1279, 300, 0, 1023], [2047, 5, 1800]])
def test_decode_attention_folds_its_chunks_three_ways_with_the_same_bits(D, Hq, Hkv, page, window, olds):
    """One chunk (the rows are written at once), 2 to 8 chunks (a cluster per entry, records through distributed shared
    memory) and the records in global memory folded by a kernel of its own give the same bits; the batch's longest
    context decides which of the first two runs, entries shorter than it sit in the same clusters."""
    from stride_b200.kernels import ops
    news = [1] * len(olds)
    case = _paged_case(news, olds, Hq, Hkv, D, page, torch.bfloat16, seed=D + len(olds), peak=(0, 1))
    q, cache, table, meta = case["q"], case["cache"], case["table"], case["meta"]
    E = len(news)
    items = torch.arange(E, dtype=torch.int32, device=DEV)
    chunks = max(olds) // 256 + 1
    assert 1 <= chunks <= 8
    scale = 1.0 / math.sqrt(D)
    outs = []
    for own_fold in (True, False):
        out = torch.full_like(q, float("nan"))
        scratch = torch.zeros(ops.attention_tc_scratch(E, Hkv, chunks, D), device=DEV)
        counters = torch.zeros(E * Hkv, dtype=torch.int32, device=DEV) if own_fold else None
        ops.attention_tc(q, out, cache, table, meta, items, 0, E, chunks, scratch, Hq, Hkv, D, window, scale, counters=counters)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    ref = _attention_reference(case, Hq, Hkv, D, window)
    assert (outs[0].float().cpu() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 64, 0), (128, 6, 2, 32, 0), (64, 4, 4, 16, 8500)])
def test_decode_attention_folds_the_records_of_a_long_context_three_ways_with_the_same_bits(D, Hq, Hkv, page, window):
    """Tens of chunks an entry. Few entries: the records are folded by a kernel of its own that streams them through
    shared memory. Many entries: by the CTA that finishes an entry last, or (no counters) by the plain fold kernel. The
    same rows have the same bits from all three; entries of two tokens and a short entry sit in the same launch."""
    from stride_b200.kernels import ops
    G = Hq // Hkv
    olds, news = [9000, 300, 8191], [1, min(2, 16 // G), 2]
    case = _paged_case(news, olds, Hq, Hkv, D, page, torch.bfloat16, seed=D + 3, peak=(0, 700))
    q, cache, table, meta = case["q"], case["cache"], case["table"], case["meta"]
    E = len(news)
    chunks = max(a + b - 1 for a, b in zip(olds, news)) // 256 + 1
    assert chunks >= 32
    scale = 1.0 / math.sqrt(D)

    def run(copies, with_counters):
        items = torch.arange(E, dtype=torch.int32, device=DEV).repeat(copies)   # (copies of an entry write the same rows)
        out = torch.full_like(q, float("nan"))
        scratch = torch.zeros(ops.attention_tc_scratch(E * copies, Hkv, chunks, D), device=DEV)
        counters = torch.zeros(E * copies * Hkv, dtype=torch.int32, device=DEV) if with_counters else None
        ops.attention_tc(q, out, cache, table, meta, items, 0, E * copies, chunks, scratch, Hq, Hkv, D, window, scale, counters=counters)
        return out
    streamed = run(1, True)
    many = 148 // (E * Hkv) + 1          # more (entry, head) pairs than SMs: the streaming kernel is not chosen
    assert torch.equal(run(many, True), streamed)
    assert torch.equal(run(many, False), streamed)
    assert torch.equal(run(1, False), streamed)
    ref = _attention_reference(case, Hq, Hkv, D, window)
    assert (streamed.float().cpu() - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(64, 8, 2, 16, 0), (64, 32, 8, 64, 100), (128, 6, 2, 32, 0), (64, 3, 3, 8, 0)])
def test_decode_attention_with_rotation_fused(D, Hq, Hkv, page, window):
    """The decode kernel that rotates and appends by itself gives the same output and leaves the same cache, bit for
    bit, as the rotation kernel followed by the decode kernel. Entries of one to three positions, some crossing a
    chunk edge (positions 255 | 256) or a page edge."""
    from stride_b200.kernels import ops
    G = Hq // Hkv
    news = [1, min(2, 16 // G), 1, min(3, 16 // G), 1]
    olds = [300, 255, 0, 509, 63]
    case = _paged_case(news, olds, Hq, Hkv, D, page, torch.bfloat16, seed=D + Hq)
    n = sum(news)
    g = torch.Generator().manual_seed(11)
    S = 3
    qkv = torch.randn(S, n, (Hq + 2 * Hkv) * D, generator=g).to(DEV)
    max_pos = max(a + b for a, b in zip(news, olds))
    ang = torch.rand(max_pos, D // 2, generator=g) * 6.28
    cos_sin = torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous().to(DEV)
    items = torch.arange(len(news), dtype=torch.int32, device=DEV)
    chunks = (max_pos - 1) // 256 + 1
    scale = 1.0 / math.sqrt(D)

    def buffers():
        scratch = torch.zeros(ops.attention_tc_scratch(len(news), Hkv, chunks, D), device=DEV)
        counters = torch.zeros(len(news) * Hkv, dtype=torch.int32, device=DEV)
        return case["cache"].clone(), torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV), scratch, counters

    cache_a, out_a, scratch, counters = buffers()
    q = torch.zeros(n, Hq * D, dtype=torch.bfloat16, device=DEV)
    ops.rope_append(qkv, case["positions"], case["slots"], cos_sin, D, q, cache_a, case["table"], Hq, Hkv, D)
    ops.attention_tc(q, out_a, cache_a, case["table"], case["meta"], items, 0, len(news), chunks, scratch, Hq, Hkv, D, window, scale,
                     counters=counters)
    cache_b, out_b, scratch, counters = buffers()
    ops.attention_decode_rope(qkv, cos_sin, out_b, cache_b, case["table"], case["meta"], items, len(news), chunks, scratch, counters,
                              Hq, Hkv, D, window, scale)
    assert torch.isfinite(out_a.float()).all()
    assert torch.equal(out_a, out_b)
    assert torch.equal(cache_a, cache_b)
    assert not torch.equal(cache_a, case["cache"])


@pytest.mark.parametrize("T,R", [(11, 11), (70, 70), (300, 5), (600, 130)])
def test_attention_outputs_are_nearly_all_correctly_rounded(T, R):
    """Against a 64-bit softmax on the same bfloat16 inputs: all but a few per thousand of the tensor-core kernels'
    outputs are the correctly rounded bfloat16 value (the rest are one step off). A yardstick for the 32-bit softmax and
    the two-part weights: with one-part bfloat16 weights, or with parts cut instead of rounded, several times as many
    outputs are off."""
    from stride_b200.kernels import ops
    D, Hq, Hkv, page = 64, 4, 2, 16
    G = Hq // Hkv
    case = _paged_case([R], [T - R], Hq, Hkv, D, page, torch.bfloat16, seed=T)
    q, cache, table = case["q"], case["cache"], case["table"]
    qf, kf, vf = case["qs"][0].double(), case["ks"][0].double(), case["vs"][0].double()
    ref = torch.zeros(R, Hq, D, dtype=torch.float64)
    for r in range(R):
        pos = T - R + r
        for h in range(Hq):
            p = torch.softmax((kf[:pos + 1, h // G] @ qf[r, h]) / math.sqrt(D), 0)
            ref[r, h] = p @ vf[:pos + 1, h // G]
    want = ref.reshape(R, Hq * D).to(torch.bfloat16)
    meta = torch.tensor([[0], [0], [R], [T - R]], dtype=torch.int32, device=DEV)
    for tc5 in (True, False):
        out = torch.full_like(q, float("nan"))
        if tc5:
            tiles = [x for t in range(-(-R // (128 // G))) for x in (0, t)]
            ops.attention_tc5(q, out, cache, table, meta, torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 2, Hq, Hkv, D,
                              0, 1 / math.sqrt(D))
            assert ops.attention_tc5_status() == 0
        else:
            short = 16 // G
            tiles, items = ([], [0]) if R <= short else ([x for t in range(-(-R // (64 // G))) for x in (0, t)], [])
            chunks = (T - 1) // 256 + 1
            scratch = torch.zeros(max(1, ops.attention_tc_scratch(len(items), Hkv, chunks, D)), device=DEV)
            counters = torch.zeros(max(1, len(items)) * Hkv, dtype=torch.int32, device=DEV)
            ops.attention_tc(q, out, cache, table, meta, torch.tensor(tiles + items, dtype=torch.int32, device=DEV), len(tiles) // 2,
                             len(items), chunks, scratch, Hq, Hkv, D, 0, 1 / math.sqrt(D), counters=counters)
        off = int((out.cpu() != want).sum())
        assert off <= 0.0025 * out.numel() + 1, f"{off} of {out.numel()} outputs are not the correctly rounded value"
        assert (out.cpu().float() - want.float()).abs().max() <= 2.0 ** -7 * float(want.float().abs().max())


@pytest.mark.parametrize("D,Hq,Hkv,page,window", [(48, 3, 3, 16, 0), (16, 4, 2, 64, 0), (80, 10, 2, 8, 37), (256, 2, 1, 32, 0),
                                                   (50, 2, 1, 16, 21), (7, 3, 3, 8, 0), (512, 1, 1, 16, 0), (64, 8, 2, 64, 100), (132, 2, 2, 16, 0)])
def test_attention_generic_float32(D, Hq, Hkv, page, window):
    from stride_b200.kernels import ops
    new = [1, 50, 1, 130, 2]
    old = [200, 0, 127, 5, 128]
    case = _paged_case(new, old, Hq, Hkv, D, page, torch.float32, seed=D, peak=(0, 1))
    out = torch.full_like(case["q"], float("nan"))
    ops.attention_generic(case["q"], out, case["cache"], case["table"], case["positions"], case["slots"], Hq, Hkv, D, window, D ** -0.5)
    ref = _attention_reference(case, Hq, Hkv, D, window)
    assert (out.cpu() - ref).abs().max() <= 2e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,Hq,Hkv,page,window,dtype", [(64, 8, 2, 64, 0, torch.float32), (80, 3, 1, 16, 300, torch.float32),
                                                         (128, 4, 4, 32, 0, torch.bfloat16), (256, 2, 1, 16, 0, torch.float32),
                                                         (512, 1, 1, 8, 0, torch.float32), (16, 2, 2, 64, 0, torch.float32)])
def test_attention_generic_tiles_side_by_side_give_the_bits_of_tiles_in_a_row(D, Hq, Hkv, page, window, dtype):
    """A few rows: a cluster of blocks per (row, head), each with tiles of its own, folded out of the others' shared memory.
    Many rows: one block per (row, head), tile after tile. The same rows give the same bits both ways. The longest
    request has more tiles than the cluster has blocks, so that a block holds two."""
    from stride_b200.kernels import ops
    new, old = [1, 1, 2], [1100, 130, 5]
    case = _paged_case(new, old, Hq, Hkv, D, page, dtype, seed=D + 1, peak=(0, 3))
    n = sum(new)
    few = torch.full_like(case["q"], float("nan"))
    ops.attention_generic(case["q"], few, case["cache"], case["table"], case["positions"], case["slots"], Hq, Hkv, D, window, D ** -0.5)
    copies = 4 * 148 // (n * Hq) + 2   # more blocks than a cluster per (row, head) is launched for
    q = case["q"].repeat(copies, 1)
    many = torch.full_like(q, float("nan"))
    ops.attention_generic(q, many, case["cache"], case["table"], case["positions"].repeat(copies), case["slots"].repeat(copies),
                          Hq, Hkv, D, window, D ** -0.5)
    for c in range(copies):
        assert torch.equal(many[c * n:(c + 1) * n], few)
    ref = _attention_reference(case, Hq, Hkv, D, window)
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7
    assert (few.float().cpu() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))


# ---------------------------------------------------------------------------- the small kernels
@pytest.mark.parametrize("n,H", [(1, 64), (7, 88), (33, 2048), (4, 5000), (130, 264), (300, 2048), (77, 90)])
def test_rmsnorm_with_partials(n, H):
    from stride_b200.kernels import ops
    h = _rand(n, H, seed=1)
    parts = _rand(3, n, H, seed=2)
    w = _rand(H, seed=3, dtype=torch.bfloat16)
    for out_dtype in (torch.float32, torch.bfloat16):
        hh = h.clone()
        out = torch.zeros(n, H, dtype=out_dtype, device=DEV)
        ops.rmsnorm(hh, w, 1e-5, out, partials=parts)
        x = h + ((parts[0] + parts[1]) + parts[2])
        assert torch.equal(hh, x)
        ref = w.float() * (x * (1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / H + 1e-5)))
        tol = 1e-5 if out_dtype == torch.float32 else 1e-2
        assert (out.float() - ref).abs().max() <= tol * float(ref.abs().max())


@pytest.mark.parametrize("H", [64, 264, 1024, 2048, 3072, 4096, 8192])
def test_rmsnorm_does_not_depend_on_the_batch(H):
    """A row's normed values have the same bits in a step of 3 rows and of 300 (one block per row) and of 1,700 (one warp
    per row, which takes over for many rows with at most one partial sum to add), and with two partial sums at 3 or 300."""
    from stride_b200.kernels import ops
    N = 1700
    h = _rand(N, H, seed=4, scale=3.0)
    parts = _rand(2, N, H, seed=5)
    w = _rand(H, seed=6, dtype=torch.bfloat16)
    for out_dtype in (torch.float32, torch.bfloat16):
        for P, sizes in ((1, (3, 64, 300, N)), (2, (3, 65, 300)), (0, (3, 300, N))):
            outs = []
            for n in sizes:
                hh = h[:n].clone()
                out = torch.zeros(n, H, dtype=out_dtype, device=DEV)
                ops.rmsnorm(hh, w, 1e-5, out, partials=parts[:P, :n].contiguous() if P else None)
                outs.append(out[:3].clone())
            for other in outs[1:]:
                assert torch.equal(outs[0], other)


def test_embed_swiglu_gather():
    from stride_b200.kernels import ops
    table = _rand(333, 88, seed=1, dtype=torch.bfloat16)
    tok = torch.tensor([0, 332, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.zeros(5, 88, device=DEV)
    ops.embed(tok, table, out)
    assert torch.equal(out, table.float()[tok.long()])
    gu = _rand(9, 2 * 136, seed=2)
    z = torch.zeros(9, 136, device=DEV)
    ops.swiglu(gu, z)
    a, b = gu[:, :136], gu[:, 136:]
    assert (z - (a / (1 + torch.exp(-a))) * b).abs().max() <= 1e-6
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    parts = _rand(2, 9, 272, seed=3)
    got = torch.zeros(3, 272, device=DEV)
    ops.gather_rows(gu, rows, got, partials=parts)
    assert torch.equal(got, (gu + (parts[0] + parts[1]))[rows.long()])


@pytest.mark.parametrize("M,K,wdtype,xdtype", [(333, 2048, torch.bfloat16, torch.float32), (70, 1000, torch.float32, torch.float32),
                                               (129, 203, torch.bfloat16, torch.float32), (64, 512, torch.bfloat16, torch.bfloat16),
                                               (3, 52008, torch.bfloat16, torch.float32), (1, 264, torch.float32, torch.float32)])
def test_gemm_f32_does_not_depend_on_the_batch(M, K, wdtype, xdtype):
    """One token is a stream over the weights by persistent warps (the token in shared memory, or, too wide for that, the
    tile kernel with a tile of one); 2 to 4, 5 to 16 and more tokens take tiles of three shapes; a K that is no multiple
    of eight takes the element-wise loads. A token has the same bits from all of them, alone or among others, stored or
    added to what was there."""
    from stride_b200.kernels import ops
    x = _rand(40, K, seed=5, dtype=xdtype)
    w = _rand(M, K, seed=6, dtype=wdtype)
    base = _rand(40, M, seed=7)
    tiles, tiles_acc = torch.zeros(40, M, device=DEV), base.clone()
    ops.gemm_f32(x, w, tiles)
    ops.gemm_f32(x, w, tiles_acc, accumulate=True)
    ref = x.double() @ w.double().T
    assert (tiles.double() - ref).abs().max() <= 2e-6 * float(ref.abs().max()) * math.sqrt(K)
    for rows in ([3], [0, 1], list(range(5, 21)), list(range(24, 37))):
        xs = x[rows].contiguous()
        out, acc = torch.zeros(len(rows), M, device=DEV), base[rows].clone()
        ops.gemm_f32(xs, w, out)
        ops.gemm_f32(xs, w, acc, accumulate=True)
        assert torch.equal(out, tiles[rows]) and torch.equal(acc, tiles_acc[rows]), f"{len(rows)} tokens"


@pytest.mark.parametrize("n,M,K,wdtype", [(5, 77, 33, torch.float32), (70, 130, 200, torch.bfloat16), (1, 1000, 64, torch.bfloat16)])
def test_gemm_f32(n, M, K, wdtype):
    from stride_b200.kernels import ops
    x = _rand(n, K, seed=1)
    w = _rand(M, K, seed=2, dtype=wdtype)
    ref = (x.double() @ w.double().T)
    out = torch.zeros(n, M, device=DEV)
    ops.gemm_f32(x, w, out)
    assert (out.double() - ref).abs().max() <= 2e-6 * float(ref.abs().max()) * math.sqrt(K)
    base = _rand(n, M, seed=3)
    acc = base.clone()
    ops.gemm_f32(x, w, acc, accumulate=True)
    assert (acc.double() - (base.double() + ref)).abs().max() <= 2e-6 * float(ref.abs().max()) * math.sqrt(K)


@pytest.mark.parametrize("Hq,Hkv,D,rot", [(3, 1, 24, 16), (5, 2, 32, 32), (2, 1, 72, 72)])
def test_rope_append_partial_rotation_and_pages(Hq, Hkv, D, rot):
    """Rotation of the first rotary_dim elements only (or of the whole head, the vectorised kernel), q stored, k and v
    appended at (slot, pos) through the table."""
    from stride_b200.kernels import ops
    page, n = 4, 6
    qkv = _rand(2, n, (Hq + 2 * Hkv) * D, seed=1)
    pos = torch.tensor([0, 1, 2, 9, 10, 5], dtype=torch.int32, device=DEV)
    slots = torch.tensor([1, 1, 1, 0, 0, 2], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 5, 1], [0, 6, 2], [7, 4, 8]], dtype=torch.int32, device=DEV)
    ang = (torch.arange(32, dtype=torch.float32)[:, None] * torch.linspace(1.0, 0.1, rot // 2)[None]).double()
    cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], -1).float().to(DEV)
    cache = torch.zeros(9, 2, Hkv, page, D, device=DEV)
    q_out = torch.zeros(n, Hq * D, device=DEV)
    ops.rope_append(qkv, pos, slots, cos_sin, rot, q_out, cache, table, Hq, Hkv, D)
    full = (qkv[0] + qkv[1]).reshape(n, Hq + 2 * Hkv, D).cpu()
    c, s = cos_sin.cpu()[pos.cpu().long(), :, 0][:, None], cos_sin.cpu()[pos.cpu().long(), :, 1][:, None]

    def rotate(x):
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., rot:]], -1)

    assert (q_out.cpu().reshape(n, Hq, D) - rotate(full[:, :Hq])).abs().max() <= 1e-6
    k_ref, v_ref = rotate(full[:, Hq:Hq + Hkv]), full[:, Hq + Hkv:]
    for i in range(n):
        pg = int(table[slots[i], pos[i] // page])
        assert (cache[pg, 0, :, int(pos[i]) % page].cpu() - k_ref[i]).abs().max() <= 1e-6
        assert torch.equal(cache[pg, 1, :, int(pos[i]) % page].cpu(), v_ref[i])
    assert float(cache.abs().sum()) > 0 and int((cache.abs().sum(dim=(1, 2, 4)) > 0).sum()) == n


def test_argmax_and_temperature_sampling():
    import plain_llama as plain
    from stride_b200.kernels import ops
    rows, V = 6, 3001
    logits = _rand(rows, V, seed=4, scale=3.0)
    logits[1, 100] = logits[1, 2000] = logits[1].max() + 1      # a tie: the smaller index wins
    logits[2, 5] = float("nan")
    tok = torch.zeros(rows, dtype=torch.int32, device=DEV)
    val = torch.zeros(rows, device=DEV)
    ops.argmax(logits, tok, val)
    clean = torch.nan_to_num(logits, nan=-float("inf")).cpu()
    for r in range(rows):
        want, _ = plain.choose_token(clean[r], 0.0, 1.0, 0, 0, 1)
        assert int(tok[r]) == want and float(val[r]) == float(clean[r, want])
    temps = torch.tensor([0.8, 1.0, 0.5, 2.0, 0.05, 1.3], device=DEV)
    seeds = torch.tensor([1, 2**62 + 5, 3, -7, 5, 6], dtype=torch.int64, device=DEV)
    for length in (1, 17, 300, 4097):
        lengths = torch.full((rows,), length, dtype=torch.int32, device=DEV)
        ops.sample_temperature(torch.nan_to_num(logits, nan=-1e30), temps, seeds, lengths, tok, val)
        for r in range(rows):
            l = torch.nan_to_num(logits[r], nan=-1e30).cpu()
            want, wv = plain.choose_token(l, float(temps[r]), 1.0, 0, int(seeds[r]) & (2**64 - 1), length)
            assert int(tok[r]) == want and float(val[r]) == wv


@pytest.mark.parametrize("temperature", [0.02, 0.7, 1.5, 50.0])
def test_temperature_sampling_follows_the_plain_sampler_at_every_temperature(temperature):
    """The two-level search (bins of the distance from the largest logit, then the logit's bits) picks the plain
    sampler's token whether the temperature leaves one candidate or spreads the draw over the whole vocabulary; equal
    logits rank by index; masked (-inf) and not-a-number logits are never drawn."""
    import plain_llama as plain
    from stride_b200.kernels import ops
    rows, V = 4, 12007
    logits = _rand(rows, V, seed=31, scale=2.5)
    logits[1, 100:140] = logits[1].max()            # forty equal maxima
    logits[2, ::3] = -float("inf")
    logits[3, 7] = float("nan")
    temps = torch.full((rows,), temperature, device=DEV)
    tok = torch.zeros(rows, dtype=torch.int32, device=DEV)
    val = torch.zeros(rows, device=DEV)
    clean = torch.nan_to_num(logits, nan=-float("inf")).cpu()
    for length in (3, 90, 2500):
        seeds = torch.tensor([11, 2**63 - 9, 5, 77], dtype=torch.int64, device=DEV)
        lengths = torch.full((rows,), length, dtype=torch.int32, device=DEV)
        ops.sample_temperature(logits, temps, seeds, lengths, tok, val)
        for r in range(rows):
            want, wv = plain.choose_token(clean[r], temperature, 1.0, 0, int(seeds[r]), length)
            assert int(tok[r]) == want and float(val[r]) == wv, (temperature, length, r)


def test_temperature_sampling_among_equal_logits():
    """Vocabularies of equal logits (all of them, or all but a few): every token weighs the same and the draw picks by
    index; far more candidates than a CTA lists, so the walks over the whole row take over."""
    import plain_llama as plain
    from stride_b200.kernels import ops
    rows, V = 3, 20011
    logits = torch.full((rows, V), 1.25, device=DEV)
    logits[1, 5:9] = -3.0
    logits[2, ::2] = 1.25000012                       # two values one step of float32 apart
    temps = torch.tensor([1.0, 0.6, 2.0], device=DEV)
    tok = torch.zeros(rows, dtype=torch.int32, device=DEV)
    val = torch.zeros(rows, device=DEV)
    for length in (1, 50, 51, 3000):
        seeds = torch.tensor([9, 10, 11], dtype=torch.int64, device=DEV)
        lengths = torch.full((rows,), length, dtype=torch.int32, device=DEV)
        ops.sample_temperature(logits, temps, seeds, lengths, tok, val)
        for r in range(rows):
            want, wv = plain.choose_token(logits[r].cpu(), float(temps[r]), 1.0, 0, int(seeds[r]), length)
            assert int(tok[r]) == want and float(val[r]) == wv, (length, r, int(tok[r]), want)


def test_temperature_sampling_of_a_large_vocabulary_on_a_cluster():
    """70,001 logits a row: eight CTAs share a row, their histograms joined through distributed shared memory."""
    import plain_llama as plain
    from stride_b200.kernels import ops
    rows, V = 3, 70001
    logits = _rand(rows, V, seed=41, scale=3.0)
    logits[1, 60000:60020] = logits[1].max()         # equal maxima in the last CTA's slice
    logits[2, 8740:8770] = logits[2].max() + 3.0     # thirty equal maxima across the border of the first two slices (8,752)
    temps = torch.tensor([0.9, 0.3, 0.05], device=DEV)
    seeds = torch.tensor([3, 4, 5], dtype=torch.int64, device=DEV)
    tok = torch.zeros(rows, dtype=torch.int32, device=DEV)
    val = torch.zeros(rows, device=DEV)
    for length in (10, 777, 778, 779, 780, 2000):
        lengths = torch.full((rows,), length, dtype=torch.int32, device=DEV)
        ops.sample_temperature(logits, temps, seeds, lengths, tok, val)
        for r in range(rows):
            want, wv = plain.choose_token(logits[r].cpu(), float(temps[r]), 1.0, 0, int(seeds[r]), length)
            assert int(tok[r]) == want and float(val[r]) == wv, (length, r)


def test_argmax_of_a_large_vocabulary_in_slices():
    """A large vocabulary is cut into slices, one CTA each: the largest logit and the smallest index among equals still
    win, whichever slices they lie in; not-a-numbers are passed over; a second call finds the library's words clean."""
    from stride_b200.kernels import ops
    rows, V = 5, 70003
    for call in range(3):
        logits = _rand(rows, V, seed=20 + call, scale=2.0)
        top = float(logits.max()) + 1.0
        logits[0, 69000] = logits[0, 41] = logits[0, 30000] = top       # equal maxima in three slices: index 41 wins
        logits[1, V - 1] = top                                          # the very last logit
        logits[2, 17] = float("nan")
        logits[2, 5000] = top
        logits[3] = float("nan")                                        # nothing to choose from: token 0
        slots = torch.tensor([3, 0, 4, 1, 2], dtype=torch.int32, device=DEV)
        table = torch.full((5,), -1, dtype=torch.int32, device=DEV)
        tok = torch.full((rows,), -5, dtype=torch.int32, device=DEV)
        val = torch.zeros(rows, device=DEV)
        ops.argmax(logits, tok, val, slots, table)
        clean = torch.nan_to_num(logits, nan=-float("inf"))
        want = clean.argmax(dim=1)
        assert tok.tolist()[:3] == [41, V - 1, 5000] and int(tok[3]) == 0 and int(tok[4]) == int(want[4])
        assert float(val[0]) == top and float(val[4]) == float(clean[4, want[4]])
        assert table[slots.long()].tolist() == tok.tolist()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Hq,Hkv,page,window", [(8, 2, 16, 0), (4, 4, 8, 0), (12, 4, 64, 100), (16, 1, 128, 0), (6, 2, 256, 0), (32, 8, 64, 0)])
def test_attention_tc5_against_plain(Hq, Hkv, page, window, D):
    """The tcgen05 prompt-attention kernel at both head sizes: portions with and without cached history, several key
    tiles, shuffled pages, ratios that do and do not divide 128, one far key that dominates a query."""
    from stride_b200.kernels import ops
    assert ops.attention_tc5_supported(Hq, Hkv, D, page)
    new = [77, 200, 40, 130, 64, 300]
    old = [0, 100, 510, 5, 63, 0]
    case = _paged_case(new, old, Hq, Hkv, D, page, torch.bfloat16, seed=Hq + page, peak=(2, 3))
    G = Hq // Hkv
    ppt = 128 // G
    tiles = [x for e, L in enumerate(new) for t in range(-(-L // ppt)) for x in (e, t)]
    work = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    out = torch.full_like(case["q"], float("nan"))
    scale = 1.0 / math.sqrt(D)
    ops.attention_tc5(case["q"], out, case["cache"], case["table"], case["meta"], work, len(tiles) // 2, Hq, Hkv, D, window, scale)
    assert ops.attention_tc5_status() == 0
    ref = _attention_reference(case, Hq, Hkv, D, window)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))
