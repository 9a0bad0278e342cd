"""The layer sizes of the real models (Llama 3.2 1B / 3B, Llama 3.1 8B) with one or two layers and random weights:
the same comparisons as for the tiny configurations, so that tile edges, split-K ranges, the large vocabulary, the
head ratio 3 and head size 128 are exercised at the sizes that are served."""
from __future__ import annotations

import pytest
import torch

import plain_llama as plain
from conftest import bf16_noise, check_mean_deviation, logit_tolerance, random_tokens

pytestmark = pytest.mark.gpu

ROPE = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 8192}
SHAPES = {
    "1b": {"architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 2,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "rope_theta": 500000.0,
           "rope_scaling": ROPE, "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096},
    "3b": {"architectures": ["LlamaForCausalLM"], "hidden_size": 3072, "intermediate_size": 8192, "num_hidden_layers": 1,
           "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256, "rope_theta": 500000.0,
           "rope_scaling": ROPE, "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096},
    "8b": {"architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 1,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256, "rope_theta": 500000.0,
           "rope_scaling": dict(ROPE, factor=8.0), "tie_word_embeddings": False, "rms_norm_eps": 1e-5,
           "max_position_embeddings": 8192},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["1b", "3b", "8b"])
def test_real_layer_sizes(name, dtype):
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.weights.random_init import random_tensors
    cfg_dict = SHAPES[name]
    # weights N(0, 0.05) and gains 1 + 0.1 N: larger than the 0.02 of a fresh model, so that attention is not uniform
    tensors = random_tensors(cfg_dict, seed=1, std=0.05, gain_std=0.1)
    cfg = plain.PlainConfig.from_dict(cfg_dict)
    reqs = [random_tokens(cfg.vocab_size, n, 30 + n) for n in (300, 160)]
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = [plain.forward(cfg, tensors, r, torch.float32, act) for r in reqs]
    noise = [bf16_noise(cfg, tensors, r) if act is not None else None for r in reqs]
    eng = Engine(None, EngineOptions(dtype=dtype, max_rows=320, max_full_rows=320, max_slots=4, kv_pages=12, page_size=64,
                                     max_context=512), config=cfg_dict, tensors=tensors)
    cm = eng.cache
    slots = [cm.acquire_slot() for _ in reqs]

    def check(logits, i, a, b, what):
        ref = want[i][a:b]
        got = logits.cpu()
        tol = logit_tolerance(dtype, ref, noise[i])
        assert (got - ref).abs().max() <= tol, f"{name} {dtype} {what}: {(got - ref).abs().max():.3e} > {tol:.3e}"

    # request 0: 257 tokens in one step (two tcgen05 tiles and a bit), then a portion of 11 beside request 1's first 150,
    # then both decode token by token, request 1 starting a step later
    assert cm.ensure(slots[0], 257)
    check(eng.step([StepEntry(slots[0], 0, reqs[0][:257], list(range(257)))]), 0, 0, 257, "prompt of 257")
    assert cm.ensure(slots[0], 268) and cm.ensure(slots[1], 140)
    lg = eng.step([StepEntry(slots[0], 257, reqs[0][257:268], list(range(11))), StepEntry(slots[1], 0, reqs[1][:140], [0, 70, 139])])
    check(lg[:11], 0, 257, 268, "portion of 11")
    assert (lg[11:].cpu() - want[1][[0, 70, 139]]).abs().max() <= logit_tolerance(dtype, want[1], noise[1])
    fed = [268, 140]
    for k in range(12):
        entries = []
        for i in (0, 1):
            if i == 1 and k == 0:
                continue
            n = 1 if k % 5 else 2          # now and then two tokens at once
            n = min(n, len(reqs[i]) - fed[i])
            if n == 0:
                continue
            assert cm.ensure(slots[i], fed[i] + n)
            entries.append((i, StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + n], list(range(n)))))
        lg = eng.step([e for _, e in entries])
        at = 0
        for i, e in entries:
            n = len(e.tokens)
            check(lg[at:at + n], i, fed[i], fed[i] + n, f"decode step {k}")
            at += n
            fed[i] += n
    if dtype == "bfloat16":
        from stride_b200.kernels import ops
        assert ops.gemm_tc_status() == 0
        if cfg.head_dim == 64:
            assert ops.attention_tc5_status() == 0
    for s in slots:
        cm.release_slot(s)
    cm.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bits_do_not_depend_on_the_batch(dtype):
    """With the 1B layer sizes (whose attention and down projections are cut into K ranges): a request has the same
    logits, bit for bit, alone and among other requests, whatever their number, their order in the batch, the size of
    the step (1 token or 400), the pages it gets and the portions it is fed in."""
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.weights.random_init import random_tensors
    cfg_dict = SHAPES["1b"]
    tensors = random_tensors(cfg_dict, seed=2, std=0.05, gain_std=0.1)
    vocab = cfg_dict["vocab_size"]
    mine = random_tokens(vocab, 90, 5)
    others = [random_tokens(vocab, 450, 6 + i) for i in range(5)]
    cuts = [(0, 70), (70, 75), (75, 76), (76, 77), (77, 79), (79, 80)] + [(p, p + 1) for p in range(80, 90)]

    def run(seed, company, cuts=cuts):
        """company[k]: for step k a list of (other request, tokens it brings), placed before or after mine."""
        eng = Engine(None, EngineOptions(dtype=dtype, max_rows=512, max_full_rows=96, max_slots=8, kv_pages=48, page_size=64,
                                         max_context=512, kv_shuffle_seed=seed), config=cfg_dict, tensors=tensors)
        cm = eng.cache
        slots = {}
        fed = {}
        out = []
        for k, (a, b) in enumerate(cuts):
            entries = []
            for j, n in company[k] if k < len(company) else []:
                if j not in slots:
                    slots[j], fed[j] = cm.acquire_slot(), 0
                assert cm.ensure(slots[j], fed[j] + n)
                entries.append(StepEntry(slots[j], fed[j], others[j][fed[j]:fed[j] + n], []))
                fed[j] += n
            if "me" not in slots:
                slots["me"] = cm.acquire_slot()
            assert cm.ensure(slots["me"], b)
            me = StepEntry(slots["me"], a, mine[a:b], list(range(b - a)))
            at = (k * 7 + seed) % (len(entries) + 1)
            entries.insert(at, me)
            out.append(eng.step(entries).clone())
        return torch.cat(out)

    alone = run(0, [])
    decoders = [[(j, 40)] for j in range(3)]                         # three others start ..
    decoders = [sum(decoders, [])] + [[(0, 1), (1, 1), (2, 1)]] * 20    # .. and then decode beside me
    among_decoders = run(3, decoders)
    big = [[(0, 150)], [(1, 300), (0, 1)], [(2, 60), (1, 1)], [(3, 399)], [(4, 130), (3, 1)]] + [[(0, 1), (4, 200)]] + [[(0, 1), (1, 1), (2, 1), (3, 1)]] * 12
    among_prompts = run(11, big)
    assert torch.equal(alone, among_decoders)
    assert torch.equal(alone, among_prompts)
    # nor on how the request itself is cut into steps: whole, token by token, in portions beside other requests
    assert torch.equal(alone, run(5, [], [(0, 90)]))
    assert torch.equal(alone, run(6, [], [(p, p + 1) for p in range(90)]))
    assert torch.equal(alone, run(7, big, [(0, 3), (3, 40), (40, 42), (42, 43), (43, 90)]))


def test_serving_under_pressure_keeps_every_request_exact():
    """The 1B layer sizes (four layers) through the public entry point: 40 requests of 200 to 300 tokens, 24 at a time, in
    a pool that cannot hold them all, so that some are preempted and replayed; greedy and sampled requests mixed in one
    run. Every request ends with exactly the tokens (and the bits of the chosen logits) it gets when it runs alone."""
    from stride_b200 import LLM, Engine, EngineOptions
    from stride_b200.weights.random_init import random_tensors
    cfg = dict(SHAPES["1b"], num_hidden_layers=4)
    tensors = random_tensors(cfg, seed=3, std=0.05, gain_std=0.1)
    vocab = cfg["vocab_size"]
    prompts = [random_tokens(vocab, 200 + (37 * i) % 101, 900 + i) for i in range(40)]
    new = 48

    def engine(pages):
        return Engine(None, EngineOptions(dtype="bfloat16", max_rows=512, max_full_rows=64, max_slots=32, kv_pages=pages, page_size=64,
                                          max_context=512), config=cfg, tensors=tensors)

    busy = LLM(engine=engine(24 * 4), concurrency=24, max_rows=512, prefill_chunk=128, row_shuffle_seed=5)
    got = busy.generate(prompts, new, temperature=0.7, seed=11)
    stats = busy.last_stats
    assert stats.preemptions > 0 and stats.replayed_rows > 0
    busy.engine.cache.check()
    assert busy.engine.cache.free_pages() == busy.engine.cache.total_pages()
    alone = LLM(engine=engine(16), concurrency=1, max_rows=512, prefill_chunk=512)
    for i in (0, 7, 13, 22, 31, 39):
        (want,) = alone.generate([prompts[i]], new, temperature=0.7, seed=11 + i)
        assert got[i].tokens == want.tokens, f"request {i}"
        assert got[i].values == want.values, f"request {i}: the chosen logits differ in bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_of_2048_tokens_whole_in_portions_and_in_company(dtype):
    """The step the prefill figure is measured on, at the 1B layer sizes (two layers): one prompt of 2,048 tokens fed
    whole, in portions of 256, and as 1,100 + 948 beside two requests that decode. Above 512 tokens the projections with
    K ranges add their ranges in registers, above 1,536 rows the norm runs a warp per row, and the tcgen05 attention walks
    sixteen tiles of one request: the logits at the first place, at tile and portion edges and at the last place are the
    same bits in all three, and the plain implementation's within tolerance."""
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.weights.random_init import random_tensors
    cfg_dict = SHAPES["1b"]
    tensors = random_tensors(cfg_dict, seed=4, std=0.05, gain_std=0.1)
    cfg = plain.PlainConfig.from_dict(cfg_dict)
    T = 2048
    mine = random_tokens(cfg.vocab_size, T, 77)
    others = [random_tokens(cfg.vocab_size, 90, 78), random_tokens(cfg.vocab_size, 140, 79)]
    places = sorted({0, 1, 63, 64, 127, 128, 129, 255, 256, 257, 511, 512, 513, 767, 768, 1023, 1024, 1099, 1100, 1101, 1279,
                     1280, 1535, 1536, 1537, 1791, 1792, 1919, 1920, 2046, 2047})
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = plain.forward(cfg, tensors, mine, torch.float32, act, rows=places)
    noise = bf16_noise(cfg, tensors, mine, rows=places) if act is not None else None

    def engine(seed):
        return Engine(None, EngineOptions(dtype=dtype, max_rows=2048, max_full_rows=64, max_slots=4, kv_pages=40, page_size=64,
                                          max_context=2048, kv_shuffle_seed=seed), config=cfg_dict, tensors=tensors)

    def feed(eng, slot, cuts, company=None):
        """Feeds `mine` in the portions `cuts`; returns the logits at `places`, in order."""
        cm, out = eng.cache, []
        for a, b in cuts:
            assert cm.ensure(slot, b)
            me = StepEntry(slot, a, mine[a:b], [p - a for p in places if a <= p < b])
            entries = [me] if company is None else company(me)
            lg = eng.step(entries)
            at = sum(len(e.want) for e in entries[:entries.index(me)])
            out.append(lg[at:at + len(me.want)].clone())
        return torch.cat(out).cpu()

    eng = engine(0)
    whole = feed(eng, eng.cache.acquire_slot(), [(0, T)])
    tol = logit_tolerance(dtype, want, noise)
    assert (whole - want).abs().max() <= tol, f"{dtype} whole: {(whole - want).abs().max():.3e} > {tol:.3e}"
    if noise is not None:
        check_mean_deviation(whole, want, noise, "2,048 tokens whole")
    del eng

    eng = engine(3)
    portions = feed(eng, eng.cache.acquire_slot(), [(a, a + 256) for a in range(0, T, 256)])
    assert torch.equal(whole, portions), f"portions of 256 differ from the whole prompt by {(whole - portions).abs().max():.3e}"
    del eng

    eng = engine(5)
    cm = eng.cache
    slots = [cm.acquire_slot() for _ in range(3)]
    fed = [60, 100]
    for j in (0, 1):                   # the two others: most of their prompt first ..
        assert cm.ensure(slots[1 + j], fed[j])
        eng.step([StepEntry(slots[1 + j], 0, others[j][:fed[j]], [])])

    def company(me):                   # .. then each decodes one token beside every portion of mine
        entries = []
        for j in (0, 1):
            assert cm.ensure(slots[1 + j], fed[j] + 1)
            entries.append(StepEntry(slots[1 + j], fed[j], others[j][fed[j]:fed[j] + 1], [0]))
            fed[j] += 1
        return [entries[0], me, entries[1]]

    mixed = feed(eng, slots[0], [(0, 1100), (1100, T)], company)
    assert torch.equal(whole, mixed), f"1,100 + 948 beside two decoding requests differ from the whole prompt by {(whole - mixed).abs().max():.3e}"
    if dtype == "bfloat16":
        from stride_b200.kernels import ops
        assert ops.gemm_tc_status() == 0 and ops.attention_tc5_status() == 0


LONG = {"architectures": ["LlamaForCausalLM"], "hidden_size": 128, "intermediate_size": 192, "num_hidden_layers": 1,
        "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 64, "vocab_size": 300, "rope_theta": 10000.0,
        "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 9000}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_over_a_long_context_alone_and_in_company(dtype):
    """A context of 8,448 tokens (34 chunks of 256 keys, 67 tiles of 128) and eight decoded tokens, at a small width.
    The decoded tokens' attention folds tens of partial results: in bfloat16 by a kernel of its own that streams the
    chunks' records when the step's entries are few, by the entry's last CTA when they are many; in float32 by a cluster
    of blocks per head or by one block. The long request decodes alone, beside one other request and beside eighty:
    the same bits each time, and the plain implementation's logits within tolerance."""
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.weights.random_init import random_tensors
    tensors = random_tensors(LONG, seed=8, std=0.2, gain_std=0.2)
    cfg = plain.PlainConfig.from_dict(LONG)
    P, N = 8448, 8
    seq = random_tokens(cfg.vocab_size, P + N, 91)
    places = [100, P - 1] + list(range(P, P + N))
    act = torch.bfloat16 if dtype == "bfloat16" else None
    want = plain.forward(cfg, tensors, seq, torch.float32, act, rows=places)
    noise = bf16_noise(cfg, tensors, seq, rows=places) if act is not None else None

    def run(portion, others):
        eng = Engine(None, EngineOptions(dtype=dtype, max_rows=2112, max_full_rows=96, max_slots=84, kv_pages=240, page_size=64,
                                         max_context=9000, kv_shuffle_seed=others), config=LONG, tensors=tensors)
        cm = eng.cache
        mine = cm.acquire_slot()
        out = []
        for a in range(0, P, portion):
            b = min(P, a + portion)
            assert cm.ensure(mine, b)
            lg = eng.step([StepEntry(mine, a, seq[a:b], [p - a for p in places if a <= p < b])])
            if lg is not None:
                out.append(lg.clone())
        company = []
        for j in range(others):
            slot = cm.acquire_slot()
            toks = random_tokens(cfg.vocab_size, 3 + N, 200 + j)
            assert cm.ensure(slot, 3)
            eng.step([StepEntry(slot, 0, toks[:3], [])])
            company.append((slot, toks))
        for k in range(N):
            entries = []
            for slot, toks in company:
                assert cm.ensure(slot, 4 + k)
                entries.append(StepEntry(slot, 3 + k, toks[3 + k:4 + k], [0]))
            assert cm.ensure(mine, P + k + 1)
            me = StepEntry(mine, P + k, seq[P + k:P + k + 1], [0])
            entries.insert(len(entries) // 2, me)
            out.append(eng.step(entries)[entries.index(me)].clone()[None])
        return torch.cat(out).cpu()

    alone = run(2112, 0)
    tol = logit_tolerance(dtype, want, noise)
    assert (alone - want).abs().max() <= tol, f"{dtype}: {(alone - want).abs().max():.3e} > {tol:.3e}"
    assert torch.equal(run(1000, 1), alone), "beside one other request"
    assert torch.equal(run(2112, 80), alone), "beside eighty other requests"
    if dtype == "bfloat16":
        from stride_b200.kernels import ops
        assert ops.gemm_tc_status() == 0 and ops.attention_tc5_status() == 0
