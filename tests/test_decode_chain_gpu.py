"""The decode chain (all layers of a step of decoded tokens as one persistent kernel) against the layers' separate
kernels: every phase does the arithmetic of the kernel it stands for, so logits and cache are equal bit for bit,
for every batch size and context the chain takes, directly and from CUDA graphs; steps it does not take (a prompt
portion among them, more tokens than it holds) run as before."""
from __future__ import annotations

import pytest
import torch

from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu


def _engines(name, model_dirs, **kw):
    from stride_b200 import Engine, EngineOptions
    page = TINY[name][2]
    opts = dict(dtype="bfloat16", max_rows=96, max_full_rows=96, max_slots=80, kv_pages=160, page_size=page)
    opts.update(kw)
    make = lambda chain: Engine(model_dirs[name], EngineOptions(decode_chain=chain, **opts))
    return make(True), make(False)


def _chain_of(engine):
    return engine._program.chains[0] if engine._program is not None and engine._program.chains else None


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "U"])
def test_the_chain_gives_the_bits_of_the_separate_kernels(name, model_dirs):
    from stride_b200 import StepEntry
    D, G = TINY[name][0].get("head_dim", TINY[name][0]["hidden_size"] // TINY[name][0]["num_attention_heads"]), \
        TINY[name][0]["num_attention_heads"] // TINY[name][0]["num_key_value_heads"]
    chained, separate = _engines(name, model_dirs)
    if D not in (64, 128) or G > 16:
        assert _chain_of(chained) is None, "head sizes without a tensor-core decode kernel have no chain"
        pytest.skip(f"configuration {name} (head size {D}) has no decode chain")
    assert _chain_of(chained) is not None and len(_chain_of(chained)) == 7 * TINY[name][0]["num_hidden_layers"]
    assert _chain_of(separate) is None
    vocab = TINY[name][0]["vocab_size"]
    limit = TINY[name][0]["max_position_embeddings"] - 2
    lengths = [min(limit, n) for n in (300, 37, 64, 5, 129, 255, 256, 1)]
    reqs = [random_tokens(vocab, n + 12, 900 + i) for i, n in enumerate(lengths)]
    outs = []
    for eng in (chained, separate):
        cm, got = eng.cache, []
        slots = [cm.acquire_slot() for _ in reqs]
        fed = [0] * len(reqs)
        # the prompts, in portions (these steps the chain does not take)
        for i, n in enumerate(lengths):
            while fed[i] < n:
                k = min(90, n - fed[i])
                assert cm.ensure(slots[i], fed[i] + k)
                got.append(eng.step([StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + k], [k - 1])]).clone())
                fed[i] += k
        launches = []
        # decoded tokens: all requests (a graph step), some of them with wanted places of their own (a direct step),
        # two tokens of one request beside single ones (short portions are items of the decode kernel too)
        for k in range(10):
            entries = []
            for i in range(len(reqs)):
                if k % 3 == 1 and i % 2:
                    continue
                take = 2 if (k % 3 == 2 and i == 1) else 1
                if fed[i] + take > len(reqs[i]) or fed[i] + take > limit + 1:
                    continue
                assert cm.ensure(slots[i], fed[i] + take)
                entries.append(StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + take], list(range(take))))
                fed[i] += take
            if k % 2:
                entries.reverse()
            from stride_b200.kernels import ops
            before = ops.launches
            got.append(eng.step(entries).clone())
            launches.append(ops.launches - before)
        outs.append((got, launches))
        eng.check_kernels()
    (a, la), (b, lb) = outs
    assert len(a) == len(b)
    for k, (x, y) in enumerate(zip(a, b)):
        assert torch.equal(x, y), f"{name} step {k}: the chain and the separate kernels differ by {(x - y).abs().max():.3e}"
    for g in range(len(chained.cache.groups)):
        assert torch.equal(chained.cache.groups[g].arena, separate.cache.groups[g].arena), "the two left different caches"
    # the chain did run: a direct decode step launches far fewer kernels with it (graph replays launch none through ops)
    direct = [(x, y) for x, y in zip(la, lb) if y > 0]
    assert direct and all(x < y / 3 for x, y in direct), (la, lb)


@pytest.mark.parametrize("batch", [1, 7, 16, 17, 33, 64, 65])
def test_every_batch_size_and_long_contexts(batch, model_dirs):
    """Token tiles of 16, 32 and 64; 65 tokens are more than the chain takes (the separate kernels run); contexts that
    span several 256-key chunks, so that a CTA computes several attention units and the chunk records are folded."""
    from stride_b200 import StepEntry
    name = "D"
    chained, separate = _engines(name, model_dirs, max_rows=160, max_full_rows=80, kv_pages=70 * 40)
    vocab = TINY[name][0]["vocab_size"]
    limit = TINY[name][0]["max_position_embeddings"] - 2
    lengths = [min(limit - 8, 20 + (131 * i) % 580) for i in range(batch)]
    reqs = [random_tokens(vocab, n + 6, 2000 + i) for i, n in enumerate(lengths)]
    outs = []
    for eng in (chained, separate):
        cm, got = eng.cache, []
        slots = [cm.acquire_slot() for _ in reqs]
        fed = [0] * batch
        for i, n in enumerate(lengths):
            while fed[i] < n:
                k = min(150, n - fed[i])
                assert cm.ensure(slots[i], fed[i] + k)
                eng.step([StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + k], [])])
                fed[i] += k
        for k in range(6):
            entries = []
            for i in range(batch):
                assert cm.ensure(slots[i], fed[i] + 1)
                entries.append(StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + 1], [0]))
                fed[i] += 1
            got.append(eng.step(entries).clone())
        outs.append(got)
        eng.check_kernels()
    for k, (x, y) in enumerate(zip(*outs)):
        assert torch.equal(x, y), f"batch {batch} step {k}: {(x - y).abs().max():.3e}"
    for g in range(len(chained.cache.groups)):
        assert torch.equal(chained.cache.groups[g].arena, separate.cache.groups[g].arena)


def test_generation_with_and_without_the_chain(model_dirs):
    from stride_b200 import LLM, Engine, EngineOptions
    vocab = TINY["D"][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 600 + n) for n in (3, 90, 41, 130, 17, 64, 200, 9)]
    results = []
    for chain in (True, False):
        eng = Engine(model_dirs["D"], EngineOptions(dtype="bfloat16", max_rows=96, max_full_rows=8, max_slots=6, kv_pages=40, page_size=16,
                                                    decode_chain=chain))
        llm = LLM(engine=eng, concurrency=5, max_rows=96, prefill_chunk=48)
        outs = llm.generate(prompts, max_new_tokens=40, temperature=0.7, seed=3)
        results.append([(o.tokens, o.values, o.fingerprint) for o in outs])
        eng.cache.check()
        eng.check_kernels()
    assert results[0] == results[1]


def test_head_size_128_and_sizes_that_are_no_power_of_two(tmp_path):
    """Head size 128, ratio 3, a width of 320 (five blocks of K, so that the K ranges are uneven), pages of 64."""
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.weights.random_init import write_random_model
    from conftest import TEST_GAIN_STD, TEST_STD
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": 320, "intermediate_size": 448, "num_hidden_layers": 2,
           "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 300, "rope_theta": 10000.0,
           "tie_word_embeddings": False, "rms_norm_eps": 1e-6, "max_position_embeddings": 600}
    folder = write_random_model(tmp_path / "m", cfg, 31, std=TEST_STD, gain_std=TEST_GAIN_STD)
    lengths = [290, 5, 511, 64]
    reqs = [random_tokens(300, n + 8, 70 + i) for i, n in enumerate(lengths)]
    outs = []
    for chain in (True, False):
        eng = Engine(folder, EngineOptions(dtype="bfloat16", max_rows=128, max_full_rows=16, max_slots=6, kv_pages=40, page_size=64, decode_chain=chain))
        assert bool(eng._program.chains) == chain
        cm, got = eng.cache, []
        slots = [cm.acquire_slot() for _ in reqs]
        fed = [0] * len(reqs)
        for i, n in enumerate(lengths):
            while fed[i] < n:
                k = min(128, n - fed[i])
                assert cm.ensure(slots[i], fed[i] + k)
                eng.step([StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + k], [])])
                fed[i] += k
        for k in range(8):
            entries = []
            for i in range(len(reqs)):
                assert cm.ensure(slots[i], fed[i] + 1)
                entries.append(StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + 1], [0]))
                fed[i] += 1
            got.append(eng.step(entries).clone())
        outs.append((got, [g.arena.clone() for g in cm.groups]))
        eng.check_kernels()
    for k, (x, y) in enumerate(zip(outs[0][0], outs[1][0])):
        assert torch.equal(x, y), f"step {k}: {(x - y).abs().max():.3e}"
    for a, b in zip(outs[0][1], outs[1][1]):
        assert torch.equal(a, b)
