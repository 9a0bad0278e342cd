"""The native step program against the Python driver: both launch the same kernels with the same arguments, so
every step gives the same logits bit for bit and leaves the same cache, whatever the step is made of."""
from __future__ import annotations

import pytest
import torch

from conftest import TINY, random_tokens

pytestmark = pytest.mark.gpu


def _engines(name, dtype, model_dirs, **kw):
    from stride_b200 import Engine, EngineOptions
    page = TINY[name][2]
    make = lambda native: Engine(model_dirs[name], EngineOptions(dtype=dtype, max_rows=192, max_full_rows=192, max_slots=6, kv_pages=64,
                                                                 page_size=page, native_step=native, **kw))
    return make(True), make(False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_native_program_equals_the_python_driver(name, dtype, model_dirs):
    from stride_b200 import StepEntry
    native, python = _engines(name, dtype, model_dirs)
    assert native._program is not None and len(native._program) > 0, "the Llama parts all have a native form"
    assert python._program is None
    vocab = TINY[name][0]["vocab_size"]
    limit = min(120, TINY[name][0]["max_position_embeddings"] - 2)
    reqs = [random_tokens(vocab, n, 400 + i) for i, n in enumerate((limit, 37, 64, 5))]
    # steps: (request, tokens it brings); whole prompts, portions down to two tokens, single tokens, all mixed,
    # entries in changing order, some steps wanting no logits at all
    plan = [[(0, 50)], [(1, 20), (0, 2)], [(2, 64), (0, 1), (1, 1)], [(3, 3), (0, 1)], [(0, 1), (1, 1), (3, 1)], [(1, 15), (3, 1)],
            [(0, 1), (1, 0)], [(0, limit - 56)]]
    outs = []
    for eng in (native, python):
        cm = eng.cache
        slots = [cm.acquire_slot() for _ in reqs]
        fed = [0] * len(reqs)
        got = []
        for k, step in enumerate(plan):
            entries = []
            for i, n in step:
                n = min(n, len(reqs[i]) - fed[i])
                if n <= 0:
                    continue
                assert cm.ensure(slots[i], fed[i] + n)
                want = [] if k == 3 else list(range(n)) if n <= 3 else [0, n - 1]
                entries.append(StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + n], want))
                fed[i] += n
            if k % 2:
                entries.reverse()
            lg = eng.step(entries)
            got.append(None if lg is None else lg.clone())
        # decode-only steps (these run from CUDA graphs, recorded from the native program or from the Python driver)
        for _ in range(5):
            entries = []
            for i in (0, 1, 3):
                if fed[i] < len(reqs[i]):
                    assert cm.ensure(slots[i], fed[i] + 1)
                    entries.append(StepEntry(slots[i], fed[i], reqs[i][fed[i]:fed[i] + 1], [0]))
                    fed[i] += 1
            if entries:
                got.append(eng.step(entries).clone())
        outs.append(got)
        eng.check_kernels()
    assert len(outs[0]) == len(outs[1])
    for k, (a, b) in enumerate(zip(*outs)):
        assert (a is None) == (b is None), f"step {k}"
        if a is not None:
            assert torch.equal(a, b), f"{name} {dtype} step {k}: the native program and the Python driver differ by {(a - b).abs().max():.3e}"
    for g in range(len(native.cache.groups)):
        assert torch.equal(native.cache.groups[g].arena, python.cache.groups[g].arena), "the two drivers left different caches"


def test_generation_is_the_same_through_both_drivers(model_dirs):
    from stride_b200 import LLM, Engine, EngineOptions
    vocab = TINY["D"][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 600 + n) for n in (3, 90, 41, 130, 17, 64)]
    results = []
    for native in (True, False):
        eng = Engine(model_dirs["D"], EngineOptions(dtype="bfloat16", max_rows=96, max_full_rows=8, max_slots=5, kv_pages=24, page_size=16,
                                                    native_step=native))
        llm = LLM(engine=eng, concurrency=4, max_rows=96, prefill_chunk=48)
        outs = llm.generate(prompts, max_new_tokens=20, temperature=0.7, seed=3)
        results.append([(o.tokens, o.values, o.fingerprint) for o in outs])
        eng.cache.check()
    assert results[0] == results[1]
