"""Generation through the public entry point, the scheduler and the command line, on the GPU."""
from __future__ import annotations

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as plain
from conftest import ROOT, TINY, bf16_noise, logit_tolerance, random_tokens

pytestmark = pytest.mark.gpu


def _prompts(name, lengths, seed=50):
    vocab = TINY[name][0]["vocab_size"]
    return [random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("name,lengths", [("A", [5, 9, 13, 17]), ("B", [1, 40, 23, 8, 31, 17])])
def test_greedy_generation_matches_plain_float32(name, lengths, model_dirs):
    """Prompts of the two tiny workloads (4 requests of 5 to 17 tokens; 6 of 1 to 40, fed in portions of 7); float32 greedy
    tokens equal the plain implementation's, token by token."""
    from stride_b200 import LLM
    cfg, w = plain.load_plain(model_dirs[name])
    prompts = _prompts(name, lengths)
    llm = LLM(model_dirs[name], dtype="float32", concurrency=len(prompts), max_rows=64, prefill_chunk=7,
              page_size=TINY[name][2], kv_pages=64, max_slots=8)
    outs = llm.generate(prompts, max_new_tokens=16)
    for p, o in zip(prompts, outs):
        assert o.tokens == plain.generate_greedy(cfg, w, p, 16)
        assert o.finish_reason == "length"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_generation_invariant_to_schedule(name, dtype, model_dirs):
    """The same requests alone, all together, with shuffled pages and batch order, in small portions: the same tokens
    and the same bits of every logit, in both precisions (arhaamatiq/stride tests/test_correctness.py:62-73 compares
    fingerprints of tokens and chosen logits the same way)."""
    from stride_b200 import LLM
    prompts = _prompts(name, [1, 40, 23, 8, 31, 17, 3, 29])
    page = TINY[name][2]
    base = dict(dtype=dtype, max_rows=64, page_size=page, kv_pages=1024 // page, max_slots=16)
    solo = LLM(model_dirs[name], concurrency=1, prefill_chunk=64, **base).generate(prompts, 24, full_logits=True)
    variants = {
        "together": dict(concurrency=8, prefill_chunk=64),
        "chunk7 mixed": dict(concurrency=5, prefill_chunk=7, row_shuffle_seed=99, kv_shuffle_seed=5),
        "chunk2": dict(concurrency=3, prefill_chunk=2, kv_shuffle_seed=11),
        "chunk1": dict(concurrency=7, prefill_chunk=1, row_shuffle_seed=3),
    }
    for what, kw in variants.items():
        outs = LLM(model_dirs[name], **{**base, **kw}).generate(prompts, 24, full_logits=True)
        for i, (a, b) in enumerate(zip(solo, outs)):
            assert a.tokens == b.tokens, f"{what}: request {i}"
            for k in range(len(a.tokens)):
                assert np.array_equal(a.logits[k], b.logits[k]), f"{what}: request {i} token {k}: logits differ in bits"


def test_preemption_replays_to_the_same_tokens(model_dirs):
    """A pool too small for all requests at once: the youngest is preempted and recomputed, and every
    request still ends with the tokens it gets alone (arhaamatiq/stride tests/test_correctness.py:76-82)."""
    from stride_b200 import LLM
    name = "B"
    prompts = _prompts(name, [30, 12, 25, 9, 18, 27])
    solo = LLM(model_dirs[name], dtype="float32", concurrency=1, max_rows=64, page_size=8, kv_pages=64, max_slots=8)
    want = solo.generate(prompts, 40)
    tight = LLM(model_dirs[name], dtype="float32", concurrency=6, max_rows=64, prefill_chunk=9, page_size=8,
                kv_pages=22, max_slots=8, kv_shuffle_seed=3)
    got = tight.generate(prompts, 40)
    assert tight.last_stats.preemptions > 0 and tight.last_stats.replayed_rows > 0
    for a, b in zip(want, got):
        assert a.tokens == b.tokens
    tight.engine.cache.check()
    assert tight.engine.cache.free_pages() == [22]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_is_keyed_and_matches_plain(dtype, model_dirs):
    """temperature 0.8: every token equals what the plain sampler picks from the engine's own logits;
    the same at concurrency 1 and 6; another seed changes the output (tests/test_correctness.py:85-91)."""
    from stride_b200 import LLM
    name = "B"
    prompts = _prompts(name, [1, 40, 23, 8, 31, 17], seed=3)
    kw = dict(dtype=dtype, max_rows=64, page_size=8, kv_pages=128, max_slots=8)
    a = LLM(model_dirs[name], concurrency=1, **kw).generate(prompts, 20, temperature=0.8, seed=4, full_logits=True)
    for i, (p, o) in enumerate(zip(prompts, a)):
        for k, tok in enumerate(o.tokens):
            want, _ = plain.choose_token(torch.from_numpy(o.logits[k]), 0.8, 1.0, 0, 4 + i, len(p) + k)
            assert tok == want, f"request {i} token {k}"
    b = LLM(model_dirs[name], concurrency=6, prefill_chunk=7, row_shuffle_seed=9, **kw).generate(prompts, 20, temperature=0.8, seed=4)
    assert [o.tokens for o in a] == [o.tokens for o in b]
    c = LLM(model_dirs[name], concurrency=6, **kw).generate(prompts, 20, temperature=0.8, seed=5)
    assert [o.tokens for o in a] != [o.tokens for o in c]
    d = LLM(model_dirs[name], concurrency=6, **kw).generate(prompts, 12, temperature=0.7, top_p=0.9, top_k=50, seed=4, full_logits=True)
    for i, (p, o) in enumerate(zip(prompts, d)):
        for k, tok in enumerate(o.tokens):
            want, _ = plain.choose_token(torch.from_numpy(o.logits[k]), 0.7, 0.9, 50, 4 + i, len(p) + k)
            assert tok == want


def test_long_decoding_and_first_tokens(model_dirs):
    """A one-token prompt decoded for 180 tokens (crossing many pages), logits at every generated token
    against the plain implementation run on the whole sequence at once."""
    from stride_b200 import LLM
    name = "B"
    cfg, w = plain.load_plain(model_dirs[name])
    for dtype, act in (("float32", None), ("bfloat16", torch.bfloat16)):
        llm = LLM(model_dirs[name], dtype=dtype, concurrency=1, max_rows=16, page_size=8, kv_pages=32, max_slots=2)
        (o,) = llm.generate([[7]], 180, full_logits=True)
        seq = [7] + o.tokens
        ref = plain.forward(cfg, w, seq[:-1], torch.float32, act)
        got = torch.from_numpy(np.stack(o.logits))
        noise = bf16_noise(cfg, w, seq[:-1]) if act is not None else None
        assert (got - ref).abs().max() <= logit_tolerance(dtype, ref, noise)
        # the first tokens of a sequence: positions 0, 1, 2 have one, two, three keys
        assert (got[:3] - ref[:3]).abs().max() <= logit_tolerance(dtype, ref[:3], noise)


def test_stop_tokens_context_limit_and_empty_prompt(model_dirs):
    from stride_b200 import LLM
    name = "A"
    llm = LLM(model_dirs[name], dtype="float32", concurrency=4, max_rows=32, kv_pages=16, max_slots=4)
    p = _prompts(name, [6])[0]
    (free,) = llm.generate([p], 8)
    stop = free.tokens[3]
    (o,) = llm.generate([p], 8, stop_tokens=(stop,))
    k = free.tokens.index(stop)
    assert o.tokens == free.tokens[:k + 1] and o.finish_reason == "stop"
    outs = llm.generate([[], random_tokens(256, 128, 1), random_tokens(256, 126, 2)], 8)
    assert outs[0].finish_reason == "empty_prompt" and outs[0].tokens == []
    assert outs[1].finish_reason == "context_length" and outs[1].tokens == []
    assert outs[2].finish_reason == "length" and len(outs[2].tokens) == 2      # clamped to the room left
    llm.engine.cache.check()


def test_command_line(model_dirs, tmp_path):
    """bin/stride_cli with stride's flags: greedy tokens equal the plain implementation's; dumped logits too."""
    name = "A"
    cfg, w = plain.load_plain(model_dirs[name])
    prompts = _prompts(name, [5, 9, 13, 17], seed=1)
    inp, out, dump = tmp_path / "in.jsonl", tmp_path / "out.jsonl", tmp_path / "logits.f32"
    inp.write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "stride_cli"), "--model", str(model_dirs[name]), "--input", str(inp),
                        "--output", str(out), "--max-new", "16", "--concurrency", "3", "--prefill-chunk", "4", "--path", "exact",
                        "--kv-blocks", "12", "--max-slots", "4", "--max-rows", "32", "--full", "--dump-logits", str(dump),
                        "--dump-steps", "2", "--arrival-seed", "3"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    summary = json.loads(r.stderr.strip().splitlines()[-1])
    assert summary["generated"] == 64 and summary["weight_bytes_per_pass"] > 0
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    logits = np.fromfile(dump, dtype="<f4").reshape(len(prompts), 2, cfg.vocab_size)
    for i, (p, row) in enumerate(zip(prompts, rows)):
        assert row["id"] == i and row["finish"] == "length" and len(row["values"]) == 16
        assert row["tokens"] == plain.generate_greedy(cfg, w, p, 16)
        ref = plain.forward(cfg, w, p + row["tokens"][:1])
        assert np.abs(logits[i, 0] - ref[len(p) - 1].numpy()).max() <= 2e-4
        assert np.abs(logits[i, 1] - ref[len(p)].numpy()).max() <= 2e-4


def test_a_lost_signal_inside_a_kernel_is_an_error(model_dirs):
    """A bounded wait that gives up (here: a kernel whose only wait nothing answers, which ends by itself after about
    a second) leaves its code in the status word that the engine reads back with every step: generation raises instead
    of returning tokens, and works again afterwards."""
    from stride_b200 import LLM
    from stride_b200.engine.engine import EngineError
    from stride_b200.kernels import ops
    llm = LLM(model_dirs["A"], dtype="bfloat16", concurrency=2, max_rows=64, page_size=TINY["A"][2], kv_pages=64, max_slots=4)
    prompts = _prompts("A", [5, 9])
    good = llm.generate(prompts, max_new_tokens=4)
    ops.lost_signal_selftest(code=9)
    with pytest.raises(EngineError, match="code 9"):
        llm.generate(prompts, max_new_tokens=4)
    assert ops.gemm_tc_status() == 0          # the engine cleared the word when it raised
    llm2 = LLM(model_dirs["A"], dtype="bfloat16", concurrency=2, max_rows=64, page_size=TINY["A"][2], kv_pages=64, max_slots=4)
    again = llm2.generate(prompts, max_new_tokens=4)
    assert [o.tokens for o in again] == [o.tokens for o in good]


def test_the_engine_refuses_steps_that_disagree_with_the_cache(model_dirs):
    """Bad entries are an error before anything runs (unknown or repeated slot, tokens without pages, a token id out
    of range, a wanted place outside the entry), for prompt portions and for decoded tokens (the graph path); the
    engine works on afterwards. A batch given as arrays gives the same bits as the same batch given as entries."""
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.engine.engine import EngineError
    cfg, page = TINY["A"][0], TINY["A"][2]
    eng = Engine(model_dirs["A"], EngineOptions(dtype="bfloat16", max_rows=32, max_full_rows=8, max_slots=4, kv_pages=32, page_size=page))
    a, b = eng.cache.acquire_slot(), eng.cache.acquire_slot()
    assert eng.cache.ensure(a, 12) and eng.cache.ensure(b, 6)
    vocab = cfg["vocab_size"]
    for entries, reason in (
            ([StepEntry(a, 0, [1, 2], []), StepEntry(a, 2, [3], [0])], "appears twice"),
            ([StepEntry(3, 0, [1, 2], [])], "not held by a request"),
            ([StepEntry(b, 4, [1, 2, 3], [])], "have no pages"),
            ([StepEntry(a, 0, [1, vocab], [])], "out of range"),
            ([StepEntry(a, 0, [1, 2], [2])], "outside the entry"),
            ([StepEntry(a, 0, [1, 2], []), StepEntry(b, 0, [], [])], "without tokens"),
            ([StepEntry(a, 0, list(range(33)), [])], "exceeds max_rows"),
            ([StepEntry(a, 0, [1], [0]), StepEntry(a, 1, [2], [0])], "appears twice"),          # decoded tokens: the graph path
            ([StepEntry(b, 6, [1], [0])], "has no page")):
        with pytest.raises(EngineError, match=reason):
            eng.step(entries)
    batch = [StepEntry(a, 0, [5, 6, 7, 8, 9], [4]), StepEntry(b, 0, [11, 12, 13], [0, 2])]
    first = eng.step(batch).clone()
    i32 = lambda v: np.asarray(v, dtype=np.int32)
    again = eng.step_arrays(2, i32([a, b]), i32([0, 0]), i32([5, 3]), i32([5, 6, 7, 8, 9, 11, 12, 13]), i32([1, 2]), i32([4, 0, 2]))
    assert first.shape == (3, vocab) and torch.equal(first, again)
    one = eng.step([StepEntry(a, 5, [3], [0]), StepEntry(b, 3, [4], [0])]).clone()              # from a graph, padded to two rows
    same = eng.step_arrays(2, i32([a, b]), i32([5, 3]), i32([1, 1]), i32([3, 4]), i32([1, 1]), i32([0, 0]))
    assert torch.equal(one, same)
