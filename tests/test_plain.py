"""The plain implementation itself: against arhaamatiq/stride's own CPU build (golden file), its
parts against each other, its sampler, and that the bfloat16 yardstick of the GPU tests notices
a single dropped key."""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import pytest
import torch

import plain_llama as plain
from conftest import TINY, TEST_GAIN_STD, TEST_STD, bf16_noise, logit_tolerance, random_tokens

GOLDEN = Path(__file__).parent / "golden" / "ref_cpu_ratio4.json"


def test_plain_matches_the_reference_cpu_build():
    """Logits of stride's exact path on the golden model (tests/golden/make_golden.py) within 2e-4,
    the tolerance of its own suite; every greedy token equal."""
    import sys
    sys.path.insert(0, str(GOLDEN.parent))
    import make_golden as mg
    g = json.loads(GOLDEN.read_text())
    cfg = plain.PlainConfig.from_dict(g["config"])
    w = mg.golden_model(g["seed"])
    V = cfg.vocab_size
    raw = b"".join(struct.pack("<I", int(h, 16)) for h in g["logits_hex"])
    ref = torch.tensor(struct.unpack(f"<{len(raw) // 4}f", raw)).reshape(len(g["prompts"]), g["dump_steps"], V)
    for i, (p, t) in enumerate(zip(g["prompts"], g["tokens"])):
        logits = plain.forward(cfg, w, (p + t)[:-1])
        for s in range(g["dump_steps"]):
            assert (logits[len(p) - 1 + s] - ref[i, s]).abs().max() <= 2e-4
        assert [int(logits[len(p) - 1 + s].argmax()) for s in range(len(t))] == t


def test_rope_table_values():
    cfg = plain.PlainConfig.from_dict(TINY["B"][0])
    inv = plain.rope_inverse_frequencies(cfg)
    assert inv.shape == (16,) and float(inv[0]) == 1.0
    # the longest waves are slowed by the factor, the shortest are untouched
    plain_inv = torch.tensor([1.0 / math.pow(cfg.rope_theta, 2 * i / 32) for i in range(16)])
    assert abs(float(inv[-1]) / float(plain_inv[-1]) - 1 / 32) < 1e-6
    cos, sin = plain.rope_table(cfg, torch.arange(5))
    assert torch.allclose(cos[0], torch.ones(16)) and torch.allclose(sin[0], torch.zeros(16))
    x = torch.randn(5, 3, 32)
    y = plain.rope_apply(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)      # a rotation keeps lengths


def test_attention_is_causal_and_grouped():
    T, Hq, Hkv, D = 9, 6, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(T, Hq, D, generator=g), torch.randn(T, Hkv, D, generator=g), torch.randn(T, Hkv, D, generator=g)
    out = plain.attention(q, k, v, torch.arange(T)).reshape(T, Hq, D)
    assert torch.allclose(out[0], v[0].repeat_interleave(3, dim=0))          # position 0 sees only itself
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0                                                     # later keys do not matter for position 4
    out2 = plain.attention(q, k2, v2, torch.arange(T)).reshape(T, Hq, D)
    assert torch.allclose(out[:5], out2[:5])
    w = plain.attention(q, k, v, torch.arange(T), window=3).reshape(T, Hq, D)
    ref = plain.attention(q[6:7], k[4:7], v[4:7], torch.tensor([2]) * 0 + 2)  # keys 4, 5, 6 only
    assert torch.allclose(w[6], plain.attention(torch.cat([q[4:6] * 0, q[6:7]]), k[4:7], v[4:7], torch.arange(3)).reshape(3, Hq, D)[2], atol=1e-6)


def test_sampler_rules():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0, 0.5])
    assert plain.choose_token(logits, 0.0, 1.0, 0, 0, 3) == (1, 2.0)       # first maximum
    assert plain.choose_token(logits, 0.8, 1.0, 1, 123, 3)[0] == 1         # top_k 1 is greedy
    draws = {plain.choose_token(logits, 1.0, 1.0, 0, s, 7)[0] for s in range(200)}
    assert draws == {0, 1, 2, 3, 4}
    draws = {plain.choose_token(logits, 1.0, 0.5, 0, s, 7)[0] for s in range(200)}
    assert draws == {1, 2}                                                  # top_p 0.5 keeps the two best
    a = plain.choose_token(logits, 1.0, 1.0, 0, 5, 7)
    assert a == plain.choose_token(logits, 1.0, 1.0, 0, 5, 7)
    assert plain.splitmix64(0) == 0xE220A8397B1DCDAF


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_bfloat16_yardstick_notices_a_shifted_window_edge(name, tmp_path):
    """The tolerance the GPU tests use for bfloat16 (half of bfloat16's own rounding noise) is smaller
    than what eight keys missing at the far edge do to the last positions' logits. (A single far key
    can carry a weight of exactly zero in these models; the kernel tests and the model with near-uniform
    attention make single keys count.)"""
    from stride_b200.weights.random_init import write_random_model
    cfg_dict, seed, _ = TINY[name]
    model = write_random_model(tmp_path / name, cfg_dict, seed, std=TEST_STD, gain_std=TEST_GAIN_STD)
    cfg, w = plain.load_plain(model)
    T = 100
    toks = random_tokens(cfg.vocab_size, T, 100)
    good = plain.forward(cfg, w, toks, torch.float32, torch.bfloat16)
    tol = logit_tolerance("bfloat16", good, bf16_noise(cfg, w, toks))
    dropped = plain.forward(cfg, w, toks, torch.float32, torch.bfloat16, window=T - 8)   # the last 8 tokens miss old keys
    assert (dropped[:-8] - good[:-8]).abs().max() == 0
    assert (dropped[-1] - good[-1]).abs().max() > tol
