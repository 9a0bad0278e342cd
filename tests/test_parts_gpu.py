"""Each part of a layer alone, built from a PartSpec and stepped on the GPU, against the plain function
of the same name, in float32 and bfloat16, at sizes of their own."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama as plain
from stride_b200.cache.manager import CacheManager
from stride_b200.parts import BuildEnv, PartSpec, ResidualStream, StepContext, Workspace, part_class

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _env(dtype, max_tokens=64, max_positions=128):
    return BuildEnv(device=DEV, compute_dtype=dtype, max_tokens=max_tokens, max_positions=max_positions, max_requests=4)


def _ctx(env, ws, entries):
    """entries: [(slot, first_pos, n tokens)] -> StepContext with the device tables an engine step makes."""
    rows = sum(n for _, _, n in entries)
    pos = torch.tensor([p0 + i for _, p0, n in entries for i in range(n)], dtype=torch.int32, device=DEV)
    slots = torch.tensor([s for s, _, n in entries for _ in range(n)], dtype=torch.int32, device=DEV)
    meta = torch.zeros(4, len(entries), dtype=torch.int32)
    at = 0
    for i, (s, p0, n) in enumerate(entries):
        meta[:, i] = torch.tensor([s, at, n, p0])
        at += n
    return StepContext(n=rows, token_ids=torch.zeros(rows, dtype=torch.int32, device=DEV), positions=pos, slots=slots,
                       workspace=ws, compute_dtype=env.compute_dtype, entry_slots=[e[0] for e in entries],
                       entry_first_row=[int(x) for x in meta[1]], entry_length=[e[2] for e in entries],
                       entry_first_pos=[e[1] for e in entries], entry_meta=meta.to(DEV),
                       upload_ints=lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV))


def _rand(*shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _tol(dtype, ref):
    return (2e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    env = _env(dtype)
    norm = part_class("norm", "rmsnorm")(PartSpec("rmsnorm", {"size": 200, "eps": 3e-4}, {"weight": "w"}), env)
    assert list(norm.tensor_plan()) == ["w"] and norm.tensor_plan()["w"].shape == (200,)
    w = _rand(200, seed=1)
    norm.bind({"w": w.to(DEV)})
    h = _rand(9, 200, seed=2, dtype=torch.float32)
    out = torch.zeros(9, 200, dtype=dtype, device=DEV)
    norm.forward(None, ResidualStream(h.to(DEV).clone()), out)
    ref = plain.rms_norm(h, w, 3e-4)
    assert (out.float().cpu() - ref).abs().max() <= _tol(dtype, ref)


def test_rotary_table_matches_plain():
    for cfg_dict in ({"hidden_size": 8, "intermediate_size": 8, "num_hidden_layers": 1, "num_attention_heads": 1, "vocab_size": 8,
                      "head_dim": 48, "rope_theta": 2500.0,
                      "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                       "original_max_position_embeddings": 32}},
                     {"hidden_size": 8, "intermediate_size": 8, "num_hidden_layers": 1, "num_attention_heads": 1, "vocab_size": 8,
                      "head_dim": 16, "rope_theta": 1e6}):
        cfg = plain.PlainConfig.from_dict(cfg_dict)
        scaling = {"rope_type": cfg.rope_type, "factor": cfg.rope_factor, "low_freq_factor": cfg.rope_low,
                   "high_freq_factor": cfg.rope_high, "original_max_position_embeddings": cfg.rope_orig}
        rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling}),
                                              _env(torch.float32, max_positions=300))
        cos, sin = plain.rope_table(cfg, torch.arange(300))
        assert torch.equal(rope.cos_sin[..., 0].cpu(), cos) and torch.equal(rope.cos_sin[..., 1].cpu(), sin)


@pytest.mark.parametrize("dtype,D,Hq,Hkv,window", [(torch.float32, 24, 6, 2, 0), (torch.bfloat16, 64, 8, 2, 0),
                                                   (torch.float32, 16, 4, 4, 9), (torch.bfloat16, 128, 4, 1, 40)])
def test_attention_mixer_alone(dtype, D, Hq, Hkv, window):
    """q/k/v projection, rotation, append, attention and output projection of one mixer, over two steps
    (a portion, then more tokens beside a second request), against the plain functions."""
    H, page = 80, 8
    env = _env(dtype)
    pos_spec = PartSpec("rope", {"head_dim": D, "rotary_dim": D, "theta": 10000.0, "scaling": {}})
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "window": window,
                                  "position": pos_spec}, {"q": "q", "k": "k", "v": "v", "o": "o"})
    mixer = part_class("mixer", "attention")(spec, env)
    plan = mixer.tensor_plan()
    assert plan["q"].shape == (Hq * D, H) and plan["o"].shape == (H, Hq * D)
    w = {"q": _rand(Hq * D, H, seed=1, scale=0.15), "k": _rand(Hkv * D, H, seed=2, scale=0.15),
         "v": _rand(Hkv * D, H, seed=3, scale=0.15), "o": _rand(H, Hq * D, seed=4, scale=0.1)}
    mixer.bind({k: v.to(DEV) for k, v in w.items()})
    need = mixer.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window, need.dtype) == ("pages", Hkv, D, window, dtype)
    cm = CacheManager([need], device=DEV, max_slots=4, max_context=128, page_size=page, num_pages=24, shuffle_seed=3)
    ws = Workspace(DEV, 64)
    seqs = {0: _rand(50, H, seed=5, dtype=torch.float32), 1: _rand(21, H, seed=6, dtype=torch.float32)}
    slots = {0: cm.acquire_slot(), 1: cm.acquire_slot()}
    got = {0: [], 1: []}
    fed = {0: 0, 1: 0}
    for step in ([(0, 37)], [(0, 1), (1, 21)], [(0, 12)]):
        entries, xs = [], []
        for r, n in step:
            cm.ensure(slots[r], fed[r] + n)
            entries.append((slots[r], fed[r], n))
            xs.append(seqs[r][fed[r]:fed[r] + n])
        cm.sync()
        ctx = _ctx(env, ws, entries)
        x = torch.cat(xs).to(dtype).to(DEV)
        stream = ResidualStream(torch.zeros(ctx.n, H, device=DEV))
        mixer.forward(ctx, x, stream, cm.layer_cache(0))
        stream.fold()
        at = 0
        for r, n in step:
            got[r].append(stream.h[at:at + n].cpu())
            at += n
            fed[r] += n
            cm.trim(slots[r])
    cfg = plain.PlainConfig(hidden_size=H, intermediate_size=8, num_hidden_layers=1, num_attention_heads=Hq, vocab_size=8,
                            num_key_value_heads=Hkv, head_dim=D, rope_theta=10000.0)
    act = torch.bfloat16 if dtype == torch.bfloat16 else None
    for r in (0, 1):
        x = plain._round(seqs[r], act)
        T = x.shape[0]
        cos, sin = plain.rope_table(cfg, torch.arange(T))
        q = plain._round(plain.rope_apply((x @ w["q"].float().T).reshape(T, Hq, D), cos, sin), act)
        k = plain._round(plain.rope_apply((x @ w["k"].float().T).reshape(T, Hkv, D), cos, sin), act)
        v = plain._round((x @ w["v"].float().T).reshape(T, Hkv, D), act)
        ref = plain._round(plain.attention(q, k, v, torch.arange(T), window), act) @ w["o"].float().T
        out = torch.cat(got[r])
        assert (out - ref).abs().max() <= _tol(dtype, ref) * (1 if dtype == torch.float32 else 2), f"request {r}"
    cm.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_embedding_head_and_block(dtype):
    H, I, V = 72, 200, 333
    env = _env(dtype)
    act = torch.bfloat16 if dtype == torch.bfloat16 else None
    ff = part_class("feed_forward", "swiglu")(PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I},
                                                       {"gate": "g", "up": "u", "down": "d"}), env)
    w = {"g": _rand(I, H, seed=1, scale=0.15), "u": _rand(I, H, seed=2, scale=0.15), "d": _rand(H, I, seed=3, scale=0.1)}
    ff.bind({k: v.to(DEV) for k, v in w.items()})
    ws = Workspace(DEV, 64)
    ctx = _ctx(env, ws, [(0, 0, 11)])
    x = plain._round(_rand(11, H, seed=4, dtype=torch.float32), act)
    base = _rand(11, H, seed=5, dtype=torch.float32)
    stream = ResidualStream(base.to(DEV).clone())
    ff.forward(ctx, x.to(dtype).to(DEV), stream)
    stream.fold()
    ref = base + plain._round(plain.swiglu(x, w["g"], w["u"]), act) @ w["d"].float().T
    assert (stream.h.cpu() - ref).abs().max() <= _tol(dtype, ref)

    emb = part_class("embedding", "lookup")(PartSpec("lookup", {"vocab_size": V, "hidden_size": H}, {"weight": "e"}), env)
    table = _rand(V, H, seed=6)
    emb.bind({"e": table.to(DEV)})
    ctx.token_ids = torch.tensor([0, 5, 332, 7, 7, 1, 2, 3, 4, 100, 200], dtype=torch.int32, device=DEV)
    out = torch.zeros(11, H, device=DEV)
    emb.forward(ctx, out)
    assert torch.equal(out.cpu(), plain.embedding(ctx.token_ids.cpu(), table))

    for tied, tensors in ((True, {"e": table}), (None, {"e": table}), (None, {"e": table, "lm": _rand(V, H, seed=7)}),
                          (False, {"lm": _rand(V, H, seed=7)})):
        head = part_class("head", "linear")(PartSpec("linear", {"vocab_size": V, "hidden_size": H, "tied": tied},
                                                     {"weight": "lm", "tied_to": "e"}), env)
        head.bind({k: v.to(DEV) for k, v in tensors.items()})
        logits = torch.zeros(11, V, device=DEV)
        head.forward(x.to(dtype).to(DEV), logits)
        ref = x @ tensors.get("lm", table).float().T
        assert head.is_tied == ("lm" not in tensors)
        assert (logits.cpu() - ref).abs().max() <= _tol(dtype, ref)
