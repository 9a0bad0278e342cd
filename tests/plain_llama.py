"""Plain, slow restatement of the Llama decoder for whole sequences, no cache.

One function per part, in torch on the CPU. It shares no code with the
`stride_b200` package: the tests compare the engine's logits with what these
functions give. Every function cites the place in arhaamatiq/stride (paths
within that project) whose arithmetic it restates.

The comparison with stride's own CPU build on a tiny random model (head ratio 4,
the only ratio that build accepts) is `tests/golden/make_golden.py`; its small
outputs are committed beside it and `tests/test_plain.py` checks this file
against them.

`rounding` hooks: with `act_dtype=torch.bfloat16` the functions round at the
places where stride's tensor-core path rounds (normed activations, cached keys
and values, attention output, the SwiGLU product; `docs/ARCHITECTURE.md:24-31`)
plus the rotated query, which this engine's serving path also keeps in bfloat16.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass, field
from pathlib import Path

import torch


# --------------------------------------------------------------------------- config

@dataclass
class PlainConfig:
    """The config.json keys that stride reads (src/model.cpp:15-52)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_type: str = "default"
    rope_factor: float = 32.0
    rope_low: float = 1.0
    rope_high: float = 4.0
    rope_orig: float = 8192.0
    eos: list = field(default_factory=list)

    @staticmethod
    def from_dict(j: dict) -> "PlainConfig":
        c = PlainConfig(
            hidden_size=j["hidden_size"], intermediate_size=j["intermediate_size"],
            num_hidden_layers=j["num_hidden_layers"], num_attention_heads=j["num_attention_heads"],
            vocab_size=j["vocab_size"])
        c.num_key_value_heads = j.get("num_key_value_heads", c.num_attention_heads)
        c.head_dim = j.get("head_dim", c.hidden_size // c.num_attention_heads)
        c.rms_norm_eps = j.get("rms_norm_eps", 1e-5)
        c.rope_theta = j.get("rope_theta", 10000.0)
        r = j.get("rope_scaling")
        if r:
            t = r.get("rope_type", r.get("type", ""))
            if t == "llama3":
                c.rope_type = "llama3"
                c.rope_factor = r.get("factor", 32.0)
                c.rope_low = r.get("low_freq_factor", 1.0)
                c.rope_high = r.get("high_freq_factor", 4.0)
                c.rope_orig = r.get("original_max_position_embeddings", 8192.0)
            elif t not in ("", "default"):
                raise ValueError("unsupported rope type " + t)
        e = j.get("eos_token_id")
        if e is not None:
            c.eos = list(e) if isinstance(e, list) else [e]
        return c


# --------------------------------------------------------------------------- weights

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict:
    """u64 little-endian header length, JSON header, raw data (src/safetensors.cpp:14-49)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + b:8 + n + e]), dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def write_safetensors(path, tensors: dict) -> None:
    """The same container, written: header length, JSON header, data in name order."""
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16",
             torch.int32: "I32", torch.int64: "I64"}
    header, blobs, at = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def load_plain(model_dir):
    model_dir = Path(model_dir)
    cfg = PlainConfig.from_dict(json.loads((model_dir / "config.json").read_text()))
    return cfg, read_safetensors(model_dir / "model.safetensors")


# --------------------------------------------------------------------------- parts

def _round(x: torch.Tensor, act_dtype) -> torch.Tensor:
    if act_dtype is None or act_dtype == x.dtype:
        return x
    return x.to(act_dtype).to(x.dtype)


def embedding(tokens: torch.Tensor, table: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """h = widen(embed[token]); no scaling (src/kernels.cu:98-116)."""
    return table[tokens.long()].to(dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """r = 1/sqrt(sum(x^2)/dim + eps); y = w * (x * r) (src/kernels.cu:166-182)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return weight.to(x.dtype) * (x * r)


def rope_inverse_frequencies(cfg: PlainConfig) -> torch.Tensor:
    """inv_i in 32-bit, llama3 scaling included (src/model.cpp:54-77)."""
    dim = cfg.head_dim
    half = dim // 2
    f32 = torch.float32
    inv = torch.empty(half, dtype=f32)
    pi2 = torch.tensor(2.0 * math.pi, dtype=f32)
    for i in range(half):
        e = torch.tensor(float(2 * i), dtype=f32) / torch.tensor(float(dim), dtype=f32)
        base = torch.tensor(math.pow(cfg.rope_theta, float(e)), dtype=f32)
        f = torch.tensor(1.0, dtype=f32) / base
        if cfg.rope_type == "llama3":
            factor = torch.tensor(cfg.rope_factor, dtype=f32)
            low_wave = torch.tensor(cfg.rope_orig / cfg.rope_low, dtype=f32)
            high_wave = torch.tensor(cfg.rope_orig / cfg.rope_high, dtype=f32)
            wave = pi2 / f
            smooth = (torch.tensor(cfg.rope_orig, dtype=f32) / wave - torch.tensor(cfg.rope_low, dtype=f32)) \
                / torch.tensor(cfg.rope_high - cfg.rope_low, dtype=f32)
            if wave > low_wave:
                f = f / factor
            elif not (wave < high_wave):
                f = (torch.tensor(1.0, dtype=f32) - smooth) * (f / factor) + smooth * f
        inv[i] = f
    return inv


def rope_table(cfg: PlainConfig, positions: torch.Tensor):
    """angle = inv * float(pos) in 32-bit; cos and sin in double, then cast (src/model.cpp:78-86)."""
    inv = rope_inverse_frequencies(cfg)
    angle = inv[None, :] * positions.to(torch.float32)[:, None]
    a64 = angle.to(torch.float64)
    return torch.cos(a64).to(torch.float32), torch.sin(a64).to(torch.float32)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (d, d+D/2): a' = a cos - b sin, b' = b cos + a sin
    (src/kernels.cu:255-266). x: [T, heads, D]; cos, sin: [T, D/2]."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
              window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    A query at position p sees keys 0..p (src/kernel_common.h:123); query head h
    reads key/value head h // (Hq/Hkv) (src/kernel_common.h:128-135);
    scale = float(pow(double(D), -0.5)) multiplies the finished dot product
    (src/engine.cpp:151, src/kernel_common.h:155-158); softmax by max-subtraction
    and the sum of exponentials (src/kernel_common.h:194-203, 272-305).
    `window` > 0 keeps only the last `window` keys (not in stride; used by the
    part tests). q: [T, Hq, D]; k, v: [T, Hkv, D]; returns [T, Hq*D].
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = torch.tensor(math.pow(float(D), -0.5), dtype=torch.float32).to(q.dtype)
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    pq = positions[:, None]
    pk = positions[None, :]
    visible = pk <= pq
    if window > 0:
        visible = visible & (pk > pq - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    m = scores.max(dim=-1, keepdim=True).values
    p = torch.exp(scores - m)
    out = torch.einsum("hts,shd->thd", p, vv) / p.sum(dim=-1).transpose(0, 1)[..., None]
    return out.reshape(T, Hq * D)


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """z = silu(W1 x) * (W3 x), silu(a) = a / (1 + exp(-a)) (src/kernels.cu:359-360, src/numerics.h:33)."""
    a = x @ w_gate.to(x.dtype).T
    b = x @ w_up.to(x.dtype).T
    return (a / (1.0 + torch.exp(-a))) * b


# --------------------------------------------------------------------------- model

def forward(cfg: PlainConfig, w: dict, tokens, dtype=torch.float32, act_dtype=None,
            window: int = 0, rows=None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence, or [len(rows), vocab] at the
    positions `rows` alone (the layers run on the whole sequence either way).

    Order of a block: norm, q/k/v, rope on q and k, attention, o_proj added to the
    residual, norm, SwiGLU, down_proj added to the residual (src/engine.cpp:166-237);
    final norm and lm_head, which is embed_tokens when the file has no
    lm_head.weight (src/model.cpp:228-232).
    """
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    cos, sin = rope_table(cfg, positions)
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    h = embedding(tokens, w["model.embed_tokens.weight"], dtype)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        x = _round(rms_norm(h, w[p + "input_layernorm.weight"], cfg.rms_norm_eps), act_dtype)
        q = (x @ w[p + "self_attn.q_proj.weight"].to(dtype).T).reshape(T, Hq, D)
        k = (x @ w[p + "self_attn.k_proj.weight"].to(dtype).T).reshape(T, Hkv, D)
        v = (x @ w[p + "self_attn.v_proj.weight"].to(dtype).T).reshape(T, Hkv, D)
        q = _round(rope_apply(q, cos, sin), act_dtype)
        k = _round(rope_apply(k, cos, sin), act_dtype)
        v = _round(v, act_dtype)
        a = _round(attention(q, k, v, positions, window), act_dtype)
        h = h + a @ w[p + "self_attn.o_proj.weight"].to(dtype).T
        x = _round(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps), act_dtype)
        z = _round(swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]), act_dtype)
        h = h + z @ w[p + "mlp.down_proj.weight"].to(dtype).T
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long)]
    x = _round(rms_norm(h, w["model.norm.weight"], cfg.rms_norm_eps), act_dtype)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ head.to(dtype).T


# --------------------------------------------------------------------------- sampling

_MASK = (1 << 64) - 1


def splitmix64(x: int) -> int:
    """src/scheduler.cpp:26-31."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def choose_token(logits, temperature: float, top_p: float, top_k: int, seed: int, n_tokens: int):
    """stride's sampler in 64-bit on the host (src/scheduler.cpp:193-243).

    `n_tokens` is the length of the sequence (prompt and generated) before the
    new token is appended: the draw is keyed on (seed, n_tokens) only.
    Returns (token, logit of the token).
    """
    l = [float(v) for v in logits]
    best = 0
    for i in range(1, len(l)):
        if l[i] > l[best]:
            best = i
    if temperature <= 0.0:
        return best, l[best]
    idx = sorted(range(len(l)), key=lambda i: (-l[i], i))
    count = len(l)
    if top_k > 0:
        count = min(count, top_k)
    t32 = float(torch.tensor(temperature, dtype=torch.float32))
    top = l[idx[0]]
    probs = [math.exp((l[idx[i]] - top) / t32) for i in range(count)]
    total = 0.0
    for p in probs:
        total += p
    if top_p < 1.0:
        p32 = float(torch.tensor(top_p, dtype=torch.float32))
        cum, kept = 0.0, 0
        for i in range(count):
            cum += probs[i] / total
            kept += 1
            if cum >= p32:
                break
        count = kept
        total = 0.0
        for i in range(count):
            total += probs[i]
    r = splitmix64((seed ^ ((n_tokens * 0x9E3779B97F4A7C15) & _MASK)) & _MASK)
    u = float(r >> 11) * (1.0 / 9007199254740992.0) * total
    cum = 0.0
    for i in range(count):
        cum += probs[i]
        if u < cum:
            return idx[i], l[idx[i]]
    return idx[count - 1], l[idx[count - 1]]


def generate_greedy(cfg: PlainConfig, w: dict, prompt, max_new: int, dtype=torch.float32, act_dtype=None):
    """Whole-sequence recomputation for every new token: slow, and free of any cache."""
    tokens = list(prompt)
    out = []
    for _ in range(max_new):
        logits = forward(cfg, w, tokens, dtype, act_dtype)[-1]
        t, _ = choose_token(logits, 0.0, 1.0, 0, 0, len(tokens))
        tokens.append(t)
        out.append(t)
    return out
