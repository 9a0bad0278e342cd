"""A toy architecture defined here, without touching the framework's files: a mixer with state of its own
(an exponential moving average of its inputs per request), registered as a part, mixed with attention
layers in one model; a schedule that runs one layer twice, the second time reading the first call's
cache; and a windowed attention layer whose pages are given back as the window passes. The model is built
by the registry, stepped through the engine in portions and single tokens beside other requests, and
compared with a plain whole-sequence computation written out below. A second toy architecture further down has a
feed-forward with routing and another position encoding (a rotation of half of every head by other angles)."""
from __future__ import annotations

import pytest
import torch

import plain_llama as plain
from conftest import random_tokens
from stride_b200 import Engine, EngineOptions, StepEntry
from stride_b200.config import Architecture, register_architecture
from stride_b200.parts import (CacheNeed, LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry, TensorPlan, register_part)

pytestmark = pytest.mark.gpu

H, V, D, HQ, HKV, I, WINDOW, DECAY = 48, 101, 16, 3, 1, 64, 11, 0.75


@register_part("mixer", "toy_ema")
class EmaMixer(Mixer):
    """state_t = decay * state_{t-1} + (1 - decay) * x_t per request; output = W state_t. Written with torch
    operations and host loops (it is a test double, not a kernel), so it is not graph-safe."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size, self.decay = spec.params["hidden_size"], spec.params["decay"]

    def tensor_plan(self):
        return {self.spec.tensors["w"]: TensorPlan((self.size, self.size))}

    def bind(self, tensors):
        self.w = tensors[self.spec.tensors["w"]].float()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.size,), state_dtype=torch.float32)

    def forward(self, ctx, x, stream, cache):
        out = torch.zeros(ctx.n, self.size, device=x.device)
        for slot, row, length in zip(ctx.entry_slots, ctx.entry_first_row, ctx.entry_length):
            state = cache.state[slot].clone()
            for t in range(length):
                state = self.decay * state + (1.0 - self.decay) * x[row + t].float()
                out[row + t] = self.w @ state
            cache.state[slot] = state
        stream.add_(out)


def _spec(cfg: dict) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": D, "theta": 10000.0, "scaling": {}})
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": name})
    ff = lambda i: PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I},
                            {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})
    layers = []
    for i, kind in enumerate(cfg["mixers"]):
        if kind == "ema":
            mixer = PartSpec("toy_ema", {"hidden_size": H, "decay": DECAY}, {"w": f"l{i}.ema"})
        else:
            mixer = PartSpec("attention", {"hidden_size": H, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D,
                                           "window": WINDOW if kind == "window" else 0, "position": rope},
                             {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
        layers.append(LayerSpec(mixer, ff(i), norm(f"l{i}.n1"), norm(f"l{i}.n2")))
    schedule = tuple(ScheduleEntry(l, c) for l, c in cfg["schedule"])
    return ModelSpec(vocab_size=V, hidden_size=H, embedding=PartSpec("lookup", {"vocab_size": V, "hidden_size": H}, {"weight": "emb"}),
                     layers=tuple(layers), schedule=schedule, final_norm=norm("final"),
                     head=PartSpec("linear", {"vocab_size": V, "hidden_size": H, "tied": True}, {"weight": "head", "tied_to": "emb"}),
                     max_positions=256)


register_architecture(Architecture("ToyEmaForCausalLM", lambda d: d, _spec))

CONFIG = {"architectures": ["ToyEmaForCausalLM"], "mixers": ["ema", "full", "window", "ema"],
          # layer 1 (attention over all keys) runs twice; its second call reads the first call's cache
          "schedule": [[0, None], [1, None], [2, None], [1, 1], [3, None]]}


def _weights():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.2).to(torch.bfloat16)
    gain = lambda: (1 + 0.2 * torch.randn(H, generator=g)).to(torch.bfloat16)
    w = {"emb": r(V, H), "final": gain()}
    for i, kind in enumerate(CONFIG["mixers"]):
        w.update({f"l{i}.n1": gain(), f"l{i}.n2": gain(), f"l{i}.gate": r(I, H), f"l{i}.up": r(I, H), f"l{i}.down": r(H, I)})
        if kind == "ema":
            w[f"l{i}.ema"] = r(H, H)
        else:
            w.update({f"l{i}.q": r(HQ * D, H), f"l{i}.k": r(HKV * D, H), f"l{i}.v": r(HKV * D, H), f"l{i}.o": r(H, HQ * D)})
    return w


def _plain_forward(w, tokens):
    T = len(tokens)
    pos = torch.arange(T)
    cfg = plain.PlainConfig(hidden_size=H, intermediate_size=I, num_hidden_layers=1, num_attention_heads=HQ, vocab_size=V,
                            num_key_value_heads=HKV, head_dim=D)
    cos, sin = plain.rope_table(cfg, pos)
    h = plain.embedding(torch.tensor(tokens), w["emb"])
    kv_of = {}
    for e, (l, cache_of) in enumerate(CONFIG["schedule"]):
        kind = CONFIG["mixers"][l]
        x = plain.rms_norm(h, w[f"l{l}.n1"], 1e-5)
        if kind == "ema":
            state, ys = torch.zeros(H), []
            for t in range(T):
                state = DECAY * state + (1 - DECAY) * x[t]
                ys.append(w[f"l{l}.ema"].float() @ state)
            h = h + torch.stack(ys)
        else:
            q = plain.rope_apply((x @ w[f"l{l}.q"].float().T).reshape(T, HQ, D), cos, sin)
            if cache_of is None:
                k = plain.rope_apply((x @ w[f"l{l}.k"].float().T).reshape(T, HKV, D), cos, sin)
                v = (x @ w[f"l{l}.v"].float().T).reshape(T, HKV, D)
                kv_of[e] = (k, v)
            else:
                k, v = kv_of[cache_of]
            h = h + plain.attention(q, k, v, pos, WINDOW if kind == "window" else 0) @ w[f"l{l}.o"].float().T
        x = plain.rms_norm(h, w[f"l{l}.n2"], 1e-5)
        h = h + plain.swiglu(x, w[f"l{l}.gate"], w[f"l{l}.up"]) @ w[f"l{l}.down"].float().T
    return plain.rms_norm(h, w["final"], 1e-5) @ w["emb"].float().T


def test_toy_architecture_is_registered_built_and_stepped():
    w = _weights()
    eng = Engine(None, EngineOptions(dtype="float32", max_rows=64, max_full_rows=64, max_slots=4, kv_pages=60, page_size=4,
                                     max_context=256), config=CONFIG, tensors=w)
    assert eng.architecture.name == "ToyEmaForCausalLM" and not eng.model.graph_safe
    cm = eng.cache
    # attention over all keys (entries 1 and 3 share a cache) and the windowed layer get groups of their own; the two
    # state mixers get one record per request each
    assert len(cm.groups) == 2 and sorted(g.window for g in cm.groups) == [0, WINDOW]
    assert set(cm.states) == {0, 4} and cm.entry_shared == {3: 1}
    reqs = [random_tokens(V, n, 7 + n) for n in (90, 33, 61)]
    want = [_plain_forward(w, r) for r in reqs]
    slots = [cm.acquire_slot() for _ in reqs]
    fed = [0, 0, 0]
    sizes = [[13, 1, 1, 7, 2], [5, 1, 1, 1], [30, 1, 3]]
    step = 0
    while any(f < len(r) for f, r in zip(fed, reqs)):
        entries, spans = [], []
        for i, r in enumerate(reqs):
            if fed[i] >= len(r) or (step + i) % 4 == 3:
                continue
            n = min(sizes[i][step % len(sizes[i])], len(r) - fed[i])
            assert cm.ensure(slots[i], fed[i] + n)
            entries.append(StepEntry(slots[i], fed[i], r[fed[i]:fed[i] + n], list(range(n))))
            spans.append((i, fed[i], fed[i] + n))
            fed[i] += n
        if entries:
            logits = eng.step(entries).cpu()
            at = 0
            for i, a, b in spans:
                ref = want[i][a:b]
                assert (logits[at:at + b - a] - ref).abs().max() <= 2e-4 * max(1.0, float(ref.pow(2).mean().sqrt())), (step, i, a, b)
                at += b - a
            for i, _, _ in spans:
                cm.trim(slots[i])
        step += 1
    # the windowed group gave pages back as the window passed: far fewer than the 90 tokens' 23 pages are held
    win = next(g for g in cm.groups if g.window)
    assert len(win.held[slots[0]]) <= WINDOW // 4 + 2 < 23
    for s in slots:
        cm.release_slot(s)
    cm.check()
    assert cm.free_pages() == cm.total_pages()


# ----------------------------------------------------------------------------------------------------------------
# A second toy architecture: a feed-forward with routing (a router in 32-bit picks two of four small experts per
# token) and another position encoding (angles that grow with the square root of the position, on the first half of
# every head only), again registered from here and built by the framework's registry.
from stride_b200.parts import FeedForward, PositionEncoding   # noqa: E402

E, TOPK, IE, ROT = 4, 2, 24, 8


@register_part("feed_forward", "toy_routed")
class RoutedFeedForward(FeedForward):
    """logits = R x in 32-bit; the TOPK largest (lower index on ties) get weights softmax(their logits); the token's
    output is the weighted sum of those experts' gated MLPs. Torch operations: a test double, not a kernel."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.experts, self.top_k = spec.params["hidden_size"], spec.params["experts"], spec.params["top_k"]

    def tensor_plan(self):
        t, p = self.spec.tensors, self.spec.params
        return {t["router"]: TensorPlan((self.experts, self.hidden)),
                t["gate"]: TensorPlan((self.experts, p["intermediate_size"], self.hidden)),
                t["up"]: TensorPlan((self.experts, p["intermediate_size"], self.hidden)),
                t["down"]: TensorPlan((self.experts, self.hidden, p["intermediate_size"]))}

    def bind(self, tensors):
        t = self.spec.tensors
        self.router, self.gate, self.up, self.down = (tensors[t[k]].float() for k in ("router", "gate", "up", "down"))

    def forward(self, ctx, x, stream):
        xf = x.float()
        logits = xf @ self.router.T                                    # [n, E] float32
        order = torch.argsort(-logits, dim=1, stable=True)[:, :self.top_k]
        weights = torch.softmax(torch.gather(logits, 1, order), dim=1)
        out = torch.zeros_like(xf)
        for e in range(self.experts):
            for k in range(self.top_k):
                rows = (order[:, k] == e).nonzero().flatten()
                if rows.numel():
                    a, b = xf[rows] @ self.gate[e].T, xf[rows] @ self.up[e].T
                    out[rows] += weights[rows, k, None] * (((a / (1 + torch.exp(-a))) * b) @ self.down[e].T)
        stream.add_(out)


@register_part("position", "toy_sqrt")
class SqrtRotation(PositionEncoding):
    """Rotation of the first `rotary_dim` elements of a head by angle_i(pos) = sqrt(pos) * base^-i: the table that
    the framework's rotation kernel reads ([positions, rotary_dim / 2, (cos, sin)] float32) and `rotary_dim`."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rotary_dim = spec.params["rotary_dim"]
        self.cos_sin = _sqrt_table(env.max_positions, self.rotary_dim, spec.params["base"]).to(env.device)


def _sqrt_table(positions, rotary_dim, base):
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    angle = torch.arange(positions, dtype=torch.float64).sqrt()[:, None] * base ** -i[None, :]
    return torch.stack([angle.cos(), angle.sin()], dim=-1).float()


def _routed_spec(cfg: dict) -> ModelSpec:
    pos = PartSpec("toy_sqrt", {"rotary_dim": ROT, "base": 3.0})
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-6}, {"weight": name})
    layers = []
    for i in range(cfg["layers"]):
        mixer = PartSpec("attention", {"hidden_size": H, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D, "window": 0, "position": pos},
                         {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
        ff = PartSpec("toy_routed", {"hidden_size": H, "intermediate_size": IE, "experts": E, "top_k": TOPK},
                      {"router": f"l{i}.router", "gate": f"l{i}.egate", "up": f"l{i}.eup", "down": f"l{i}.edown"})
        layers.append(LayerSpec(mixer, ff, norm(f"l{i}.n1"), norm(f"l{i}.n2")))
    return ModelSpec(vocab_size=V, hidden_size=H, embedding=PartSpec("lookup", {"vocab_size": V, "hidden_size": H}, {"weight": "emb"}),
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(i, None) for i in range(cfg["layers"])), final_norm=norm("final"),
                     head=PartSpec("linear", {"vocab_size": V, "hidden_size": H, "tied": True}, {"weight": "head", "tied_to": "emb"}),
                     max_positions=128)


register_architecture(Architecture("ToyRoutedForCausalLM", lambda d: d, _routed_spec))


def _routed_weights(layers):
    g = torch.Generator().manual_seed(1)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.25).to(torch.bfloat16)
    gain = lambda: (1 + 0.2 * torch.randn(H, generator=g)).to(torch.bfloat16)
    w = {"emb": r(V, H), "final": gain()}
    for i in range(layers):
        w.update({f"l{i}.n1": gain(), f"l{i}.n2": gain(), f"l{i}.q": r(HQ * D, H), f"l{i}.k": r(HKV * D, H), f"l{i}.v": r(HKV * D, H),
                  f"l{i}.o": r(H, HQ * D), f"l{i}.router": r(E, H) * 4, f"l{i}.egate": r(E, IE, H), f"l{i}.eup": r(E, IE, H),
                  f"l{i}.edown": r(E, H, IE)})
    return w


def _routed_plain(w, tokens, layers):
    T = len(tokens)
    pos = torch.arange(T)
    table = _sqrt_table(T, ROT, 3.0)
    cos, sin = table[..., 0], table[..., 1]

    def rotate(x):      # [T, heads, D]: the first ROT elements, element j paired with j + ROT / 2
        a, b, rest = x[..., :ROT // 2], x[..., ROT // 2:ROT], x[..., ROT:]
        c, s = cos[:, None, :], sin[:, None, :]
        return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)

    h = plain.embedding(torch.tensor(tokens), w["emb"])
    for l in range(layers):
        x = plain.rms_norm(h, w[f"l{l}.n1"], 1e-6)
        q = rotate((x @ w[f"l{l}.q"].float().T).reshape(T, HQ, D))
        k = rotate((x @ w[f"l{l}.k"].float().T).reshape(T, HKV, D))
        v = (x @ w[f"l{l}.v"].float().T).reshape(T, HKV, D)
        h = h + plain.attention(q, k, v, pos, 0) @ w[f"l{l}.o"].float().T
        x = plain.rms_norm(h, w[f"l{l}.n2"], 1e-6)
        logits = x @ w[f"l{l}.router"].float().T
        y = torch.zeros_like(x)
        for t in range(T):
            chosen = sorted(range(E), key=lambda e: (-float(logits[t, e]), e))[:TOPK]
            wts = torch.softmax(logits[t, chosen], dim=0)
            for wt, e in zip(wts, chosen):
                a, b = w[f"l{l}.egate"][e].float() @ x[t], w[f"l{l}.eup"][e].float() @ x[t]
                y[t] += wt * (w[f"l{l}.edown"][e].float() @ ((a / (1 + torch.exp(-a))) * b))
        h = h + y
    return plain.rms_norm(h, w["final"], 1e-6) @ w["emb"].float().T


def test_toy_routed_feed_forward_and_position_encoding():
    layers = 2
    config = {"architectures": ["ToyRoutedForCausalLM"], "layers": layers}
    w = _routed_weights(layers)
    eng = Engine(None, EngineOptions(dtype="float32", max_rows=64, max_full_rows=64, max_slots=4, kv_pages=40, page_size=8,
                                     max_context=128), config=config, tensors=w)
    assert eng.architecture.name == "ToyRoutedForCausalLM"
    cm = eng.cache
    reqs = [random_tokens(V, n, 3 + n) for n in (70, 41)]
    want = [_routed_plain(w, r, layers) for r in reqs]
    slots = [cm.acquire_slot() for _ in reqs]
    fed = [0, 0]
    sizes = [[9, 1, 1, 20, 2], [5, 1, 1, 13]]
    step = 0
    while any(f < len(r) for f, r in zip(fed, reqs)):
        entries, spans = [], []
        for i, r in enumerate(reqs):
            if fed[i] >= len(r):
                continue
            n = min(sizes[i][step % len(sizes[i])], len(r) - fed[i])
            assert cm.ensure(slots[i], fed[i] + n)
            entries.append(StepEntry(slots[i], fed[i], r[fed[i]:fed[i] + n], list(range(n))))
            spans.append((i, fed[i], fed[i] + n))
            fed[i] += n
        logits = eng.step(entries).cpu()
        at = 0
        for i, a, b in spans:
            ref = want[i][a:b]
            assert (logits[at:at + b - a] - ref).abs().max() <= 2e-4 * max(1.0, float(ref.pow(2).mean().sqrt())), (step, i, a, b)
            at += b - a
        step += 1
    for s in slots:
        cm.release_slot(s)
    cm.check()


# ----------------------------------------------------------------------------------------------------------------
# A third toy architecture: a block of its own kind (ONE norm whose output feeds the mixer and the feed-forward side by
# side: h += mixer(norm(h)) + ff(norm(h))) and a feed-forward that brings its own CUDA source, registered as a kernel
# library from here, with a native operation, so that the whole toy model runs as one native step program. Nothing in
# the framework's files knows of either.
import ctypes   # noqa: E402

from stride_b200.kernels import ops as _ops   # noqa: E402
from stride_b200.kernels.build import library, register_kernel_library   # noqa: E402
from stride_b200.parts import Block   # noqa: E402

TOY_KERNEL = r'''
#include "common.cuh"
#include "step_ops.h"
SB_DEFINE_LAST_ERROR()
namespace {
// h[t, j] += a[j] * tanhf(b[j] * x[t, j]): a per-token transform with two learned vectors
__global__ void vecgate_kernel(const float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ h, int n, int H) {
  sb::grid_launch_dependents();
  sb::grid_dependency_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n * H) h[i] += a[i % H] * tanhf(b[i % H] * x[i]);
}
}  // namespace
SB_EXPORT int toy_vecgate(const float* x, const float* a, const float* b, float* h, int n, int H, cudaStream_t stream) {
  if (n <= 0) return 0;
  sb::launch_pdl(vecgate_kernel, dim3((n * H + 255) / 256), dim3(256), 0, stream, x, a, b, h, n, H);
  return sb::check_launch("toy_vecgate");
}
// the same as an operation of the native step program. i: 0 x, 1 a, 2 b, 3 h, 4 H
SB_EXPORT int toy_op_vecgate(const SbOp* op, const SbStep* s, void* stream) {
  using namespace sbstep;
  return toy_vecgate(ptr<const float>(op->i[0]), ptr<const float>(op->i[1]), ptr<const float>(op->i[2]), ptr<float>(op->i[3]), s->n,
                     (int)op->i[4], static_cast<cudaStream_t>(stream));
}
'''


@pytest.fixture(scope="module")
def toy_library(tmp_path_factory):
    src = tmp_path_factory.mktemp("toy_kernels") / "toy_vecgate.cu"
    src.write_text(TOY_KERNEL)
    register_kernel_library("toy_vecgate", src)
    return "toy_vecgate"


@register_part("feed_forward", "toy_vecgate")
class VecGate(FeedForward):
    """h += a * tanh(b * x), by a kernel of the test's own library. float32 activations only."""
    graph_safe = True

    def tensor_plan(self):
        size = self.spec.params["hidden_size"]
        return {self.spec.tensors["a"]: TensorPlan((size,)), self.spec.tensors["b"]: TensorPlan((size,))}

    def bind(self, tensors):
        self.a, self.b = (tensors[self.spec.tensors[k]].float().contiguous() for k in ("a", "b"))

    def kernel_libraries(self):
        return {"toy_vecgate"}

    def forward(self, ctx, x, stream):
        stream.fold()
        fn = library("toy_vecgate").toy_vecgate
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        assert fn(x.data_ptr(), self.a.data_ptr(), self.b.data_ptr(), stream.h.data_ptr(), ctx.n, x.shape[1], _ops._stream()) == 0

    def emit(self, program, x):
        program.need_folded("the vector gate")
        program.add("toy_vecgate", "toy_op_vecgate", [x, self.a, self.b, program.h, x.shape[1]])


@register_part("block", "toy_parallel")
class ParallelBlock(Block):
    """One norm; the mixer and the feed-forward both read its output and both add to the residual."""
    ROLES = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    graph_safe = True

    def forward(self, ctx, stream, cache):
        x = ctx.workspace.get("toy_parallel.x", ctx.n, (stream.h.shape[1],), ctx.act_dtype)
        self.norm.forward(ctx, stream, x)
        self.mixer.forward(ctx, x, stream, cache)
        self.feed_forward.forward(ctx, x, stream)

    def emit(self, program, cache):
        ws = program.workspace
        x = ws.get("toy_parallel.x", ws.max_tokens, (program.h.shape[1],), self.env.act_dtype)
        self.norm.emit(program, x)
        self.mixer.emit(program, x, cache)
        self.feed_forward.emit(program, x)


def _parallel_spec(cfg: dict) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": D, "theta": 10000.0, "scaling": {}})
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": name})
    layers = []
    for i in range(cfg["layers"]):
        mixer = PartSpec("attention", {"hidden_size": H, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D, "window": 0, "position": rope},
                         {"q": f"l{i}.q", "k": f"l{i}.k", "v": f"l{i}.v", "o": f"l{i}.o"})
        ff = PartSpec("toy_vecgate", {"hidden_size": H}, {"a": f"l{i}.a", "b": f"l{i}.b"})
        layers.append(LayerSpec("toy_parallel", {"norm": norm(f"l{i}.n"), "mixer": mixer, "feed_forward": ff}))
    return ModelSpec(vocab_size=V, hidden_size=H, embedding=PartSpec("lookup", {"vocab_size": V, "hidden_size": H}, {"weight": "emb"}),
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(i, None) for i in range(cfg["layers"])), final_norm=norm("final"),
                     head=PartSpec("linear", {"vocab_size": V, "hidden_size": H, "tied": True}, {"weight": "head", "tied_to": "emb"}),
                     max_positions=128)


register_architecture(Architecture("ToyParallelForCausalLM", lambda d: d, _parallel_spec))


def _parallel_plain(w, tokens, layers):
    T = len(tokens)
    pos = torch.arange(T)
    cfg = plain.PlainConfig(hidden_size=H, intermediate_size=I, num_hidden_layers=1, num_attention_heads=HQ, vocab_size=V,
                            num_key_value_heads=HKV, head_dim=D)
    cos, sin = plain.rope_table(cfg, pos)
    h = plain.embedding(torch.tensor(tokens), w["emb"])
    for l in range(layers):
        x = plain.rms_norm(h, w[f"l{l}.n"], 1e-5)
        q = plain.rope_apply((x @ w[f"l{l}.q"].float().T).reshape(T, HQ, D), cos, sin)
        k = plain.rope_apply((x @ w[f"l{l}.k"].float().T).reshape(T, HKV, D), cos, sin)
        v = (x @ w[f"l{l}.v"].float().T).reshape(T, HKV, D)
        h = h + plain.attention(q, k, v, pos, 0) @ w[f"l{l}.o"].float().T + w[f"l{l}.a"].float() * torch.tanh(w[f"l{l}.b"].float() * x)
    return plain.rms_norm(h, w["final"], 1e-5) @ w["emb"].float().T


def test_a_block_of_its_own_kind_with_a_part_that_brings_its_kernel(toy_library):
    layers = 3
    config = {"architectures": ["ToyParallelForCausalLM"], "layers": layers}
    g = torch.Generator().manual_seed(2)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.25).to(torch.bfloat16)
    gain = lambda: (1 + 0.2 * torch.randn(H, generator=g)).to(torch.bfloat16)
    w = {"emb": r(V, H), "final": gain()}
    for i in range(layers):
        w.update({f"l{i}.n": gain(), f"l{i}.q": r(HQ * D, H), f"l{i}.k": r(HKV * D, H), f"l{i}.v": r(HKV * D, H), f"l{i}.o": r(H, HQ * D),
                  f"l{i}.a": r(H) * 4, f"l{i}.b": r(H) * 4})
    reqs = [random_tokens(V, n, 11 + n) for n in (50, 23)]
    want = [_parallel_plain(w, q, layers) for q in reqs]
    results = {}
    for native in (True, False):
        eng = Engine(None, EngineOptions(dtype="float32", max_rows=64, max_full_rows=64, max_slots=4, kv_pages=40, page_size=8,
                                         max_context=128, native_step=native), config=config, tensors=w)
        # every part of this model has a native form, the test's own among them: the step is one native program
        assert (eng._program is not None) == native
        cm = eng.cache
        slots = [cm.acquire_slot() for _ in reqs]
        fed, step, got = [0, 0], 0, []
        sizes = [[7, 1, 1, 16, 2], [3, 1, 1, 9]]
        while any(f < len(q) for f, q in zip(fed, reqs)):
            entries, spans = [], []
            for i, q in enumerate(reqs):
                if fed[i] >= len(q):
                    continue
                n = min(sizes[i][step % len(sizes[i])], len(q) - fed[i])
                assert cm.ensure(slots[i], fed[i] + n)
                entries.append(StepEntry(slots[i], fed[i], q[fed[i]:fed[i] + n], list(range(n))))
                spans.append((i, fed[i], fed[i] + n))
                fed[i] += n
            logits = eng.step(entries).cpu()
            got.append(logits.clone())
            at = 0
            for i, a, b in spans:
                ref = want[i][a:b]
                assert (logits[at:at + b - a] - ref).abs().max() <= 2e-4 * max(1.0, float(ref.pow(2).mean().sqrt())), (native, step, i, a, b)
                at += b - a
            step += 1
        results[native] = got
    assert all(torch.equal(a, b) for a, b in zip(results[True], results[False]))


def test_a_position_part_of_another_nature_is_refused_with_a_reason():
    @register_part("position", "toy_bias_only")
    class BiasOnly(PositionEncoding):
        """No rotation tables: an encoding that the attention mixer's kernels cannot apply."""

    mixer = PartSpec("attention", {"hidden_size": H, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D, "window": 0,
                                   "position": PartSpec("toy_bias_only", {})}, {"q": "q", "k": "k", "v": "v", "o": "o"})
    from stride_b200.parts import BuildEnv
    from stride_b200.parts.base import part_class
    env = BuildEnv(device=torch.device("cuda"), compute_dtype=torch.float32, max_tokens=8, max_positions=16)
    part = part_class("mixer", "attention")(mixer, env)
    z = lambda *s: torch.zeros(*s, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="cos_sin"):
        part.bind({"q": z(HQ * D, H), "k": z(HKV * D, H), "v": z(HKV * D, H), "o": z(H, HQ * D)})
