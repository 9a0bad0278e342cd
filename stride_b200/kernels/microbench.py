"""Microbenchmarks of single kernels, timed with CUDA events after warm-up; also the small, self-contained
workloads that the ncu summaries under profiles/ were captured on.

    python -m stride_b200.kernels.microbench gemm --tokens 8 --rows 16384 --cols 2048 --epilogue swiglu
    python -m stride_b200.kernels.microbench gemm --tokens 2048 --rows 2048 --cols 8192 --epilogue add
    python -m stride_b200.kernels.microbench attention --batch 64 --context 512          # decode
    python -m stride_b200.kernels.microbench attention --batch 1 --new 2048 --context 0  # one prompt
    python -m stride_b200.kernels.microbench step --batch 8                              # timeline of a decode step
    python -m stride_b200.kernels.microbench step --prefill 2048                         # timeline of a 2,048-token prompt
    python -m stride_b200.kernels.microbench host --tokens 256                           # the host's cost of queueing a mixed step

Weights are cycled through `--copies` buffers larger than L2 in total, so every launch streams from HBM.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops

L2_BYTES = 126 << 20


def _time(fn, reps: int, warmup: int = 3) -> float:
    """Microseconds per call of `fn`, its `reps` calls recorded in a CUDA graph and replayed, so that short kernels
    are not timed by the host's launches."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / reps      # microseconds


def gemm_f32(a) -> dict:
    """The linear layer of the 32-bit path: float32 activations, bfloat16 weights, FMA on the CUDA cores."""
    n, M, K = a.tokens, a.rows, a.cols
    copies = a.copies or max(1, min(64, (2 * L2_BYTES) // (M * K * 2) + 1))
    ws = [(torch.randn(M, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(n, K, device="cuda")
    out = torch.zeros(n, M, device="cuda")
    state = {"i": 0}

    def run():
        ops.gemm_f32(x, ws[state["i"] % copies], out, a.epilogue == "add")
        state["i"] += 1
    us = _time(run, a.reps)
    return {"kernel": "gemm_f32", "tokens": n, "rows": M, "cols": K, "epilogue": a.epilogue, "us": round(us, 2),
            "weight_GBps": round(M * K * 2 / us / 1e3, 1), "TFLOPs": round(2.0 * n * M * K / us / 1e6, 2)}


def gemm(a) -> dict:
    if a.float32:
        return gemm_f32(a)
    n, M, K = a.tokens, a.rows, a.cols
    epi = {"store": ops.STORE, "add": ops.ADD, "swiglu": ops.SWIGLU}[a.epilogue]
    copies = a.copies or max(1, min(64, (2 * L2_BYTES) // (M * K * 2) + 1))
    ws = [(torch.randn(M, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(n, K, device="cuda").bfloat16()
    S = ops.gemm_tc_splits(M, K) if epi == ops.STORE and not a.one_range else 1
    if epi == ops.SWIGLU:
        out = torch.zeros(n, M // 2, device="cuda", dtype=torch.bfloat16)
    else:
        out = torch.zeros((S, n, M) if S > 1 and n <= ops.gemm_tc_partial_tokens() else (n, M), device="cuda")
    state = {"i": 0}

    def run():
        ops.gemm_tc(x, ws[state["i"] % copies], out, epi, splits=S, half_rows=M // 2 if epi == ops.SWIGLU else 0)
        state["i"] += 1
    us = _time(run, a.reps)
    if ops.gemm_tc_status() != 0:
        raise RuntimeError("a wait inside the GEMM kernel timed out")
    return {"kernel": "gemm_tc", "tokens": n, "rows": M, "cols": K, "epilogue": a.epilogue, "splits": S, "us": round(us, 2),
            "weight_GBps": round(M * K * 2 / us / 1e3, 1), "TFLOPs": round(2.0 * n * M * K / us / 1e6, 1)}


def attention(a) -> dict:
    """`batch` requests with `context` cached tokens each bring `new` tokens."""
    Hq, Hkv, D, page = a.heads, a.kv_heads, a.head_dim, a.page
    B, old, new = a.batch, a.context, a.new
    total = old + new
    pages_per = -(-total // page)
    cache = (torch.randn(B * pages_per + 1, 2, Hkv, page, D, device="cuda") * 0.5).bfloat16()
    table = torch.arange(B * pages_per, dtype=torch.int32, device="cuda").reshape(B, pages_per)
    q = (torch.randn(B * new, Hq * D, device="cuda") * 0.5).bfloat16()
    out = torch.zeros_like(q)
    meta = torch.tensor([[i, i * new, new, old] for i in range(B)], dtype=torch.int32).T.contiguous().cuda()
    G = Hq // Hkv
    ppt, short = 64 // G, 16 // G
    tc5 = new > short and not a.mma_sync and ops.attention_tc5_supported(Hq, Hkv, D, page)
    if tc5:
        ppt = 128 // G
    if new <= short:
        tiles, items, chunks = [], list(range(B)), (total - 1) // 256 + 1
    else:
        tiles, items, chunks = [x for t in reversed(range(-(-new // ppt))) for e in range(B) for x in (e, t)], [], 0   # longest first
    work = torch.tensor(tiles + items, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(max(1, ops.attention_tc_scratch(len(items), Hkv, chunks, D)), device="cuda")
    counters = torch.zeros(max(1, len(items) * Hkv), dtype=torch.int32, device="cuda")

    def run():
        if tc5:
            ops.attention_tc5(q, out, cache, table, meta, work, len(tiles) // 2, Hq, Hkv, D, 0, D ** -0.5)
        else:
            ops.attention_tc(q, out, cache, table, meta, work, len(tiles) // 2, len(items), chunks, scratch, Hq, Hkv, D, 0,
                             D ** -0.5, counters=counters)
    us = _time(run, a.reps)
    if tc5 and ops.attention_tc5_status() != 0:
        raise RuntimeError("a wait inside the tcgen05 attention kernel timed out")
    kv_bytes = B * total * Hkv * D * 2 * 2
    flops = 4.0 * B * Hq * D * (new * old + new * (new + 1) / 2)
    return {"kernel": "attention_tc5" if tc5 else "attention_tc", "batch": B, "context": old, "new": new, "us": round(us, 2),
            "kv_GBps": round(kv_bytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 2)}


LLAMA_1B_SHAPE = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096,
}
# the layer sizes of Llama 3.2 3B and Llama 3.1 8B (head size 128)
LLAMA_SHAPES = {
    "1b": LLAMA_1B_SHAPE,
    "3b": dict(LLAMA_1B_SHAPE, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128),
    "8b": dict(LLAMA_1B_SHAPE, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128, tie_word_embeddings=False,
               max_position_embeddings=8192,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192}),
}


def step(a) -> dict:
    """Kernel timeline of one engine step (Llama 3.2 1B shape unless `shape` says otherwise, random weights) from torch.profiler: a decode step of
    `batch` requests replayed from its CUDA graph, or a prompt of `prefill` tokens. Kernels overlap under programmatic
    dependent launch, so each kernel is charged the time from its predecessor's end to its own end."""
    import collections
    import re

    from torch.profiler import ProfilerActivity, profile

    from .. import Engine, EngineOptions, StepEntry
    cfg = dict(LLAMA_SHAPES[a.shape], num_hidden_layers=a.layers)
    B, T = a.batch, a.prefill
    opts = EngineOptions(dtype="bfloat16", max_rows=max(512, B, T), max_full_rows=max(B, 1), max_slots=B + 2,
                         kv_pages=B * (a.context // 64 + 4) + T // 64 + 48, page_size=64, max_context=max(4096, a.context + 64, T),
                         decode_chain=a.chain)
    eng = Engine.from_random(cfg, 0, opts)
    gen = torch.Generator().manual_seed(1)
    slots = [eng.cache.acquire_slot() for _ in range(B)]
    for s in slots:
        eng.cache.ensure(s, a.context)
        for at in range(0, a.context, opts.max_rows):
            n = min(opts.max_rows, a.context - at)
            eng.step([StepEntry(s, at, torch.randint(0, 1000, (n,), generator=gen).tolist(), [])])

    def decode(k):
        entries = []
        for s in slots:
            eng.cache.ensure(s, a.context + k + 1)
            entries.append(StepEntry(s, a.context + k, [5], [0]))
        eng.step(entries)

    def prefill():
        s = eng.cache.acquire_slot()
        eng.cache.ensure(s, T)
        eng.step([StepEntry(s, 0, torch.randint(0, 1000, (T,), generator=gen).tolist(), [T - 1])])
        torch.cuda.synchronize()
        eng.cache.release_slot(s)

    run = prefill if T else (lambda: decode(step.k))
    step.k = 0
    for _ in range(4):
        run()
        step.k += 1
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    ks = sorted(((ev.name, ev.time_range.start, ev.time_range.end) for ev in prof.events()
                 if ev.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in ev.name and "Memset" not in ev.name),
                key=lambda k: k[1])
    first = max(i for i, k in enumerate(ks) if "embed" in k[0])
    ks = ks[first:]
    agg, prev = collections.defaultdict(lambda: [0, 0.0]), None
    for name, s, e in ks:
        short = re.sub(r"\(.*", "", name.replace("(anonymous namespace)::", "")).replace("void ", "")
        agg[short][0] += 1
        agg[short][1] += (e - prev) if prev is not None else (e - s)
        prev = max(prev or 0, e)
    return {"step": "prefill" if T else "decode", "batch": B, "context": a.context, "prefill": T, "layers": a.layers,
            "wall_us": round(ks[-1][2] - ks[0][1], 1), "kernels": len(ks),
            "by_kernel": {k: {"launches": c, "critical_us": round(v, 1)} for k, (c, v) in sorted(agg.items(), key=lambda x: -x[1][1])}}


def chain(a) -> dict:
    """Where the time of the decode chain goes (Llama 3.2 1B shape): the kernel's own nanosecond stamps per phase and
    CTA, summarised per phase of a layer as medians over the layers: the phase's share of the critical path (from the
    last arrival of the phase in front to its own last arrival), and for the CTAs that had a share in it the median
    time until their input was there, of their work, and of the arrival itself."""
    import ctypes
    import statistics

    from .. import Engine, EngineOptions, StepEntry
    from .build import library
    cfg = dict(LLAMA_1B_SHAPE, num_hidden_layers=a.layers)
    B = a.batch
    opts = EngineOptions(dtype="bfloat16", max_rows=max(512, B), max_full_rows=max(B, 1), max_slots=B + 2,
                         kv_pages=B * (a.context // 64 + 4) + 48, page_size=64, max_context=4096, cuda_graphs=False, decode_chain=True)
    eng = Engine.from_random(cfg, 0, opts)
    gen = torch.Generator().manual_seed(1)
    slots = [eng.cache.acquire_slot() for _ in range(B)]
    for s in slots:
        eng.cache.ensure(s, a.context)
        for at in range(0, a.context, opts.max_rows):
            n = min(opts.max_rows, a.context - at)
            eng.step([StepEntry(s, at, torch.randint(0, 1000, (n,), generator=gen).tolist(), [])])
    the_chain = eng._program.chains[0]
    phases, sms = len(the_chain), torch.cuda.get_device_properties(0).multi_processor_count
    stamps = torch.zeros(2, phases, sms, 4, dtype=torch.int64, device="cuda")
    lib = library("decode_chain")
    lib.sb_chain_trace.argtypes, lib.sb_chain_trace.restype = [ctypes.c_void_p, ctypes.c_void_p], None
    for k in range(5):
        if k == 4:
            lib.sb_chain_trace(the_chain.handle, stamps.data_ptr())
        entries = []
        for s in slots:
            eng.cache.ensure(s, a.context + k + 1)
            entries.append(StepEntry(s, a.context + k, [5], [0]))
        eng.step(entries)
    torch.cuda.synchronize()
    lib.sb_chain_trace(the_chain.handle, None)
    both = stamps.cpu().numpy().astype("float64")
    t, mma = both[0], both[1]
    t0 = t[0, :, 0].min()
    end = t[:, :, 3].max(axis=1)                      # a phase's last arrival
    per_layer = phases // a.layers
    rows = []
    for k in range(per_layer):
        crit, wait, work, arrive, busy, first, w_wait, x_wait, issued = [], [], [], [], [], [], [], [], []
        for L in range(1 if a.layers > 1 else 0, a.layers):
            ph = L * per_layer + k
            crit.append(end[ph] - end[ph - 1] if ph else end[0] - t0)
            had = t[ph, :, 1] > 0
            busy.append(int(had.sum()))
            if had.any():
                wait.append(float(statistics.median((t[ph, had, 1] - end[ph - 1]) if ph else (t[ph, had, 1] - t0))))
                work.append(float(statistics.median(t[ph, had, 2] - t[ph, had, 1])))
                arrive.append(float(statistics.median(t[ph, had, 3] - t[ph, had, 2])))
            did = mma[ph, :, 0] > 0
            if did.any() and ph:
                first.append(float(statistics.median(mma[ph, did, 0] - end[ph - 1])))
                w_wait.append(float(statistics.median(mma[ph, did, 1])))
                x_wait.append(float(statistics.median(mma[ph, did, 2])))
                issued.append(float(statistics.median(mma[ph, did, 3] - end[ph - 1])))
        med = lambda v: round(statistics.median(v) / 1000, 2) if v else None
        rows.append({"phase": k, "critical_us": med(crit), "ctas": statistics.median(busy), "input_after_us": med(wait), "work_us": med(work),
                     "arrive_us": med(arrive), "mma_first_operands_after_us": med(first), "mma_waited_for_weights_us": med(w_wait),
                     "mma_waited_for_tokens_us": med(x_wait), "mma_issued_after_us": med(issued)})
    return {"batch": B, "context": a.context, "layers": a.layers, "kernel_us": round((end[-1] - t0) / 1000, 1), "phases_of_a_layer": rows}


def host(a) -> dict:
    """What the host spends to queue one step (Llama 3.2 1B shape): `decoders` requests that decode one token each beside
    a prompt portion of `tokens - decoders` tokens, with the native step program and with the Python driver: the host's
    time to queue the step onto an idle GPU, and the time per step when the steps run back to back (the larger of the
    host's and the GPU's share)."""
    import time

    from .. import Engine, EngineOptions, StepEntry
    cfg = dict(LLAMA_1B_SHAPE, num_hidden_layers=a.layers)
    out = {"tokens": a.tokens, "decoders": a.decoders, "layers": a.layers}
    for native in (True, False):
        eng = Engine.from_random(cfg, 0, EngineOptions(dtype="bfloat16", max_rows=max(512, a.tokens), max_full_rows=a.decoders + 1,
                                                       max_slots=a.decoders + 2, kv_pages=(a.decoders + 1) * 64, page_size=64,
                                                       max_context=4096, native_step=native))
        cm = eng.cache
        slots = [cm.acquire_slot() for _ in range(a.decoders + 1)]
        for s in slots[:-1]:
            cm.ensure(s, 100)
            eng.step([StepEntry(s, 0, list(range(100)), [])])
        portion = a.tokens - a.decoders

        def one(k):
            entries = []
            for s in slots[:-1]:
                cm.ensure(s, 101 + k)
                entries.append(StepEntry(s, 100 + k, [7], [0]))
            cm.ensure(slots[-1], portion)
            entries.append(StepEntry(slots[-1], 0, list(range(portion)), [portion - 1]))     # the same portion again and again
            eng.step(entries)

        for k in range(3):
            one(k)
        # the host's share: each step queued onto an idle GPU (a full launch queue would make the host wait for the GPU)
        spent = 0.0
        for k in range(3, 3 + a.reps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            one(k)
            spent += time.perf_counter() - t0
        # the GPU's share: the same steps back to back
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(3 + a.reps, 3 + 2 * a.reps):
            one(k)
        stop.record()
        torch.cuda.synchronize()
        key = "native" if native else "python"
        out[key + "_host_us_per_step"] = round(spent * 1e6 / a.reps, 1)
        out[key + "_back_to_back_us_per_step"] = round(start.elapsed_time(stop) * 1e3 / a.reps, 1)
        del eng
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8)
    g.add_argument("--rows", type=int, default=16384)
    g.add_argument("--cols", type=int, default=2048)
    g.add_argument("--epilogue", choices=["store", "add", "swiglu"], default="store")
    g.add_argument("--copies", type=int, default=0)
    g.add_argument("--one-range", action="store_true", help="keep K in one range whatever the weight's shape")
    g.add_argument("--reps", type=int, default=50)
    g.add_argument("--float32", action="store_true", help="the 32-bit path's linear layer (FMA, no tensor cores)")
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=512)
    t.add_argument("--new", type=int, default=1)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--page", type=int, default=64)
    t.add_argument("--reps", type=int, default=50)
    t.add_argument("--mma-sync", action="store_true", help="prompt portions on the mma.sync kernel instead of tcgen05")
    st = sub.add_parser("step")
    st.add_argument("--batch", type=int, default=8)
    st.add_argument("--context", type=int, default=256)
    st.add_argument("--prefill", type=int, default=0, help="time one prompt of this many tokens instead of a decode step")
    st.add_argument("--layers", type=int, default=16)
    st.add_argument("--shape", choices=sorted(LLAMA_SHAPES), default="1b", help="layer sizes: Llama 3.2 1B, 3.2 3B or 3.1 8B")
    st.add_argument("--chain", action="store_true", help="decode steps with all layers as one persistent kernel (the decode chain)")
    h = sub.add_parser("host")
    ch = sub.add_parser("chain", help="the decode chain's own per-phase time stamps")
    ch.add_argument("--batch", type=int, default=8)
    ch.add_argument("--context", type=int, default=256)
    ch.add_argument("--layers", type=int, default=16)
    h.add_argument("--tokens", type=int, default=256)
    h.add_argument("--decoders", type=int, default=8)
    h.add_argument("--layers", type=int, default=16)
    h.add_argument("--reps", type=int, default=30)
    a = ap.parse_args(argv)
    print(json.dumps({"gemm": gemm, "attention": attention, "step": step, "host": host, "chain": chain}[a.what](a), indent=1 if a.what in ("step", "chain") else None))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
