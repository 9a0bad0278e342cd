"""Microbenchmarks of single kernels, timed with CUDA events after warm-up; also the small, self-contained
workloads that the ncu summaries under profiles/ were captured on.

    python -m stride_b200.kernels.microbench gemm --tokens 8 --rows 16384 --cols 2048 --epilogue swiglu
    python -m stride_b200.kernels.microbench gemm --tokens 2048 --rows 2048 --cols 8192 --epilogue add
    python -m stride_b200.kernels.microbench attention --batch 64 --context 512          # decode
    python -m stride_b200.kernels.microbench attention --batch 1 --new 2048 --context 0  # one prompt

Weights are cycled through `--copies` buffers larger than L2 in total, so every launch streams from HBM.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops

L2_BYTES = 126 << 20


def _time(fn, reps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / reps      # microseconds


def gemm(a) -> dict:
    n, M, K = a.tokens, a.rows, a.cols
    epi = {"store": ops.STORE, "add": ops.ADD, "swiglu": ops.SWIGLU}[a.epilogue]
    copies = a.copies or max(1, min(64, (2 * L2_BYTES) // (M * K * 2) + 1))
    ws = [(torch.randn(M, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(n, K, device="cuda").bfloat16()
    S = ops.gemm_tc_splits(n, M, K) if epi == ops.STORE else 1
    if epi == ops.SWIGLU:
        out = torch.zeros(n, M // 2, device="cuda", dtype=torch.bfloat16)
    else:
        out = torch.zeros((S, n, M) if S > 1 else (n, M), device="cuda")
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
    if new <= short:
        tiles, items, chunks = [], list(range(B)), (total - 1) // 256 + 1
    else:
        tiles, items, chunks = [x for e in range(B) for t in range(-(-new // ppt)) for x in (e, t)], [], 0
    work = torch.tensor(tiles + items, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(max(1, ops.attention_tc_scratch(len(items), Hkv, chunks, D)), device="cuda")
    counters = torch.zeros(max(1, len(items) * Hkv), dtype=torch.int32, device="cuda")

    def run():
        ops.attention_tc(q, out, cache, table, meta, work, len(tiles) // 2, len(items), chunks, scratch, Hq, Hkv, D, 0,
                         D ** -0.5, counters=counters)
    us = _time(run, a.reps)
    kv_bytes = B * total * Hkv * D * 2 * 2
    flops = 4.0 * B * Hq * D * (new * old + new * (new + 1) / 2)
    return {"kernel": "attention_tc", "batch": B, "context": old, "new": new, "us": round(us, 2),
            "kv_GBps": round(kv_bytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 2)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8)
    g.add_argument("--rows", type=int, default=16384)
    g.add_argument("--cols", type=int, default=2048)
    g.add_argument("--epilogue", choices=["store", "add", "swiglu"], default="store")
    g.add_argument("--copies", type=int, default=0)
    g.add_argument("--reps", type=int, default=50)
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=512)
    t.add_argument("--new", type=int, default=1)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=64)
    t.add_argument("--page", type=int, default=64)
    t.add_argument("--reps", type=int, default=50)
    a = ap.parse_args(argv)
    print(json.dumps({"gemm": gemm, "attention": attention}[a.what](a)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
