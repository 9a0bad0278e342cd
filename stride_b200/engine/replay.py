"""Trace replay: feed given token ids through the engine step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch for `Engine.step`; `want` lists the places among an
entry's tokens whose logits are written, as little-endian float32 [wanted, vocab], to
`<out>/<step>.f32` (no file when nothing is wanted). `end` names requests that are
finished after the step: their slot and pages go back to the pool. After each step
`done <step>` is printed and flushed. Nothing is sampled; the model, the step function,
the cache manager and the kernels are the ones that generation uses.

`--max-tokens` sizes the page pool: the most tokens live requests hold at any time, each
request's count rounded up to whole pages (64 tokens, or `--page-size`).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page (default 64)")
    ap.add_argument("--max-requests", type=int, default=16, help="most requests alive at once")
    ap.add_argument("--kv-shuffle", type=int, default=0, help="hand out pages in a random order (seed; 0 = off)")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    print("[trace_run] starting (the first call compiles the CUDA kernels this model needs)", file=sys.stderr, flush=True)
    import torch
    from .engine import Engine, EngineOptions, StepEntry

    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    ps = a.page_size
    pages = max(1, (a.max_tokens + ps - 1) // ps)
    capacity = pages * ps
    opts = EngineOptions(dtype=a.dtype, max_rows=capacity, max_full_rows=capacity, max_slots=a.max_requests,
                         kv_pages=pages, page_size=ps, max_context=capacity, kv_shuffle_seed=a.kv_shuffle,
                         device=a.device)
    engine = Engine(a.model, opts)
    print(f"[trace_run] model loaded: {engine.architecture.name}, {a.dtype}, {pages} pages of {ps} tokens",
          file=sys.stderr, flush=True)

    live: dict = {}     # request id -> [slot, tokens fed so far]
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid, tokens = e["id"], list(e["tokens"])
            if not tokens:
                continue
            if rid not in live:
                slot = engine.cache.acquire_slot()
                if slot < 0:
                    raise SystemExit(f"trace_run: step {step}: more than {a.max_requests} requests are alive")
                live[rid] = [slot, 0]
            slot, fed = live[rid]
            if not engine.cache.ensure(slot, fed + len(tokens)):
                raise SystemExit(f"trace_run: step {step}: request {rid!r} needs more pages than --max-tokens {a.max_tokens} gives")
            entries.append(StepEntry(slot=slot, first_pos=fed, tokens=tokens, want=list(e.get("want", []))))
            live[rid][1] = fed + len(tokens)
        logits = engine.step(entries) if entries else None
        if logits is not None:
            host = logits.detach().to("cpu", torch.float32)
            engine.check_kernels()        # the copy waited for the step: a wait that gave up inside a kernel is an error
            host.numpy().astype("<f4", copy=False).tofile(out / f"{step}.f32")
        else:
            torch.cuda.synchronize()
        for slot, _ in (live[r] for r in live):
            engine.cache.trim(slot)
        for rid in rec.get("end", []):
            if rid in live:
                engine.cache.release_slot(live.pop(rid)[0])
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
