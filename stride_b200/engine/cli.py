"""Command line in the manner of arhaamatiq/stride's stride_cli (tools/stride_cli.cpp:53-100,
124-251): the same flag names and meanings, the same files.

    bin/stride_cli --model DIR --input prompts.jsonl --output out.jsonl [options]

--input holds one {"id": int, "tokens": [int, ...]} a line; --output gets one
{"id", "tokens", "values" (hex of each chosen token's float32 logit), "fingerprint", "finish"}
a line, in input order. With --dump-logits FILE the float32 logits of the first
--dump-steps generated tokens of every request are written in id order (requires --full).
One JSON line with run statistics goes to standard error.

Flags of stride_cli that select variants of stride's own kernels or inject its test
mutations (--bug, --norm-tile, --micro-r, --micro-lt) have no meaning here and are not
accepted. --path exact selects the float32 engine, --path tc the bfloat16 one.
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="stride_cli", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--input", required=True, help='JSONL of {"id": int, "tokens": [int]}')
    ap.add_argument("--output", required=True, help="JSONL of results")
    ap.add_argument("--max-new", type=int, default=16, help="new tokens per request")
    ap.add_argument("--concurrency", type=int, default=1, help="most requests running at once")
    ap.add_argument("--max-rows", type=int, default=256, help="tokens per step")
    ap.add_argument("--prefill-chunk", type=int, default=64, help="most prompt tokens of one request per step")
    ap.add_argument("--max-slots", type=int, default=256, help="block-table slots")
    ap.add_argument("--kv-gb", type=float, default=1.0, help="cache pool in GiB")
    ap.add_argument("--kv-blocks", type=int, default=0, help="cache pool in pages (overrides --kv-gb)")
    ap.add_argument("--kv-shuffle", type=int, default=0, help="randomise page placement (0 = off)")
    ap.add_argument("--row-shuffle", type=int, default=0, help="randomise the order of requests in a batch (0 = off)")
    ap.add_argument("--arrival-seed", type=int, default=0, help="shuffle the submission order (0 = off)")
    ap.add_argument("--path", choices=["exact", "tc"], default="exact", help="exact: float32 engine; tc: bfloat16 engine")
    ap.add_argument("--full", action="store_true", help="request full logits at every step")
    ap.add_argument("--dump-logits", default="", help="file for raw float32 logits")
    ap.add_argument("--dump-steps", type=int, default=1, help="generated steps per request to dump")
    ap.add_argument("--use-eos", action="store_true", help="stop on config.json's eos ids")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0, help="request i samples with seed + id")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--max-context", type=int, default=0, help="longest sequence (0: config.json's max_position_embeddings)")
    ap.add_argument("--device", default="cuda:0")
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    prompts = []
    try:
        with open(a.input) as f:
            for line in f:
                if line.strip():
                    j = json.loads(line)
                    prompts.append((int(j["id"]), list(j["tokens"])))
    except OSError as e:
        print(f"cannot open {a.input}: {e.strerror}", file=sys.stderr)
        return 2

    from ..sampling.sampler import SamplingParams
    from .engine import Engine, EngineOptions
    from .scheduler import GenRequest, Scheduler, SchedulerOptions

    eo = EngineOptions(dtype="bfloat16" if a.path == "tc" else "float32", max_rows=a.max_rows, max_slots=a.max_slots,
                       max_full_rows=min(a.max_rows, max(a.concurrency, 1)), kv_bytes=int(a.kv_gb * 1024 ** 3),
                       kv_pages=a.kv_blocks, kv_shuffle_seed=a.kv_shuffle, page_size=a.page_size,
                       max_context=a.max_context, device=a.device)
    t0 = time.perf_counter()
    engine = Engine(a.model, eo)
    t1 = time.perf_counter()
    sched = Scheduler(engine, SchedulerOptions(max_seqs=a.concurrency, max_rows=a.max_rows, prefill_chunk=a.prefill_chunk,
                                               row_shuffle_seed=a.row_shuffle))
    results = {i: {"tokens": [], "values": [], "fingerprint": 0, "finish": ""} for i, _ in prompts}
    dumped = {i: [] for i, _ in prompts}
    order = list(range(len(prompts)))
    if a.arrival_seed:
        random.Random(a.arrival_seed).shuffle(order)

    def make_callback(rid):
        def on_token(ev, logits):
            r = results[rid]
            if ev.token >= 0:
                r["tokens"].append(ev.token)
                r["values"].append("%08x" % int(np.float32(ev.value).view(np.uint32)))
                r["fingerprint"] = ev.fingerprint
                if logits is not None and a.dump_logits and ev.index < a.dump_steps:
                    dumped[rid].append(np.asarray(logits, dtype="<f4").copy())
            if ev.finished:
                r["finish"] = ev.finish_reason or ""
        return on_token

    for k in order:
        rid, toks = prompts[k]
        sched.submit(GenRequest(prompt=toks, max_new_tokens=a.max_new,
                                sampling=SamplingParams(a.temperature, a.top_p, a.top_k, a.seed + rid),
                                stop_tokens=tuple(engine.spec.eos_token_ids) if a.use_eos else (),
                                full_logits=a.full, on_token=make_callback(rid)))
    t2 = time.perf_counter()
    sched.run()
    t3 = time.perf_counter()

    with open(a.output, "w") as out:
        for rid, _ in prompts:
            r = results[rid]
            out.write(json.dumps({"id": rid, "tokens": r["tokens"], "values": r["values"],
                                  "fingerprint": "%016x" % r["fingerprint"], "finish": r["finish"]}) + "\n")
    if a.dump_logits:
        with open(a.dump_logits, "wb") as f:
            for rid, _ in prompts:
                for row in dumped[rid]:
                    f.write(row.tobytes())
    import torch
    s = sched.stats
    g = engine.cache.groups
    print(json.dumps({
        "device": torch.cuda.get_device_name(engine.device), "load_seconds": t1 - t0, "run_seconds": t3 - t2,
        "steps": s.steps, "rows": s.rows, "generated": s.generated, "preemptions": s.preemptions,
        "replayed_rows": s.replayed_rows, "peak_seqs": s.peak_seqs, "peak_blocks": s.peak_blocks,
        "total_blocks": g[0].num_pages if g else 0, "block_bytes": sum(x.page_bytes for x in g),
        "weight_bytes_per_pass": engine.weight_bytes_per_step()}), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
