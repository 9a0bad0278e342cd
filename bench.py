"""Benchmark of the serving step: decode tokens per second of a Llama 3.2 1B shaped model
with random weights on one B200, with prefill, roofline fractions and an end-to-end figure.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of `--batch` requests (256-token prompts, decoding from position
256 on). W warm-up steps, then exactly K steps timed with CUDA events on the launching stream,
synchronised on both sides. Weights (2.47 GB) are far larger than L2 (126 MB), so every step
streams them from HBM again; no explicit flush is needed. One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096,
}
CONTEXT = 4096
PROMPT = 256
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            j = json.loads(p.read_text())
            return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prefill_flops(cfg: dict, T: int, layers: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2.0 * T * layers * (H * (Hq + 2 * Hkv) * D + Hq * D * H + 3 * H * I)
    attention = layers * 2.0 * 2.0 * Hq * D * (T * (T + 1) / 2.0)
    return linear + attention + 2.0 * H * V


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "arhaamatiq/stride is a CMake C++/CUDA project built for sm_89 with no Python package; "
                          "pip cannot install it offline (no setup.py or pyproject.toml)"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from stride_b200 import Engine, EngineOptions, StepEntry
    from stride_b200.engine.scheduler import GenRequest, Scheduler, SchedulerOptions
    from stride_b200.kernels import ops

    cfg = dict(LLAMA_1B)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    max_batch = max(a.batch, 1 if a.skip_points else 64)
    page = 64
    pages = max_batch * (CONTEXT // page) // 4 + PREFILL_TOKENS // page + 8
    opts = EngineOptions(dtype="bfloat16", max_rows=max(PREFILL_TOKENS, max_batch), max_full_rows=max_batch, max_slots=max_batch + 1,
                         kv_pages=pages, page_size=page, max_context=CONTEXT)
    engine = Engine.from_random(cfg, seed=0, options=opts)
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    kv_token_bytes = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    weight_bytes = engine.weight_bytes_per_step()

    def decode_run(batch: int, steps: int, warmup: int):
        """Prefill `batch` prompts of PROMPT tokens, then time `steps` decode steps. Returns (ms/step, launches/step)."""
        cache = engine.cache
        slots = [cache.acquire_slot() for _ in range(batch)]
        prompts = torch.randint(0, vocab, (batch, PROMPT), generator=gen).tolist()
        per_step = max(1, opts.max_rows // PROMPT)
        for i in range(0, batch, per_step):
            entries = []
            for s, p in zip(slots[i:i + per_step], prompts[i:i + per_step]):
                cache.ensure(s, PROMPT)
                entries.append(StepEntry(s, 0, p, []))
            engine.step(entries)
        tokens = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
        out_tok = torch.zeros(batch, dtype=torch.int32, device=engine.device)
        out_val = torch.zeros(batch, dtype=torch.float32, device=engine.device)

        def one(k):
            pos = PROMPT + k
            entries = []
            for b, s in enumerate(slots):
                cache.ensure(s, pos + 1)
                entries.append(StepEntry(s, pos, [tokens[k][b]], [0]))
            logits = engine.step(entries)
            ops.argmax(logits, out_tok, out_val)

        for k in range(warmup):
            one(k)
        torch.cuda.synchronize()
        l0 = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(warmup, warmup + steps):
            one(k)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches = (ops.launches - l0) // steps
        for s in slots:
            cache.release_slot(s)
        return ms, launches

    def e2e_run(batch: int, steps: int, warmup: int):
        """The same through the scheduler: host token ids in, sampled ids back to the host every step."""
        sched = Scheduler(engine, SchedulerOptions(max_seqs=batch, max_rows=opts.max_rows, prefill_chunk=PROMPT))
        prompts = torch.randint(0, vocab, (batch, PROMPT), generator=gen).tolist()
        for p in prompts:
            sched.submit(GenRequest(prompt=p, max_new_tokens=warmup + steps + 4))
        while sched.stats.generated < batch * warmup:
            sched.run(steps=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        g0 = sched.stats.generated
        sched.run(steps=steps)          # every step: pinned H2D of its inputs, D2H of its sampled tokens
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        made = sched.stats.generated - g0
        sched.run()
        return made / dt

    def prefill_run(reps: int = 3):
        cache = engine.cache
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        best = None
        for r in range(reps + 1):
            slot = cache.acquire_slot()
            cache.ensure(slot, PREFILL_TOKENS)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry(slot, 0, toks, [PREFILL_TOKENS - 1])])
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop)
            if r > 0:
                best = ms if best is None else min(best, ms)
            cache.release_slot(slot)
        return best

    clocks = ClockSampler()
    clocks.start()
    ms, launches = decode_run(a.batch, a.steps, a.warmup)
    clock_info = clocks.stop()
    value = a.batch * 1000.0 / ms
    mean_ctx = PROMPT + a.warmup + (a.steps + 1) / 2.0
    step_bytes = weight_bytes + a.batch * mean_ctx * kv_token_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e = e2e_run(a.batch, a.steps, a.warmup)
    points, prefill = {}, None
    if not a.skip_points:
        for b in (1, 64):
            pm, _ = decode_run(b, max(16, a.steps // 2), a.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pm, 1)
        pms = prefill_run()
        fl = prefill_flops(cfg, PREFILL_TOKENS, layers)
        prefill = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                   "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    h2d = engine.last_h2d_bytes if hasattr(engine, "last_h2d_bytes") else engine._ints * 4
    # stride's own published engine numbers for this workload (256-token prompts, 256 outputs; one RTX 4090, the only
    # hardware it publishes for; prefill time included there): batch 1, 8, 64 (its README.md:40-42)
    published = {1: 306.0, 8: 2276.0, 64: 10061.0}
    vs_baseline = round(value / published[a.batch], 3) if a.batch in published and layers == full_layers else None
    line = {
        "metric": f"decode tok/s at batch {a.batch} (Llama 3.2 1B shape, 256-token prompts)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": vs_baseline, "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)",
        "config": {"model": "llama-3.2-1b-shape", "layers": layers, "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "global_batch": a.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT, "page_size": page, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2: 2.47 GB of weights streamed every step", "peaks": pk["source"]},
        "clocks": clock_info,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": a.batch * 8 * 2},
        "gpu_launches": launches * a.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    if prefill:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
