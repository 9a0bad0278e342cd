"""Benchmark of the serving step: decode tokens per second of a Llama shaped model with random
weights on one B200, with prefill, roofline fractions and an end-to-end figure.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference] [--shape 1b|3b|8b]

Default (`--shape 1b`): a "step" is one decode step of `--batch` requests (256-token prompts, decoding
from position 256 on). W warm-up steps, then regions of exactly K steps each, timed with CUDA events on
the launching stream and synchronised on both sides; `ms_per_step` is the median region. The weights
(2.47 GB) are far larger than L2 (126 MB), so every step streams them from HBM again; no flush is needed.
`e2e` is the whole workload of the reference's own offline benchmark (256-token prompts, 256 outputs,
prefill included) through the Python entry point, host token ids in and out: generated tokens / wall time.

`--impl reference` builds the unmodified arhaamatiq/stride sources kept under baseline/_ref with nvcc and
drives its stock `stride_cli --path tc` on the same model shape and prompts (as its scripts/bench/offline.py
does). `--shape 3b` / `--shape 8b` measure the two larger shapes through the scheduler.
One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import shutil
import statistics
import struct
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _llama(hidden, inter, layers, heads, kv_heads, head_dim, tied, factor, max_pos):
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": hidden, "intermediate_size": inter,
            "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
            "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192},
            "tie_word_embeddings": tied, "rms_norm_eps": 1e-5, "max_position_embeddings": max_pos}


SHAPES = {
    "1b": ("llama-3.2-1b-shape", _llama(2048, 8192, 16, 32, 8, 64, True, 32.0, 4096)),
    "3b": ("llama-3.2-3b-shape", _llama(3072, 8192, 28, 24, 8, 128, True, 32.0, 4096)),
    "8b": ("llama-3.1-8b-shape", _llama(4096, 14336, 32, 32, 8, 128, False, 8.0, 8192)),
}
PROMPT = 256
OUTPUTS = 256
PREFILL_TOKENS = 2048
LONG_CONTEXT = 32768     # cached tokens of the one request of the long-context decode point
REGIONS = 5            # timed regions of K steps each; the median is reported
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


def offline_prompts(count: int, length: int, seed: int = 21) -> list:
    """Token-id prompts made the way arhaamatiq/stride's offline benchmark makes them
    (scripts/bench/offline.py:19-21): the BOS id, then uniform ids, from a seeded generator."""
    rng = random.Random(seed)
    return [[128000] + [rng.randint(1000, 100000) for _ in range(length - 1)] for _ in range(count)]


def describe(name: str, cfg: dict, layers: int, batch: int, page: int, pk: dict) -> dict:
    """The flat `config` record (the same for both arms: it describes the workload, not the program)."""
    return {"model": name, "layers": layers, "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
            "seq_len": cfg["max_position_embeddings"], "prompt_len": PROMPT, "outputs": OUTPUTS, "page_size": page,
            "parallelism": "single-gpu", "l2": "inputs larger than L2: the weights are streamed every step",
            "peaks": pk["source"]}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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


# ---------------------------------------------------------------------------------------------------- the reference arm
REF_DIR = ROOT / "baseline" / "_ref"
REF_SOURCES = ["src/safetensors.cpp", "src/model.cpp", "src/kv_cache.cpp", "src/engine.cpp", "src/scheduler.cpp",
               "src/kernels.cu", "src/device.cu", "src/kernels_tc.cu", "tools/stride_cli.cpp"]


def _json_include() -> str | None:
    """A folder that holds nlohmann/json.hpp (the reference fetches it with CMake; this image carries a copy)."""
    cands = [REF_DIR / "third_party"]
    for p in sys.path:
        cands.append(Path(p) / "include" / "cudnn_frontend" / "thirdparty")
    for c in cands:
        if (c / "nlohmann" / "json.hpp").exists():
            return str(c)
    return None


def build_reference() -> tuple:
    """(path of the reference's stride_cli, how it was built) or (None, why not). The sources are the
    reference's own files, unmodified, copied to baseline/_ref; the flags are those of its CMakeLists.txt:36-44
    with the architecture of this GPU in place of sm_89."""
    cli = REF_DIR / "build" / "stride_cli"
    how = "nvcc -O3 -fmad=false -Xcompiler=-fno-strict-aliasing -DSTRIDE_BACKEND_CUDA, arch sm_100 (CMakeLists.txt:36-44 has 89)"
    if cli.exists():
        return cli, how + "; prebuilt"
    # the unmodified copy under baseline/_ref, else a checkout named by STRIDE_REFERENCE or lying beside this repository
    src = REF_DIR if (REF_DIR / "src").exists() else Path(os.environ.get("STRIDE_REFERENCE", ROOT.parent / "reference"))
    if not (src / "src" / "engine.cpp").exists():
        return None, "the reference's sources are neither under baseline/_ref nor in a checkout beside this repository (STRIDE_REFERENCE)"
    inc = _json_include()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if inc is None or not Path(nvcc).exists():
        return None, "nvcc or nlohmann/json.hpp not found, so the reference cannot be compiled"
    cli.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-fmad=false", "-Xcompiler=-fno-strict-aliasing,-fno-fast-math,-ffp-contract=off,-O3",
           "-gencode", "arch=compute_100,code=[sm_100,compute_100]", "-DSTRIDE_BACKEND_CUDA", f"-I{src / 'src'}", f"-I{inc}",
           *[str(src / s) for s in REF_SOURCES], "-o", str(cli)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0 or not cli.exists():
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-3:]
        return None, "nvcc failed on the reference: " + " | ".join(tail)
    return cli, how


def write_reference_model(folder: Path, cfg: dict, seed: int = 0) -> None:
    """config.json + model.safetensors (bfloat16, N(0, 0.02), norm gains 1 + N(0, 0.1)) for the reference's loader,
    written with torch on the CPU alone: nothing of this repository's engine is imported in the reference arm."""
    import torch
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", True):
        shapes["lm_head.weight"] = (V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (Hq * D, H), p + "self_attn.k_proj.weight": (Hkv * D, H),
                       p + "self_attn.v_proj.weight": (Hkv * D, H), p + "self_attn.o_proj.weight": (H, Hq * D),
                       p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
                       p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,)})
    header, at = {}, 0
    for name in sorted(shapes):
        n = 2
        for s in shapes[name]:
            n *= s
        header[name] = {"dtype": "BF16", "shape": list(shapes[name]), "data_offsets": [at, at + n]}
        at += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    gen = torch.Generator().manual_seed(seed)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in sorted(shapes):
            shape = shapes[name]
            if len(shape) == 1:
                t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
            else:
                t = 0.02 * torch.randn(shape, generator=gen)
            f.write(t.to(torch.bfloat16).view(torch.uint8).numpy().tobytes())


def reference_arm(a) -> int:
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if a.gpus != 1:
        print(f"bench.py: arhaamatiq/stride runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.shape != "1b":
        return unavailable("arhaamatiq/stride takes only a head ratio of 4 and at most 2,048 tokens of context "
                           "(src/model.cpp:49, src/kernels.h:18): the 3B and 8B workloads do not fit it")
    cli, how = build_reference()
    if cli is None:
        return unavailable(how)
    name, cfg = SHAPES["1b"]
    cfg = dict(cfg)
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    pk = peaks()
    tmp = Path(tempfile.mkdtemp(prefix="stride_ref_"))
    try:
        t0 = time.time()
        write_reference_model(tmp / "model", cfg)
        wrote_s = time.time() - t0
        prompts = offline_prompts(64, PROMPT)

        def run(batch: int, max_new: int, path: str = "tc") -> dict:
            """One run of the stock command line, as scripts/bench/offline.py:70-78 calls it."""
            source = tmp / f"p{batch}.jsonl"
            if not source.exists():
                source.write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts[:batch])))
            cmd = [str(cli), "--path", path, "--model", str(tmp / "model"), "--input", str(source), "--output", str(tmp / "o.jsonl"),
                   "--max-new", str(max_new), "--kv-gb", "16", "--concurrency", str(batch), "--max-rows", "2048",
                   "--prefill-chunk", "256", "--max-slots", "256"]
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
            if proc.returncode != 0:
                raise RuntimeError(f"stride_cli exited with {proc.returncode}: " + " | ".join(proc.stderr.strip().splitlines()[-3:]))
            return json.loads(proc.stderr.strip().splitlines()[-1])

        def measure(batch: int, repeats: int, path: str = "tc") -> dict:
            """Generated tokens / run_seconds of the whole run (prefill included), first run discarded; and the
            decode steps alone: the time of the run with 256 outputs less the time of the run with one."""
            whole, first = [], []
            for r in range(repeats + 1):
                d = run(batch, OUTPUTS, path)
                if r > 0:
                    whole.append(d)
            for r in range(repeats):
                first.append(run(batch, 1, path))
            t_whole = statistics.median(d["run_seconds"] for d in whole)
            t_first = statistics.median(d["run_seconds"] for d in first)
            generated = whole[0]["generated"]
            decode_s = max(t_whole - t_first, 1e-9)
            return {"e2e": generated / t_whole, "decode": batch * (OUTPUTS - 1) / decode_s, "ms_per_step": decode_s * 1e3 / (OUTPUTS - 1),
                    "run_seconds": [round(d["run_seconds"], 4) for d in whole], "first_token_seconds": round(t_first, 4),
                    "load_seconds": round(whole[0]["load_seconds"], 2), "steps": whole[0]["steps"], "device": whole[0]["device"]}

        clocks = ClockSampler()
        clocks.start()
        try:
            main = measure(a.batch, 3)
        except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
            clocks.stop()
            return unavailable(f"the reference's stride_cli did not run here: {e}")
        clock_info = clocks.stop()
        points = {}
        if not a.skip_points:
            for b in (1, 64):
                try:
                    m = measure(b, 2)
                    points[f"decode_b{b}"] = round(m["decode"], 1)
                    points[f"e2e_b{b}"] = round(m["e2e"], 1)
                except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
                    points[f"decode_b{b}"] = None
                    points[f"error_b{b}"] = str(e)[:200]
            try:        # its exact (float32) path, the counterpart of this engine's float32 point
                points["decode_b1_float32"] = round(measure(1, 1, "exact")["decode"], 1)
            except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
                points["decode_b1_float32"] = None
                points["error_float32"] = str(e)[:200]
        weight_bytes = 2 * (cfg["num_hidden_layers"] * (cfg["hidden_size"] * (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
                                                      + cfg["num_attention_heads"] * cfg["head_dim"] * cfg["hidden_size"]
                                                      + 3 * cfg["hidden_size"] * cfg["intermediate_size"]) + cfg["vocab_size"] * cfg["hidden_size"])
        kv_token_bytes = cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
        step_bytes = weight_bytes + a.batch * (PROMPT + OUTPUTS / 2.0) * kv_token_bytes
        achieved = step_bytes / (main["ms_per_step"] * 1e-3) / 1e9
        print(json.dumps({
            "impl": "reference",
            "metric": f"decode tok/s at batch {a.batch} (Llama 3.2 1B shape, 256-token prompts)", "value": round(main["decode"], 1),
            "unit": "tokens/s", "n_gpus": 1, "steps": OUTPUTS - 1, "warmup": 1, "ms_per_step": round(main["ms_per_step"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids, random weights N(0, 0.02)",
            "config": describe(name, cfg, cfg["num_hidden_layers"], a.batch, 64, pk),
            "clocks": clock_info,
            "e2e": {"value": round(main["e2e"], 1), "unit": "tokens/s",
                    "how": "generated / run_seconds of stride_cli --path tc (256-token prompts, 256 outputs, prefill included), median of 3 after one discarded run"},
            "value_how": "decode steps alone: (run_seconds with 256 outputs - run_seconds with 1 output) / 255 steps; stride_cli prints no device time",
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "points": points,
            "prefill": {"unavailable": "a 2,048-token prompt is refused at intake: the context limit is 2,048 (src/scheduler.cpp:82-89, src/kernels.h:18)"},
            "reference": {"build": how, "device": main["device"], "run_seconds": main["run_seconds"], "first_token_seconds": main["first_token_seconds"],
                          "load_seconds": main["load_seconds"], "engine_steps": main["steps"], "model_written_s": round(wrote_s, 1),
                          "context_capacity": 2048},
        }))
        return 0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


# ---------------------------------------------------------------------------------------------------- this engine
def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="1b: the decode step (default); 3b, 8b: serving runs")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64, float32 and prefill measurements")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.shape != "1b":
        return serving_shape(a)

    import torch
    from stride_b200 import LLM, Engine, EngineOptions, StepEntry
    from stride_b200.kernels import ops

    name, cfg = SHAPES["1b"]
    cfg = dict(cfg)
    context = cfg["max_position_embeddings"]
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    max_batch = max(a.batch, 1 if a.skip_points else 64)
    page = 64
    regions = max(1, min(REGIONS, (context - PROMPT - a.warmup - 2) // max(a.steps, 1)))
    main_tokens = PROMPT + a.warmup + regions * a.steps + 1
    pages = max(a.batch * -(-main_tokens // page), max_batch * -(-(PROMPT + OUTPUTS + 8) // page)) + PREFILL_TOKENS // page + 8
    opts = EngineOptions(dtype="bfloat16", max_rows=max(PREFILL_TOKENS, max_batch), max_full_rows=max_batch, max_slots=max_batch + 1,
                         kv_pages=pages, page_size=page, max_context=context)
    engine = Engine.from_random(cfg, seed=0, options=opts)
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    kv_token_bytes = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    weight_bytes = engine.weight_bytes_per_step()

    def decode_run(eng, batch: int, steps: int, warmup: int, regions: int):
        """Prefill `batch` prompts of PROMPT tokens, run `warmup` decode steps, then time `regions` regions of exactly
        `steps` decode steps each. Returns ([(ms per step, mean context) per region], launches per step)."""
        cache = eng.cache
        slots = [cache.acquire_slot() for _ in range(batch)]
        prompts = torch.randint(0, vocab, (batch, PROMPT), generator=gen).tolist()
        per_step = max(1, eng.options.max_rows // PROMPT)
        for i in range(0, batch, per_step):
            entries = []
            for s, p in zip(slots[i:i + per_step], prompts[i:i + per_step]):
                cache.ensure(s, PROMPT)
                entries.append(StepEntry(s, 0, p, []))
            eng.step(entries)
        total = warmup + regions * steps
        tokens = torch.randint(0, vocab, (total, batch), generator=gen).tolist()
        out_tok = torch.zeros(batch, dtype=torch.int32, device=eng.device)
        out_val = torch.zeros(batch, dtype=torch.float32, device=eng.device)

        def one(k):
            pos = PROMPT + k
            entries = []
            for b, s in enumerate(slots):
                cache.ensure(s, pos + 1)
                entries.append(StepEntry(s, pos, [tokens[k][b]], [0]))
            logits = eng.step(entries)
            ops.argmax(logits, out_tok, out_val)

        for k in range(warmup):
            one(k)
        out, launches = [], 0
        for r in range(regions):
            torch.cuda.synchronize()
            l0 = ops.launches
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for k in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(k)
            stop.record()
            torch.cuda.synchronize()
            out.append((start.elapsed_time(stop) / steps, PROMPT + warmup + r * steps + (steps + 1) / 2.0))
            launches = (ops.launches - l0) // steps
        for s in slots:
            cache.release_slot(s)
        return out, launches

    def median_region(rs):
        return sorted(rs)[len(rs) // 2]

    def e2e_run(batch: int, repeats: int = 3):
        """The reference's offline workload through the Python entry point: `batch` prompts of 256 host token ids in,
        256 generated ids each back on the host, prefill included; generated / wall seconds, first run discarded."""
        llm = LLM(engine=engine, concurrency=batch, max_rows=opts.max_rows, prefill_chunk=PROMPT)
        prompts = offline_prompts(batch, PROMPT)
        rates = []
        for r in range(repeats + 1):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = llm.generate(prompts, max_new_tokens=OUTPUTS)
            dt = time.perf_counter() - t0
            if r > 0:
                rates.append(sum(len(o.tokens) for o in outs) / dt)
        return statistics.median(rates), llm.last_stats

    def prefill_run(reps: int = 5):
        cache = engine.cache
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        times = []
        for r in range(reps + 1):
            slot = cache.acquire_slot()
            cache.ensure(slot, PREFILL_TOKENS)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry(slot, 0, toks, [PREFILL_TOKENS - 1])])
            stop.record()
            torch.cuda.synchronize()
            if r > 0:
                times.append(start.elapsed_time(stop))
            cache.release_slot(slot)
        return statistics.median(times)

    def long_context_run(ctx: int, steps: int = 16, portion: int = 2048):
        """Milliseconds a decode step of one request that holds `ctx` cached tokens (its prompt fed in portions first)."""
        o = EngineOptions(dtype="bfloat16", max_rows=portion, max_full_rows=1, max_slots=2, kv_pages=ctx // page + 8, page_size=page,
                          max_context=ctx + 256)
        eng = Engine.from_random(cfg, seed=0, options=o)
        cache = eng.cache
        slot = cache.acquire_slot()
        toks = torch.randint(0, vocab, (ctx + steps + 8,), generator=gen).tolist()
        for a0 in range(0, ctx, portion):
            cache.ensure(slot, a0 + portion)
            eng.step([StepEntry(slot, a0, toks[a0:a0 + portion], [])])

        def one(k):
            cache.ensure(slot, ctx + k + 1)
            eng.step([StepEntry(slot, ctx + k, [toks[ctx + k]], [0])])
        for k in range(4):
            one(k)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(4, 4 + steps):
            one(k)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    clocks = ClockSampler()
    clocks.start()
    rs, launches = decode_run(engine, a.batch, a.steps, a.warmup, regions)
    clock_info = clocks.stop()
    ms, mean_ctx = median_region(rs)
    value = a.batch * 1000.0 / ms
    step_bytes = weight_bytes + a.batch * mean_ctx * kv_token_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e, stats = e2e_run(a.batch)
    points, prefill = {}, None
    if not a.skip_points:
        # decoding over the whole 256 outputs of the workload (contexts 256 -> 511), batch 1, 8 and 64
        for b in sorted({1, a.batch, 64}):
            pr, _ = decode_run(engine, b, OUTPUTS - 4, 3, 1)      # positions 256..510: the steps that make outputs 2..256
            points[f"decode_b{b}"] = round(b * 1000.0 / pr[0][0], 1)
        pms = prefill_run()
        fl = prefill_flops(cfg, PREFILL_TOKENS, layers)
        prefill = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                   "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        # the true 32-bit path, batch 1 (the reference publishes its exact path at batch 1 too)
        del engine
        torch.cuda.empty_cache()
        o32 = EngineOptions(dtype="float32", max_rows=PROMPT, max_full_rows=1, max_slots=2, kv_pages=16, page_size=page, max_context=context)
        e32 = Engine.from_random(cfg, seed=0, options=o32)
        r32, _ = decode_run(e32, 1, 16, 3, 1)
        points["decode_b1_float32"] = round(1000.0 / r32[0][0], 1)
        del e32
        torch.cuda.empty_cache()
        # one request with a long context (bfloat16): where a decode step is mostly the attention over its own cache
        try:
            lms = long_context_run(LONG_CONTEXT)
            points[f"decode_b1_ctx{LONG_CONTEXT}"] = round(1000.0 / lms, 1)
            points[f"hbm_frac_b1_ctx{LONG_CONTEXT}"] = round((weight_bytes + LONG_CONTEXT * kv_token_bytes) / (lms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        except Exception as e:          # the headline line does not hang on this point
            points[f"error_ctx{LONG_CONTEXT}"] = str(e)[:200]
    line = {
        "metric": f"decode tok/s at batch {a.batch} (Llama 3.2 1B shape, 256-token prompts)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random weights N(0, 0.02)",
        "config": describe(name, cfg, layers, a.batch, page, pk),
        "clocks": clock_info,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 9 * opts.max_rows * 4, "d2h_bytes_per_step": a.batch * 8,
                "how": "LLM.generate: 256-token prompts, 256 outputs, prefill included; generated / wall seconds, median of 3 after one discarded run",
                "engine_steps": stats.steps},
        "gpu_launches": launches * a.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "timed": {"regions": regions, "ms_per_step_of_each": [round(r[0], 4) for r in rs], "reported": "median"},
        "published_elsewhere": "the reference publishes RTX 4090 figures only (2,276 tok/s at batch 8 with prefill time): no vs_baseline",
        "points": points,
    }
    if prefill:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


def serving_shape(a) -> int:
    """The two larger shapes through the scheduler: 3B with 64 requests (prompts of 224 to 288 tokens, 256 outputs);
    8B with 128 requests and a cache pool small enough to force preemption, six of the requests checked against runs alone."""
    import torch
    from stride_b200 import LLM, Engine, EngineOptions

    name, cfg = SHAPES[a.shape]
    cfg = dict(cfg)
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    layers, context, page = cfg["num_hidden_layers"], cfg["max_position_embeddings"], 64
    pk = peaks()
    requests = 64 if a.shape == "3b" else 128
    rng = random.Random(33)
    prompts = [[128000] + [rng.randint(1000, 100000) for _ in range(rng.randint(224, 288) - 1)] for _ in range(requests)]
    need = sum(-(-(len(p) + OUTPUTS) // page) for p in prompts)
    pages = need + requests + 8 if a.shape == "3b" else need * 5 // 8        # 8B: five eighths of what all would hold at the end
    opts = EngineOptions(dtype="bfloat16", max_rows=2048, max_full_rows=requests, max_slots=requests + 1, kv_pages=pages,
                         page_size=page, max_context=context)
    engine = Engine.from_random(cfg, seed=0, options=opts)
    llm = LLM(engine=engine, concurrency=requests, max_rows=2048, prefill_chunk=256)
    clocks = ClockSampler()
    runs = []
    outs = None
    for r in range(3):
        if r == 1:
            clocks.start()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, max_new_tokens=OUTPUTS)
        dt = time.perf_counter() - t0
        if r > 0:
            runs.append((sum(len(o.tokens) for o in outs) / dt, dt, llm.last_stats))
    clock_info = clocks.stop()
    rate, dt, stats = sorted(runs, key=lambda x: x[0])[len(runs) // 2]
    exact = None
    if a.shape == "8b":
        # the same six requests alone: preemption and replay must not have changed a token or a logit's bits
        solo = LLM(engine=engine, concurrency=1, max_rows=2048, prefill_chunk=256)
        exact = 0
        for i in list(range(0, requests, max(1, requests // 6)))[:6]:
            alone = solo.generate([prompts[i]], max_new_tokens=OUTPUTS, seed=i)[0]
            exact += int(alone.tokens == outs[i].tokens and alone.fingerprint == outs[i].fingerprint)
    kv_token_bytes = layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    mean_ctx = sum(len(p) for p in prompts) / requests + OUTPUTS / 2.0
    line = {
        "metric": f"generated tok/s, {requests} requests through the scheduler ({name}, prompts of 224-288 tokens, {OUTPUTS} outputs, prefill included)",
        "value": round(rate, 1), "unit": "tokens/s", "n_gpus": 1, "steps": stats.steps, "warmup": 1, "ms_per_step": round(dt * 1e3 / max(stats.steps, 1), 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random weights N(0, 0.02)",
        "config": describe(name, cfg, layers, requests, page, pk), "clocks": clock_info,
        "serving": {"requests": requests, "wall_s": round(dt, 3), "engine_steps": stats.steps, "rows": stats.rows, "preemptions": stats.preemptions,
                    "replayed_rows": stats.replayed_rows, "peak_seqs": stats.peak_seqs, "peak_pages": stats.peak_blocks, "pages": pages,
                    "weight_bytes": engine.weight_bytes_per_step(), "kv_bytes_per_token": kv_token_bytes,
                    "decode_step_bytes_at_mean_context": engine.weight_bytes_per_step() + int(requests * mean_ctx * kv_token_bytes)},
    }
    if exact is not None:
        line["serving"]["requests_equal_to_solo_runs"] = f"{exact} of 6"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
