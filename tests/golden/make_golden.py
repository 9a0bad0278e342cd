"""Makes tests/golden/ref_cpu_ratio4.json: logits of arhaamatiq/stride's own CPU
exact path on a tiny random model, to anchor tests/plain_llama.py.

stride's CPU build accepts only a head ratio of 4 (src/model.cpp:49), bfloat16
weights, rows % 4 == 0 and cols % 8 == 0 (src/model.cpp:189), so the tiny
configurations of the test-suite themselves rest on the formulas; this one
configuration is what the reference can run.

Usage (needs g++ and a checkout of the reference; nothing is written outside
the given scratch folder and this folder):

    python tests/golden/make_golden.py --reference /path/to/stride --scratch /tmp/refbuild

It compiles the reference's CPU backend (kernels.cu as plain C++), writes the
model folder and prompts into the scratch folder, runs
`stride_cli --path exact --full --dump-logits` with 4 dumped steps, and stores
config, seed, prompts, generated tokens and the dumped logits (as 32-bit hex
words) in the JSON file. The weights are not stored: they are regenerated
from the seed by `golden_model()` below, which the test imports.
"""
from __future__ import annotations

import argparse
import json
import struct
import subprocess
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import plain_llama as plain  # noqa: E402

CONFIG = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 250, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": False,
}
SEED = 11
PROMPT_LENGTHS = [1, 7, 40, 130]
NEW_TOKENS = 6
DUMP_STEPS = 4


def golden_model(seed: int = SEED) -> dict:
    """Weights N(0, 0.2) so that every part matters, norm gains 1 + 0.2 N(0, 1)."""
    g = torch.Generator().manual_seed(seed)
    c = CONFIG
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    Hq, Hkv, D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]

    def mat(r, k):
        return (torch.randn(r, k, generator=g) * 0.2).to(torch.bfloat16)

    def gain(n):
        return (1.0 + 0.2 * torch.randn(n, generator=g)).to(torch.bfloat16)

    w = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": gain(H), "lm_head.weight": mat(V, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = mat(Hq * D, H)
        w[p + "self_attn.k_proj.weight"] = mat(Hkv * D, H)
        w[p + "self_attn.v_proj.weight"] = mat(Hkv * D, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, Hq * D)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
        w[p + "input_layernorm.weight"] = gain(H)
        w[p + "post_attention_layernorm.weight"] = gain(H)
    return w


def golden_prompts(seed: int = SEED) -> list:
    g = torch.Generator().manual_seed(seed + 1)
    return [torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for n in PROMPT_LENGTHS]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--scratch", required=True)
    ap.add_argument("--json-include", default="", help="folder that holds nlohmann/json.hpp")
    a = ap.parse_args()
    ref, scratch = Path(a.reference), Path(a.scratch)
    scratch.mkdir(parents=True, exist_ok=True)
    exe = scratch / "stride_cli_cpu"
    if not exe.exists():
        src = [str(ref / "src" / f) for f in ("safetensors.cpp", "model.cpp", "kv_cache.cpp", "engine.cpp", "scheduler.cpp")]
        cmd = ["g++", "-std=c++17", "-O3", "-fno-fast-math", "-ffp-contract=off", "-fno-strict-aliasing",
               "-mfma", "-mavx2", f"-I{ref / 'src'}"]
        if a.json_include:
            cmd.append(f"-I{a.json_include}")
        cmd += src + [str(ref / "tools" / "stride_cli.cpp"), "-x", "c++", str(ref / "src" / "kernels.cu"),
                      str(ref / "src" / "device.cu"), "-lpthread", "-o", str(exe)]
        subprocess.run(cmd, check=True)
    model = scratch / "golden_model"
    model.mkdir(exist_ok=True)
    (model / "config.json").write_text(json.dumps(CONFIG))
    plain.write_safetensors(model / "model.safetensors", golden_model())
    prompts = golden_prompts()
    (scratch / "prompts.jsonl").write_text("".join(json.dumps({"id": i, "tokens": p}) + "\n" for i, p in enumerate(prompts)))
    subprocess.run([str(exe), "--model", str(model), "--input", str(scratch / "prompts.jsonl"),
                    "--output", str(scratch / "out.jsonl"), "--max-new", str(NEW_TOKENS), "--path", "exact",
                    "--full", "--dump-logits", str(scratch / "logits.f32"), "--dump-steps", str(DUMP_STEPS)], check=True)
    outs = [json.loads(l) for l in (scratch / "out.jsonl").read_text().splitlines()]
    raw = (scratch / "logits.f32").read_bytes()
    V = CONFIG["vocab_size"]
    assert len(raw) == 4 * V * DUMP_STEPS * len(prompts), len(raw)
    words = struct.unpack(f"<{len(raw) // 4}I", raw)
    golden = {"config": CONFIG, "seed": SEED, "prompts": prompts, "new_tokens": NEW_TOKENS, "dump_steps": DUMP_STEPS,
              "tokens": [o["tokens"] for o in outs],
              "logits_hex": ["%08x" % x for x in words]}
    out = Path(__file__).with_name("ref_cpu_ratio4.json")
    out.write_text(json.dumps(golden))
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
