"""Shared fixtures: tiny configurations of the architecture, model folders with random
weights in a temporary place, and the replay harness."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Three tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256, "rope_theta": 10000.0,
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 128,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "intermediate_size": 320, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "rms_norm_eps": 1e-6, "max_position_embeddings": 256,
}
# Sizes that are no power of two, head_dim that is not hidden/heads, ratio 1, one more layer count.
TINY_C = {
    "model_type": "llama", "hidden_size": 88, "intermediate_size": 136, "num_hidden_layers": 1,
    "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 48, "vocab_size": 333, "rope_theta": 2500.0,
    "rope_scaling": {"type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "rms_norm_eps": 3e-4, "max_position_embeddings": 192,
}
# Head size 64 and ratio 4: the shapes the tensor-core attention kernels of the bfloat16 path take.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 512, "rope_theta": 10000.0,
    "tie_word_embeddings": True, "rms_norm_eps": 1e-5, "max_position_embeddings": 640,
}
TINY = {"A": (TINY_A, 0, 64), "B": (TINY_B, 2, 8), "C": (TINY_C, 5, 16), "D": (TINY_D, 9, 16),
        "U": (TINY_D, 13, 32)}   # config, weight seed, page size

# Weights N(0, 0.2) and gains 1 + 0.2 N(0, 1): large enough that attention is far from uniform and
# every part changes the logits, as arhaamatiq/stride's own tiny model does (tests/make_tiny_model.py:19-54).
TEST_STD, TEST_GAIN_STD = 0.2, 0.2


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> model folder written by the framework's random-weights mode."""
    from stride_b200.weights.random_init import write_random_model
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, (cfg, seed, _) in TINY.items():
        if name == "U":
            continue
        out[name] = write_random_model(root / name, cfg, seed, std=TEST_STD, gain_std=TEST_GAIN_STD)
    # "U": the shape of D with query and key projections scaled down, so that attention is close to
    # uniform and EVERY key, however far, carries weight 1/T: a kernel that loses one shows in float32.
    import json
    from stride_b200.weights.random_init import random_tensors
    from stride_b200.weights.safetensors_io import write_safetensors
    cfg, seed, _ = TINY["U"]
    tensors = random_tensors(cfg, seed, std=TEST_STD, gain_std=TEST_GAIN_STD)
    for n in tensors:
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            tensors[n] = (tensors[n].float() * 0.05).to(torch.bfloat16)
    (root / "U").mkdir()
    (root / "U" / "config.json").write_text(json.dumps(cfg))
    write_safetensors(root / "U" / "model.safetensors", tensors)
    out["U"] = root / "U"
    return out


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class TraceRun:
    """Drives bin/trace_run as a user would: one JSON line per step on its standard input, the next
    step only after `done <step>` came back."""

    def __init__(self, model_dir, dtype: str, out_dir, max_tokens: int, page_size: int = 64, extra=()):
        self.out_dir = Path(out_dir)
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
               "--out", str(out_dir), "--max-tokens", str(max_tokens), "--page-size", str(page_size), *extra]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step = 0

    def run(self, entries: list, end=()) -> int:
        """entries: [(id, tokens, want)]. Returns the step number."""
        s = self.step
        rec = {"step": s, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {s}":
            self.proc.wait(timeout=60)
            raise AssertionError(f"trace_run answered {line!r} to step {s} (exit code {self.proc.returncode})")
        self.step += 1
        return s

    def logits(self, step: int, vocab: int) -> torch.Tensor:
        return torch.from_numpy(np.fromfile(self.out_dir / f"{step}.f32", dtype="<f4").reshape(-1, vocab).copy())

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"
        return rc


def logit_tolerance(dtype: str, reference: torch.Tensor, noise: float | None = None) -> float:
    """Largest allowed |engine - plain| over a set of logits.

    float32: 2e-4 absolute at logits of rms ~1-2, the bound arhaamatiq/stride's own suite uses
    for its exact path (tests/test_correctness.py:21), scaled with the rms for other magnitudes.

    bfloat16: the engine is compared with the plain implementation rounding to bfloat16 at the same
    places. What is left: sums taken in another order, which now and then round an activation to
    the neighbouring bfloat16 value; the tensor cores accumulate with truncation (measured on B200:
    mean error 2e-6 of the result at K = 2048 against 3e-7 for a float32 FMA chain), so such flips are
    several times more frequent than between two float32 implementations. Measured on tiny
    configuration D (300 tokens): mean deviation 0.006 with SIMT contractions, 0.012 on the tensor
    cores, against a mean of 0.082 and a maximum of 1.02 for bfloat16's own rounding noise on the same
    tokens, `noise` = max |plain(bfloat16 rounding) - plain(float32)|. The yardstick is that noise:
    the engine has to stay within half of it. A dropped key, a wrong page, position or weight moves
    logits by more than the noise itself (tests/test_plain.py checks that for a single dropped key),
    and the same code paths are held to 2e-4 in float32. Without `noise`, 3% of the logits' rms.
    """
    rms = float(reference.float().pow(2).mean().sqrt())
    if dtype == "float32":
        return 2e-4 * max(rms, 1.0)
    if noise is not None:
        return 0.5 * noise
    return 3e-2 * rms


class Noise(float):
    """max |plain with bfloat16 rounding - plain in float32| over a set of logits; `.mean` is the mean of the same."""
    mean = 0.0


def bf16_noise(cfg, weights, tokens, rows=None) -> Noise:
    """The bfloat16 rounding noise of the plain implementation over all logits of the sequence (or at `rows`)."""
    import plain_llama as plain
    a = plain.forward(cfg, weights, tokens, torch.float32, torch.bfloat16, rows=rows)
    b = plain.forward(cfg, weights, tokens, torch.float32, None, rows=rows)
    noise = Noise(float((a - b).abs().max()))
    noise.mean = float((a - b).abs().mean())
    return noise


def check_mean_deviation(got: torch.Tensor, want: torch.Tensor, noise, what: str) -> None:
    """The second yardstick of the bfloat16 comparison, for whole sequences: the MEAN deviation of the engine from the
    plain implementation (rounding at the same places) stays within half of the MEAN of bfloat16's own rounding noise, the
    factor the maximum is held to as well. The maximum alone is set by the single worst logit and would let a defect pass
    that moves every logit a little. (Measured ratios of the means: 0.15 on tiny configuration D at 300 tokens, 0.29 at
    the 1B layer sizes over 2,048 tokens, where the same bits come out of 256-token portions through other kernels.)"""
    mean = float((got - want).abs().mean())
    assert mean <= 0.5 * noise.mean, f"{what}: mean |diff| {mean:.3e} > 0.5 x the mean rounding noise {noise.mean:.3e}"
