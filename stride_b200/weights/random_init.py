"""Random-weights mode: make a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors directly on a device.

Matrices are N(0, std) with std 0.02, norm gains 1 + N(0, gain_std) (0.1 by default, so
that a norm weight that is dropped or misplaced changes the result). Every tensor has its
own generator seeded from (seed, tensor name), so a tensor's values depend on neither
the order of generation nor the other tensors. arhaamatiq/stride has no such mode in its
engine; its tests build a tiny model with a Python script (tests/make_tiny_model.py:19-54).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config import resolve_architecture
from ..parts import BuildEnv, DecoderModel
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") >> 1


def model_plan(config: dict) -> dict:
    """The tensor plan (name -> TensorPlan) of the architecture that `config` names."""
    arch = resolve_architecture(config)
    spec = arch.model_spec(arch.parse_config(config))
    env = BuildEnv(device=torch.device("cpu"), compute_dtype=torch.float32, max_tokens=1, max_positions=2)
    return DecoderModel(spec, env).tensor_plan()


def random_tensors(config: dict, seed: int, device="cpu", dtype=torch.bfloat16, std: float = 0.02,
                   gain_std: float = 0.1, include_optional: bool | None = None) -> dict:
    """name -> tensor for every tensor of the plan. Optional tensors (an untied head) are made when
    `include_optional`, which defaults to config['tie_word_embeddings'] being false."""
    plan = model_plan(config)
    if include_optional is None:
        include_optional = config.get("tie_word_embeddings") is False
    device = torch.device(device)
    out = {}
    for name, want in plan.items():
        if want.optional and not include_optional:
            continue
        gen = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
        if want.integer:
            out[name] = torch.zeros(want.shape, dtype=torch.int32, device=device)
        elif len(want.shape) == 1:
            out[name] = (1.0 + gain_std * torch.randn(want.shape, generator=gen, device=device, dtype=torch.float32)).to(dtype)
        else:
            out[name] = (std * torch.randn(want.shape, generator=gen, device=device, dtype=torch.float32)).to(dtype)
    return out


def write_random_model(model_dir, config: dict, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                       gain_std: float = 0.1) -> Path:
    """Write `config.json` and `model.safetensors` for `config` into `model_dir`."""
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config, seed, "cpu", dtype, std, gain_std)
    (model_dir / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(model_dir / "model.safetensors", tensors, {"format": "pt", "seed": seed})
    return model_dir
