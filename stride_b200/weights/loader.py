"""Weights by tensor name, checked against the model's plan before anything is used.

The model's parts say which tensors they expect and with what shape
(`DecoderModel.tensor_plan()`); the loader compares that with what the file holds and
raises ONE error that lists every missing tensor, every unexpected tensor and every
wrong shape. Floating tensors stored in 16 bits are kept (or made) bfloat16; a tensor
stored in 32 bits stays float32; integer tables become int32.
Counterpart in arhaamatiq/stride: the Weights constructor (src/model.cpp:149-238), which
reads the same names and fails on the first missing one.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile


class WeightsError(RuntimeError):
    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


def check_plan(plan: dict, available: dict, source: str) -> None:
    """`plan`: name -> TensorPlan; `available`: name -> shape."""
    missing = [n for n, want in plan.items() if n not in available and not want.optional]
    unexpected = [n for n in available if n not in plan]
    wrong = [(n, tuple(available[n]), tuple(plan[n].shape)) for n in plan
             if n in available and tuple(available[n]) != tuple(plan[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"weights in {source} do not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n} is {list(have)}, expected {list(want)}" for n, have, want in sorted(wrong)))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def storage_dtype(dtype: torch.dtype, integer: bool) -> torch.dtype:
    if integer or not dtype.is_floating_point:
        return torch.int32
    return torch.float32 if dtype in (torch.float32, torch.float64) else torch.bfloat16


def load_weights(model_dir, plan: dict, device) -> dict:
    """Read `model.safetensors` of `model_dir`, check it against `plan`, return name -> device tensor."""
    path = Path(model_dir) / "model.safetensors"
    f = SafetensorsFile(path)
    try:
        check_plan(plan, {n: f.shape(n) for n in f.names()}, str(path))
        out = {}
        for name, want in plan.items():
            if not f.has(name):
                continue
            t = f.get(name)
            out[name] = t.to(device=device, dtype=storage_dtype(t.dtype, want.integer), copy=True)
        return out
    finally:
        f.close()
