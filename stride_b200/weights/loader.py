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
    """How a checkpoint tensor is kept: bfloat16 as it is, 32- and 64-bit floating point as float32, and float16 as
    float32 too (every float16 value is a float32 value, while bfloat16 would drop three bits of its mantissa without a
    word); integers as int32."""
    if integer or not dtype.is_floating_point:
        return torch.int32
    return torch.bfloat16 if dtype == torch.bfloat16 else torch.float32


def _open_files(model_dir) -> dict:
    """name of every tensor of the model folder -> the open file that holds it: `model.safetensors`, or the shards
    that `model.safetensors.index.json` names (its `weight_map`: tensor name -> file name), as large checkpoints are
    distributed. arhaamatiq/stride reads the single file only (src/model.cpp:150)."""
    folder = Path(model_dir)
    single, index = folder / "model.safetensors", folder / "model.safetensors.index.json"
    if single.exists() or not index.exists():
        f = SafetensorsFile(single)
        return {n: f for n in f.names()}
    import json
    try:
        weight_map = json.loads(index.read_text())["weight_map"]
    except (ValueError, KeyError, TypeError) as e:
        raise WeightsError(f"{index} is not a shard index (a JSON object with a weight_map): {e}") from e
    files, where = {}, {}
    try:
        for name, shard in sorted(weight_map.items()):
            if shard not in files:
                files[shard] = SafetensorsFile(folder / shard)
            if not files[shard].has(name):
                raise WeightsError(f"{index} says that {shard} holds {name}, which it does not")
            where[name] = files[shard]
    except Exception:
        for f in files.values():
            f.close()
        raise
    return where


def load_weights(model_dir, plan: dict, device) -> dict:
    """Read the model folder's safetensors (one file or shards), check them against `plan`, return name -> device tensor."""
    where = _open_files(model_dir)
    try:
        check_plan(plan, {n: f.shape(n) for n, f in where.items()}, str(Path(model_dir)))
        out = {}
        for name, want in plan.items():
            if name not in where:
                continue
            t = where[name].get(name)
            out[name] = t.to(device=device, dtype=storage_dtype(t.dtype, want.integer), copy=True)
        return out
    finally:
        for f in {id(f): f for f in where.values()}.values():
            f.close()
