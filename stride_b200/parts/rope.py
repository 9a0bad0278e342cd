"""Rotary position encoding: the table of cos and sin that the rotation kernel reads.

Restates arhaamatiq/stride's build_rope_table (src/model.cpp:54-88): the inverse
frequencies are computed in 32-bit, inv_i = 1 / float(pow(theta, double(float(2i)/float(D)))),
with the "llama3" rescaling of long waves; angle = inv_i * float(pos) in 32-bit;
cos and sin are evaluated in 64-bit and stored as 32-bit. Rotation pairs element d
with d + rotary_dim/2 (rotate-half); elements past rotary_dim are not rotated.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, register_part


def inverse_frequencies(rotary_dim: int, theta: float, scaling: dict) -> np.ndarray:
    f32 = np.float32
    half = rotary_dim // 2
    inv = np.empty(half, dtype=f32)
    kind = (scaling or {}).get("rope_type", "default")
    if kind not in ("default", "llama3"):
        raise ValueError(f"rotary encoding: unsupported scaling '{kind}' (supported: default, llama3)")
    for i in range(half):
        e = f32(2 * i) / f32(rotary_dim)
        f = f32(1.0) / f32(math.pow(theta, float(e)))
        if kind == "llama3":
            factor = f32(scaling["factor"])
            orig, low, high = scaling["original_max_position_embeddings"], scaling["low_freq_factor"], scaling["high_freq_factor"]
            low_wave, high_wave = f32(orig / low), f32(orig / high)
            wave = f32(2.0 * math.pi) / f
            smooth = (f32(orig) / wave - f32(low)) / f32(high - low)
            if wave > low_wave:
                f = f / factor
            elif not (wave < high_wave):
                f = (f32(1.0) - smooth) * (f / factor) + smooth * f
        inv[i] = f
    return inv


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim (default head_dim), theta, scaling (dict with rope_type and its factors)."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim or self.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and in 2..head_dim {self.head_dim}")
        inv = inverse_frequencies(self.rotary_dim, float(p["theta"]), p.get("scaling") or {})
        pos = np.arange(env.max_positions, dtype=np.float32)
        angle = (inv[None, :] * pos[:, None]).astype(np.float32).astype(np.float64)
        table = np.stack([np.cos(angle), np.sin(angle)], axis=-1).astype(np.float32)
        self.cos_sin = torch.from_numpy(table).to(env.device)   # [max_positions, rotary_dim / 2, 2]
