"""A linear layer without bias, out = x . W^T, with the kernel chosen by precision.

float32 engine: true 32-bit FMA (`csrc/gemm_f32.cu`) on float32 activations; the
weight stays as stored (bfloat16 is widened exactly inside the kernel).
bfloat16 engine: bfloat16 activations and weights, float32 accumulation; the
tensor-core kernel where the shape allows it, else the same SIMT kernel.
"""
from __future__ import annotations

import torch

from . import ops


class Linear:
    def __init__(self, weight: torch.Tensor, compute_dtype: torch.dtype):
        if weight.dim() != 2:
            raise ValueError("Linear takes a [out, in] matrix")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.compute_dtype = compute_dtype

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """out[n, out_features] float32 = x . W^T."""
        ops.gemm_f32(x, self.weight, out, accumulate=False)

    def forward_add(self, x: torch.Tensor, stream) -> None:
        """stream += x . W^T (the residual add)."""
        if stream.pending is not None:
            stream.fold()
        ops.gemm_f32(x, self.weight, stream.h, accumulate=True)
