"""A linear layer without bias, out = x . W^T, with the kernel chosen by precision.

float32 engine: true 32-bit FMA (`csrc/gemm_f32.cu`) on float32 activations; the weight stays
as stored (bfloat16 is widened exactly inside the kernel).
bfloat16 engine: bfloat16 activations and weights with float32 accumulation on the tcgen05
tensor cores (`csrc/gemm_tc.cu`); a weight stored in float32, or a K that TMA cannot
address (not a multiple of 8), falls back to the SIMT kernel, which takes any size.

The tensor-core kernel cuts the K of a small weight into ranges (a function of the weight's shape
alone) whose sums are added in float32 in ascending order. With few tokens it leaves one partial
sum per range, so that the ranges run on different SMs; `forward_partials` and `forward_add` hand
those to the consumer (the rotation kernel, the next norm), which adds them. With many tokens the
kernel adds them itself, in the same order: a token's result has the same bits either way.
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
        self.tensor_core = (compute_dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                            and self.in_features % 8 == 0)
        self.splits = ops.gemm_tc_splits(self.out_features, self.in_features) if self.tensor_core else 1

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def _tc(self, x: torch.Tensor) -> bool:
        return self.tensor_core and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0

    def partial_elems(self, max_tokens: int) -> int:
        """Elements of the largest partial buffer `forward_partials` may need for up to max_tokens tokens."""
        rows = max_tokens
        if self.tensor_core:
            rows = max(rows, min(max_tokens, ops.gemm_tc_partial_tokens()) * self.splits)
        return rows * self.out_features

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """out[n, out_features] float32 = x . W^T, K in one range whatever the weight's shape."""
        if self._tc(x):
            ops.gemm_tc(x, self.weight, out, ops.STORE)
        else:
            ops.gemm_f32(x, self.weight, out, accumulate=False)

    def forward_partials(self, x: torch.Tensor, flat: torch.Tensor) -> torch.Tensor:
        """x . W^T as [S, n, out_features] float32 partial sums (S >= 1) carved from the flat buffer `flat`."""
        n, M = x.shape[0], self.out_features
        if not self._tc(x):
            out = flat[:n * M].view(1, n, M)
            ops.gemm_f32(x, self.weight, out[0], accumulate=False)
            return out
        S = self.splits if n <= ops.gemm_tc_partial_tokens() else 1     # buffers left; the ranges stay the same
        out = flat[:S * n * M].view(S, n, M)
        ops.gemm_tc(x, self.weight, out if S > 1 else out[0], ops.STORE, splits=self.splits)
        return out

    def forward_add(self, x: torch.Tensor, stream, flat: torch.Tensor = None) -> None:
        """stream += x . W^T (the residual add). With `flat` given, K is cut into the weight's ranges and, for few
        tokens, their partial sums are left pending on the stream; without it K stays one range. A call site
        must choose one of the two for good: the order of the sums differs."""
        if self._tc(x):
            n, M, S = x.shape[0], self.out_features, self.splits if flat is not None else 1
            if S > 1:
                # few tokens: one partial sum per range; many: the ranges' sum. Either way the stream's next
                # consumer computes h + (range_0 + range_1 + ...).
                P = S if n <= ops.gemm_tc_partial_tokens() else 1
                parts = flat[:P * n * M].view(P, n, M)
                ops.gemm_tc(x, self.weight, parts if P > 1 else parts[0], ops.STORE, splits=S)
                stream.set_pending(parts)
                return
            stream.fold()
            ops.gemm_tc(x, self.weight, stream.h, ops.ADD)
        else:
            stream.fold()
            ops.gemm_f32(x, self.weight, stream.h, accumulate=True)

    # ------------------------------------------------------------------ the same, as operations of the native step program
    # (`x`, `out`, `flat`, `z` are the full buffers, of which a step uses its first n rows)
    def _f32_op(self, program, x, out, ldo: int, accumulate: bool, wanted_rows: bool) -> None:
        program.add("gemm_f32", "sb_op_linear_f32", [x, x.dtype, x.stride(0), self.weight, self.weight.dtype, self.weight.stride(0), out, ldo,
                                                      self.out_features, self.in_features, int(accumulate), int(wanted_rows)])

    def _tc_op(self, program, x, out, mode: int, splits: int = 1, wanted_rows: bool = False) -> None:
        # the decode chain has phases for partial sums per K range and for SwiGLU, on the step's tokens
        phase = None
        if not wanted_rows and mode in (1, 3):
            phase = lambda chain: chain.linear(x, self.weight, out, mode == 3, splits if mode == 1 else 1)
        program.add("gemm_tc", "sb_op_linear_tc", [x, x.stride(0), self.weight, self.weight.stride(0), out, self.out_features,
                                                    self.in_features, mode, splits, int(wanted_rows)], chain=phase)

    def emit(self, program, x: torch.Tensor, out: torch.Tensor, wanted_rows: bool = False) -> None:
        """`forward`; with `wanted_rows` the rows are the step's wanted rows (the head), not its tokens."""
        if self._tc(x):
            self._tc_op(program, x, out, 0, wanted_rows=wanted_rows)
        else:
            self._f32_op(program, x, out, out.stride(0), False, wanted_rows)

    def emit_partials(self, program, x: torch.Tensor, flat: torch.Tensor) -> int:
        """`forward_partials`; returns the number of K ranges S that the reader of `flat` has to expect
        ([S, n, out_features] up to `program.few_tokens` tokens, [1, n, out_features] beyond)."""
        if not self._tc(x):
            self._f32_op(program, x, flat, self.out_features, False, False)
            return 1
        self._tc_op(program, x, flat, 1, self.splits)
        return self.splits

    def emit_add(self, program, x: torch.Tensor, flat: torch.Tensor = None) -> None:
        """`forward_add` onto the program's residual stream."""
        if self._tc(x) and flat is not None and self.splits > 1:
            program.need_folded("a projection that leaves partial sums")
            self._tc_op(program, x, flat, 1, self.splits)
            program.pending = (flat, self.splits, self.out_features)
            return
        program.need_folded("a projection")
        if self._tc(x):
            self._tc_op(program, x, program.h, 2)
        else:
            self._f32_op(program, x, program.h, program.h.stride(0), True, False)

    def emit_swiglu(self, program, x: torch.Tensor, z: torch.Tensor, scratch_fn) -> None:
        """`forward_swiglu`."""
        if self._tc(x) and z.dtype == torch.bfloat16:
            self._tc_op(program, x, z, 3)
        else:
            gate_up = scratch_fn()
            self._f32_op(program, x, gate_up, gate_up.stride(0), False, False)
            program.add("elementwise", "sb_op_swiglu", [gate_up, z, z.dtype, self.out_features // 2])

    def forward_swiglu(self, x: torch.Tensor, z: torch.Tensor, scratch_fn) -> None:
        """W = [gate rows; up rows]: z[n, I] = silu(x . gate^T) * (x . up^T). `scratch_fn()` gives a
        float32 [n, 2 I] buffer for the unfused path."""
        I = self.out_features // 2
        if self._tc(x) and z.dtype == torch.bfloat16:
            ops.gemm_tc(x, self.weight, z, ops.SWIGLU, half_rows=I)
        else:
            gate_up = scratch_fn()
            ops.gemm_f32(x, self.weight, gate_up, accumulate=False)
            ops.swiglu(gate_up, z)
