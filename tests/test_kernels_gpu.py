"""Each CUDA kernel alone against a plain torch reference of the same operation, at sizes other
than the engine's test configurations."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("n,M,K", [(1, 128, 64), (5, 200, 72), (16, 256, 512), (33, 384, 2048), (64, 1000, 136),
                                   (128, 128, 8192), (200, 333, 264), (777, 520, 1024)])
def test_gemm_tc_store_and_add(n, M, K):
    from stride_b200.kernels import ops
    x = _rand(n, K, seed=1, dtype=torch.bfloat16)
    w = _rand(M, K, seed=2, scale=0.05, dtype=torch.bfloat16)
    ref = x.float() @ w.float().T
    tol = 2e-3 * float(ref.abs().max()) + 1e-5      # float32 accumulation in another order
    out = torch.full((n, M), float("nan"), device=DEV)
    ops.gemm_tc(x, w, out, ops.STORE)
    assert ops.gemm_tc_status() == 0
    assert (out - ref).abs().max() <= tol
    base = _rand(n, M, seed=3)
    acc = base.clone()
    ops.gemm_tc(x, w, acc, ops.ADD)
    assert ops.gemm_tc_status() == 0
    assert (acc - (base + ref)).abs().max() <= tol
    splits = ops.gemm_tc_splits(n, M, K)
    if splits > 1:
        parts = torch.full((splits, n, M), float("nan"), device=DEV)
        ops.gemm_tc(x, w, parts, ops.STORE, splits=splits)
        assert ops.gemm_tc_status() == 0
        assert (parts.sum(0) - ref).abs().max() <= tol


def test_gemm_tc_one_hot_positions():
    """x rows that are unit vectors pick single columns of W: any wrong swizzle, descriptor step or
    tile offset shows as a wrong element, not as a small numeric difference."""
    from stride_b200.kernels import ops
    n, M, K = 96, 256, 256
    w = _rand(M, K, seed=4, dtype=torch.bfloat16)
    idx = torch.arange(n) * 37 % K
    x = torch.zeros(n, K, dtype=torch.bfloat16, device=DEV)
    x[torch.arange(n), idx] = 1.0
    out = torch.zeros(n, M, device=DEV)
    ops.gemm_tc(x, w, out, ops.STORE)
    assert ops.gemm_tc_status() == 0
    assert torch.equal(out, w.float()[:, idx.to(DEV)].T.contiguous())


@pytest.mark.parametrize("n,I,K", [(3, 64, 64), (40, 200, 136), (130, 320, 192), (300, 1024, 512)])
def test_gemm_tc_swiglu(n, I, K):
    from stride_b200.kernels import ops
    x = _rand(n, K, seed=5, dtype=torch.bfloat16)
    w = _rand(2 * I, K, seed=6, scale=0.1, dtype=torch.bfloat16)
    g = x.float() @ w[:I].float().T
    u = x.float() @ w[I:].float().T
    ref = (g / (1 + torch.exp(-g))) * u
    out = torch.full((n, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, out, ops.SWIGLU, half_rows=I)
    assert ops.gemm_tc_status() == 0
    assert (out.float() - ref).abs().max() <= 1e-2 * float(ref.abs().max()) + 1e-4


def test_gemm_tc_does_not_depend_on_the_batch():
    """A token's result has the same bits alone, among 7 and among 200 other tokens (same split-K)."""
    from stride_b200.kernels import ops
    M, K = 384, 1024
    w = _rand(M, K, seed=7, scale=0.05, dtype=torch.bfloat16)
    x = _rand(200, K, seed=8, dtype=torch.bfloat16)
    outs = []
    for n in (1, 8, 200):
        out = torch.zeros(n, M, device=DEV)
        ops.gemm_tc(x[:n].contiguous(), w, out, ops.STORE)
        outs.append(out[0].clone())
    assert ops.gemm_tc_status() == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
