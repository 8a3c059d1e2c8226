"""Kernels that use no floating-point atomics must return the same bits on every run: each is run
twice on the same inputs and the outputs are compared exactly.  The SpGEMM forward is included for
rows of at most 32 products, which one warp forms without a table and sums in the reference's
order (the stencil and Galerkin products of the benchmark configuration); rows that go through the
hash tables accumulate colliding products with atomics and are order-stable only in structure."""
import pytest
import torch

from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _twice(fn):
    a = fn()
    torch.cuda.synchronize()
    b = fn()
    torch.cuda.synchronize()
    a = a if isinstance(a, (list, tuple)) else [a]
    b = b if isinstance(b, (list, tuple)) else [b]
    for u, v in zip(a, b):
        assert torch.equal(u, v), "two runs on the same inputs differ"


def test_products_and_their_backward_are_run_to_run_identical():
    import numml_b200.numml_torch_cpp as ops
    assert ops.spmv_backward_mode == "transpose"          # the default backward has no atomics
    d, i, p, (m, k) = W.powerlaw_graph(1 << 14, scale=4, seed=3, dtype=torch.float32)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    x, g = W.randn(k, 0, torch.float32).cuda(), W.randn(m, 1, torch.float32).cuda()
    X, G = W.randn((k, 24), 2, torch.float32).cuda(), W.randn((m, 24), 3, torch.float32).cuda()
    _twice(lambda: ops.spgemv_forward(m, k, dd, di, dp, x))
    _twice(lambda: ops.spgemv_backward(g, m, k, dd, di, dp, x))
    _twice(lambda: ops.spdmm_forward(m, k, dd, di, dp, X))
    _twice(lambda: ops.spdmm_backward(m, k, dd, di, dp, X, G))
    _twice(lambda: ops.csr_transpose_forward(m, k, dd, di, dp))


def test_stencil_kernels_solves_and_cg_are_run_to_run_identical():
    import numml_b200.numml_torch_cpp as ops
    d, i, p, (m, k) = W.poisson3d_7pt(32, torch.float64)
    d = W.randn(d.numel(), 5, torch.float64)              # values that are not symmetric
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    x, g = W.randn(k, 0, torch.float64).cuda(), W.randn(m, 1, torch.float64).cuda()
    _twice(lambda: ops.spgemv_forward(m, k, dd, di, dp, x))
    _twice(lambda: ops.spgemv_backward(g, m, k, dd, di, dp, x))            # fused one-pass backward
    A = W.poisson2d_5pt(48, torch.float64)
    Ad = [t.cuda() for t in A[:3]]
    n = 48 * 48
    _twice(lambda: ops.spgemm_forward(n, n, *Ad, n, n, *Ad))                # every row has at most 25 products
    C = ops.spgemm_forward(n, n, *Ad, n, n, *Ad)
    gC = W.randn(C[0].numel(), 6, torch.float64).cuda()
    _twice(lambda: ops.spgemm_backward(gC, C[1], C[2], n, n, *Ad, n, n, *Ad))
    ld, li, lp, (lm, _) = W.poisson2d_9pt_lower(64, torch.float64)
    Ld = [t.cuda() for t in (ld, li, lp)]
    B = W.randn((lm, 3), 7, torch.float64).cuda()
    _twice(lambda: ops.sptrsv_forward(lm, lm, *Ld, True, False, B))
    Xs = ops.sptrsv_forward(lm, lm, *Ld, True, False, B)
    _twice(lambda: ops.sptrsv_backward(B, Xs, lm, lm, *Ld, True, False, B))
    spd = [t.cuda() for t in W.poisson3d_7pt(16, torch.float64)[:3]]
    b = W.randn(16 ** 3, 8, torch.float64).cuda()
    _twice(lambda: ops.cg_fixed_iterations(16 ** 3, *spd, b, None, 30))
