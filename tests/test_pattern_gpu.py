"""GPU parity of the pattern-building operators (tril / triu, linear combination on the union
pattern, COO -> CSR) against the CPU oracle: structure and values bit for bit, gradients through
the public API."""
import numpy as np
import pytest
import torch

from parity import assert_same
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from numml_b200 import numml_torch_cpp
    return numml_torch_cpp


@pytest.fixture(scope="module")
def sp():
    import numml_b200.sparse as sp
    return sp


def cuda(*ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape,density", [((1, 1), 1.0), ((40, 70), 0.2), ((900, 700), 0.01), ((300, 300), 0.08)])
def test_triangle_vs_oracle(oracle, ops, dtype, shape, density):
    d, i, p, (m, n) = W.random_csr(shape[0], shape[1], density, seed=11, dtype=dtype)
    dd, di, dp = cuda(d, i, p)
    for k in (-3, 0, 2):
        for lower in (True, False):
            ref = oracle.triangle(m, d, i, p, k, lower)
            got = ops.csr_triangle(m, n, dd, di, dp, k, lower)
            for name, a, b in zip(("data", "indices", "indptr", "positions"), ref, got):
                assert_same(a, b, f"{name} k={k} lower={lower}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_lincomb_vs_oracle(oracle, ops, dtype):
    cases = [(W.random_csr(500, 400, 0.02, seed=21, dtype=dtype), W.random_csr(500, 400, 0.03, seed=22, dtype=dtype)),
             (W.poisson2d_5pt(40, dtype), W.random_csr(1600, 1600, 0.002, seed=23, dtype=dtype)),
             (W.random_csr(7, 5, 0.5, seed=24, dtype=dtype), W.random_csr(7, 5, 0.0, seed=25, dtype=dtype))]
    for A, B in cases:
        (ad, ai, ap, (m, n)), (bd, bi, bp, _) = A, B
        for alpha, beta in ((1.0, 1.0), (1.0, -1.0), (0.3, 2.5)):
            ref = oracle.splincomb_forward(m, n, alpha, ad, ai, ap, beta, bd, bi, bp)
            got = ops.splincomb_forward(m, n, alpha, *cuda(ad, ai, ap), beta, *cuda(bd, bi, bp))
            for name, a, b in zip(("data", "indices", "indptr"), ref, got):
                assert_same(a, b, f"{name} alpha={alpha} beta={beta}")
            gC = W.randn(ref[0].numel(), 3, dtype)
            gref = oracle.splincomb_backward(m, n, alpha, ad, ai, ap, beta, bd, bi, bp, gC, ref[1], ref[2])
            ggot = ops.splincomb_backward(m, n, alpha, *cuda(ad, ai, ap), beta, *cuda(bd, bi, bp), gC.cuda(), got[1], got[2])
            assert_same(gref[0], ggot[0], "grad_A")
            assert_same(gref[1], ggot[1], "grad_B")


def test_coo_to_csr_order(ops):
    rng = np.random.default_rng(4)
    nrows, ncols, n = 700, 900, 20000
    r = torch.from_numpy(rng.integers(0, nrows, n)).cuda()
    c = torch.from_numpy(rng.integers(0, ncols, n)).cuda()          # with repeated (row, column) pairs
    perm, indptr = ops.coo_to_csr_order(r, c, nrows, ncols, sort_columns=True)
    expect = torch.argsort(r * ncols + c, stable=True)
    assert_same(expect, perm, "order by (row, column), stable")
    counts = torch.bincount(r, minlength=nrows)
    assert_same(torch.cat((torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(counts, 0))), indptr, "indptr")
    perm, indptr2 = ops.coo_to_csr_order(r, c, nrows, ncols, sort_columns=False)
    assert_same(torch.argsort(r, stable=True), perm, "order by row only, stable")
    assert_same(indptr, indptr2, "indptr")
    perm, indptr = ops.coo_to_csr_order(r[:0], c[:0], 5, 5)
    assert perm.numel() == 0 and indptr.tolist() == [0] * 6
    with pytest.raises(RuntimeError):
        ops.coo_to_csr_order(torch.tensor([7]).cuda(), torch.tensor([0]).cuda(), 5, 5)


def test_api_builds_and_differentiates_on_the_device(sp, oracle):
    """The public methods on CUDA tensors: tril / triu, A + B, A - B, and the COO constructor, with
    gradients flowing to the stored values of the operands."""
    d, i, p, (m, n) = W.random_csr(120, 120, 0.08, seed=31, dtype=torch.float64)
    d2, i2, p2, _ = W.random_csr(120, 120, 0.05, seed=32, dtype=torch.float64)
    A = sp.SparseCSRTensor((d, i, p), (m, n)).to("cuda")
    B = sp.SparseCSRTensor((d2, i2, p2), (m, n)).to("cuda")
    A.requires_grad = True
    B.requires_grad = True
    L = A.tril(-1)
    ref = oracle.triangle(m, d, i, p, -1, True)
    assert_same(ref[0], L.data.detach(), "tril data")
    assert_same(ref[1], L.indices, "tril indices")
    assert_same(ref[2], L.indptr, "tril indptr")
    w = W.randn(L.nnz, 1, torch.float64).cuda()
    (L.data * w).sum().backward()
    expect = torch.zeros_like(d)
    expect[ref[3]] = w.cpu()
    assert_same(expect, A.data.grad, "gradient through tril")
    A.data.grad = None
    C = A - B
    cref = oracle.splincomb_forward(m, n, 1.0, d, i, p, -1.0, d2, i2, p2)
    assert_same(cref[0], C.data.detach(), "A - B data")
    assert_same(cref[1], C.indices, "A - B indices")
    wc = W.randn(C.nnz, 2, torch.float64).cuda()
    (C.data * wc).sum().backward()
    gref = oracle.splincomb_backward(m, n, 1.0, d, i, p, -1.0, d2, i2, p2, wc.cpu(), cref[1], cref[2])
    assert_same(gref[0], A.data.grad, "gradient of A through A - B")
    assert_same(gref[1], B.data.grad, "gradient of B through A - B")
    # COO constructor on the device
    rows = torch.repeat_interleave(torch.arange(m), p[1:] - p[:-1])
    shuffle = torch.randperm(d.numel(), generator=torch.Generator().manual_seed(0))
    M = sp.SparseCSRTensor((d[shuffle].cuda(), (rows[shuffle].cuda(), i[shuffle].cuda())), shape=(m, n))
    assert_same(d, M.data, "COO -> CSR data")
    assert_same(i, M.indices, "COO -> CSR indices")
    assert_same(p, M.indptr, "COO -> CSR indptr")
