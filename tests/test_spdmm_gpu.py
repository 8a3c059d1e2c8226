"""GPU parity of the sparse x dense product and its backward, through the operator functions
on the C ABI, against golden vectors from the reference and the CPU oracle."""
import pytest
import torch

from parity import assert_close, assert_same, case, case_names
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["compiled shim", "python shim"])
def ops(request):
    from numml_b200 import numml_torch_cpp
    old = numml_torch_cpp.use_compiled_shim
    numml_torch_cpp.use_compiled_shim = request.param == "compiled shim"
    yield numml_torch_cpp
    numml_torch_cpp.use_compiled_shim = old


def test_golden_spdmm(golden_ops, ops):
    for name in case_names(golden_ops, "spdmm_"):
        c = case(golden_ops, name)
        m, n = int(c["shape"][0]), int(c["shape"][1])
        d, i, p, B, G = [c[k].cuda() for k in ("data", "indices", "indptr", "B", "G")]
        assert_same(c["C"], ops.spdmm_forward(m, n, d, i, p, B), name)      # storage-order sums: bit-exact
        gA, gB = ops.spdmm_backward(m, n, d, i, p, B, G)
        assert_close(c["grad_A"], gA, name)                                 # dot product is tree-reduced
        assert_same(c["grad_B"], gB, name)                                  # gather over A^T: bit-exact


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("K", [1, 3, 4, 8, 16, 30, 32, 64, 128, 130, 260])
def test_random_vs_oracle(oracle, ops, dtype, K):
    d, i, p, (m, n) = W.random_csr(300, 200, 0.03, seed=K, dtype=dtype)
    B, G = W.randn((n, K), 1, dtype), W.randn((m, K), 2, dtype)
    C_ref = oracle.spdmm_forward(m, n, d, i, p, B)
    gA_ref, gB_ref = oracle.spdmm_backward(m, n, d, i, p, B, G)
    dd, di, dp, dB, dG = [t.cuda() for t in (d, i, p, B, G)]
    assert_same(C_ref, ops.spdmm_forward(m, n, dd, di, dp, dB), "C")
    gA, gB = ops.spdmm_backward(m, n, dd, di, dp, dB, dG)
    assert_close(gA_ref, gA, "grad_A")
    assert_same(gB_ref, gB, "grad_B")


def _rows_of_given_lengths(lengths, n, seed):
    """CSR matrix whose row r has lengths[r] entries in sorted distinct random columns, N(0,1) values."""
    import numpy as np
    rng = np.random.default_rng(seed)
    cols = [np.sort(rng.choice(n, size=int(k), replace=False)) for k in lengths]
    ptr = np.concatenate(([0], np.cumsum([len(c) for c in cols])))
    idx = np.concatenate(cols) if ptr[-1] > 0 else np.zeros(0, dtype=np.int64)
    dat = rng.standard_normal(int(ptr[-1])).astype(np.float32)
    return torch.from_numpy(dat), torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(ptr.astype(np.int64))


def test_long_and_empty_rows(oracle, ops):
    """Power-law rows (1 ... 700 entries) next to empty ones, a random matrix with empty rows, and rows of 4096
    and 5000 entries (the graph benchmark's longest rows and beyond) between empty and one-entry rows: the
    degree-ordered row schedule and the lane-group walk of a long row give the oracle's bits."""
    d, i, p, (m, n) = W.powerlaw_graph(3000, scale=8, max_deg=700, seed=3, dtype=torch.float32)
    d2, i2, p2, _ = W.random_csr(m, n, 0.0005, seed=9, dtype=torch.float32)   # has empty rows
    lengths = [4096, 0, 5000, 1, 0, 700, 4096, 33, 0, 2] + [7] * 200 + [0, 4096] + [1] * 50
    d3, i3, p3 = _rows_of_given_lengths(lengths, 6000, seed=11)
    for (dat, idx, ptr, m, n) in ((d, i, p, m, n), (d2, i2, p2, m, n), (d3, i3, p3, len(lengths), 6000)):
        B, G = W.randn((n, 128), 1, torch.float32), W.randn((m, 128), 2, torch.float32)
        C_ref = oracle.spdmm_forward(m, n, dat, idx, ptr, B)
        gA_ref, gB_ref = oracle.spdmm_backward(m, n, dat, idx, ptr, B, G)
        dd, di, dp, dB, dG = [t.cuda() for t in (dat, idx, ptr, B, G)]
        assert_same(C_ref, ops.spdmm_forward(m, n, dd, di, dp, dB), "C")
        gA, gB = ops.spdmm_backward(m, n, dd, di, dp, dB, dG)
        assert_close(gA_ref, gA, "grad_A")
        assert_same(gB_ref, gB, "grad_B")


def test_noncontiguous_dense_operand(oracle, ops):
    d, i, p, (m, n) = W.random_csr(50, 40, 0.2, seed=1, dtype=torch.float64)
    Bt = W.randn((16, n), 1, torch.float64)
    C_ref = oracle.spdmm_forward(m, n, d, i, p, Bt.T.contiguous())
    assert_same(C_ref, ops.spdmm_forward(m, n, d.cuda(), i.cuda(), p.cuda(), Bt.cuda().T), "C")


def test_linearity_at_scale(ops):
    """Size-independent property on a large graph: A(aX + Y) == a AX + AY up to rounding, and
    row-normalised A maps the all-ones matrix to all-ones."""
    d, i, p, (m, n) = W.powerlaw_graph(1 << 18, seed=0, dtype=torch.float32)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    X, Y = W.randn((n, 128), 1, torch.float32).cuda(), W.randn((n, 128), 2, torch.float32).cuda()
    lhs = ops.spdmm_forward(m, n, dd, di, dp, 2.5 * X + Y)
    rhs = 2.5 * ops.spdmm_forward(m, n, dd, di, dp, X) + ops.spdmm_forward(m, n, dd, di, dp, Y)
    assert_close(rhs, lhs, "linearity", tol=1e-5)
    ones = ops.spdmm_forward(m, n, dd, di, dp, torch.ones((n, 128), dtype=torch.float32, device="cuda"))
    assert torch.allclose(ones, torch.ones_like(ones), atol=1e-3)  # rows of up to 4096 fp32 terms
