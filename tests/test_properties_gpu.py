"""Property tests over small random CSR matrices (hypothesis): ragged rows, empty rows and
columns, 1 x n and n x 1 shapes, both value types.  Every operator is compared with the CPU
oracle on the same input; index arrays must match exactly."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from parity import assert_close, assert_same

pytestmark = pytest.mark.gpu
SETTINGS = dict(max_examples=30, deadline=None, derandomize=True,
                suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


@st.composite
def csr(draw, max_rows=40, max_cols=40, square=False):
    rows = draw(st.integers(1, max_rows))
    cols = rows if square else draw(st.integers(1, max_cols))
    density = draw(st.sampled_from([0.0, 0.05, 0.3, 1.0]))
    seed = draw(st.integers(0, 2 ** 16))
    dtype = draw(st.sampled_from([torch.float32, torch.float64]))
    rng = np.random.default_rng(seed)
    mask = rng.random((rows, cols)) < density
    if draw(st.booleans()) and rows > 2:
        mask[rng.integers(0, rows)] = False          # an empty row
    r, c = np.nonzero(mask)
    indptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(np.bincount(r, minlength=rows), out=indptr[1:])
    data = torch.from_numpy(rng.standard_normal(len(c))).to(dtype)
    return data, torch.from_numpy(c.astype(np.int64)), torch.from_numpy(indptr), (rows, cols), seed


def _ops():
    from numml_b200 import numml_torch_cpp
    return numml_torch_cpp


@settings(**SETTINGS)
@given(csr())
def test_spmv_and_transpose(oracle, A):
    ops = _ops()
    d, i, p, (m, n), seed = A
    g = torch.Generator().manual_seed(seed)
    x, up = torch.randn(n, generator=g, dtype=d.dtype), torch.randn(m, generator=g, dtype=d.dtype)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    assert_close(oracle.spgemv_forward(m, n, d, i, p, x), ops.spgemv_forward(m, n, dd, di, dp, x.cuda()), "y")
    gA_ref, gx_ref = oracle.spgemv_backward(up, m, n, d, i, p, x)
    gA, gx = ops.spgemv_backward(up.cuda(), m, n, dd, di, dp, x.cuda())
    assert_same(gA_ref, gA, "grad_A")
    assert_close(gx_ref, gx, "grad_x")
    for ref, got, what in zip(oracle.csr_transpose_forward(m, n, d, i, p), ops.csr_transpose_forward(m, n, dd, di, dp),
                              ("t_data", "t_indices", "t_indptr", "t_perm")):
        assert_same(ref, got, what)


@settings(**SETTINGS)
@given(csr(), st.integers(1, 40), st.integers(0, 2 ** 16))
def test_spgemm_structure_and_gradients(oracle, A, b_cols, seed):
    ops = _ops()
    d, i, p, (m, n), _ = A
    rng = np.random.default_rng(seed)
    mask = rng.random((n, b_cols)) < 0.3
    r, c = np.nonzero(mask)
    bp = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(r, minlength=n), out=bp[1:])
    bd, bi, bp = torch.from_numpy(rng.standard_normal(len(c))).to(d.dtype), torch.from_numpy(c.astype(np.int64)), torch.from_numpy(bp)
    Cd_ref, Ci_ref, Cp_ref = oracle.spgemm_forward(m, n, d, i, p, n, b_cols, bd, bi, bp)
    dA, dB = [t.cuda() for t in (d, i, p)], [t.cuda() for t in (bd, bi, bp)]
    Cd, Ci, Cp = ops.spgemm_forward(m, n, *dA, n, b_cols, *dB)
    assert_same(Cp_ref, Cp, "C_indptr")
    assert_same(Ci_ref, Ci, "C_indices")
    assert_close(Cd_ref, Cd, "C_data", tol=1e-5 if d.dtype == torch.float32 else 1e-12)
    gC = torch.from_numpy(rng.standard_normal(Cd_ref.numel())).to(d.dtype)
    gA_ref, gB_ref = oracle.spgemm_backward(gC, Ci_ref, Cp_ref, m, n, d, i, p, n, b_cols, bd, bi, bp)
    gA, gB = ops.spgemm_backward(gC.cuda(), Ci, Cp, m, n, *dA, n, b_cols, *dB)
    assert_same(gA_ref, gA, "grad_A")
    assert_same(gB_ref, gB, "grad_B")


@settings(**SETTINGS)
@given(csr(), st.integers(1, 20))
def test_spdmm(oracle, A, K):
    ops = _ops()
    d, i, p, (m, n), seed = A
    g = torch.Generator().manual_seed(seed)
    B, G = torch.randn((n, K), generator=g, dtype=d.dtype), torch.randn((m, K), generator=g, dtype=d.dtype)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    assert_same(oracle.spdmm_forward(m, n, d, i, p, B), ops.spdmm_forward(m, n, dd, di, dp, B.cuda()), "C")
    gA_ref, gB_ref = oracle.spdmm_backward(m, n, d, i, p, B, G)
    gA, gB = ops.spdmm_backward(m, n, dd, di, dp, B.cuda(), G.cuda())
    assert_close(gA_ref, gA, "grad_A")
    assert_same(gB_ref, gB, "grad_B")
