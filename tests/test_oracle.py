"""CPU tests of the oracle itself: the plain-C restatement must reproduce, bit for bit, the
golden vectors that the reference produced, and (where the compiled reference module is
available) the reference on fresh seeded inputs."""
import pytest
import torch

from parity import assert_same, case, case_names
from numml_b200 import workloads as W


def _shape(c, key="shape"):
    return int(c[key][0]), int(c[key][1])


def test_golden_spmv(golden_ops, oracle):
    for name in case_names(golden_ops, "spmv_"):
        c = case(golden_ops, name)
        m, n = _shape(c)
        assert_same(c["y"], oracle.spgemv_forward(m, n, c["data"], c["indices"], c["indptr"], c["x"]), name)
        gA, gx = oracle.spgemv_backward(c["g"], m, n, c["data"], c["indices"], c["indptr"], c["x"])
        assert_same(c["grad_A"], gA, name)
        assert_same(c["grad_x"], gx, name)


def test_golden_spdmm(golden_ops, oracle):
    for name in case_names(golden_ops, "spdmm_"):
        c = case(golden_ops, name)
        m, n = _shape(c)
        assert_same(c["C"], oracle.spdmm_forward(m, n, c["data"], c["indices"], c["indptr"], c["B"]), name)
        gA, gB = oracle.spdmm_backward(m, n, c["data"], c["indices"], c["indptr"], c["B"], c["G"])
        assert_same(c["grad_A"], gA, name)
        assert_same(c["grad_B"], gB, name)


def test_golden_spgemm(golden_ops, oracle):
    for name in case_names(golden_ops, "spgemm_"):
        c = case(golden_ops, name)
        am, an = _shape(c, "A_shape")
        bm, bn = _shape(c, "B_shape")
        Cd, Ci, Cp = oracle.spgemm_forward(am, an, c["A_data"], c["A_indices"], c["A_indptr"],
                                           bm, bn, c["B_data"], c["B_indices"], c["B_indptr"])
        assert_same(c["C_indptr"], Cp, name)
        assert_same(c["C_indices"], Ci, name)
        assert_same(c["C_data"], Cd, name)
        gA, gB = oracle.spgemm_backward(c["grad_C"], Ci, Cp, am, an, c["A_data"], c["A_indices"], c["A_indptr"],
                                        bm, bn, c["B_data"], c["B_indices"], c["B_indptr"])
        assert_same(c["grad_A"], gA, name)
        assert_same(c["grad_B"], gB, name)


def test_golden_cancellation_is_kept(golden_ops):
    c = case(golden_ops, "spgemm_cancel_f64")
    assert c["C_indptr"].tolist() == [0, 1] and c["C_indices"].tolist() == [0] and c["C_data"].tolist() == [0.0]


def test_golden_transpose(golden_ops, oracle):
    for name in case_names(golden_ops, "transpose_"):
        c = case(golden_ops, name)
        m, n = _shape(c)
        td, ti, tp, perm = oracle.csr_transpose_forward(m, n, c["data"], c["indices"], c["indptr"])
        for k, v in (("t_data", td), ("t_indices", ti), ("t_indptr", tp), ("t_perm", perm)):
            assert_same(c[k], v, f"{name}/{k}")
        assert_same(c["grad_A"], oracle.csr_transpose_backward(c["grad_At"], perm), name)


def test_golden_sptrsv(golden_ops, oracle):
    names = case_names(golden_ops, "sptrsv_")
    assert len(names) == 8
    for name in names:
        c = case(golden_ops, name)
        m, n = _shape(c)
        lower, unit = bool(c["lower"]), bool(c["unit"])
        x = oracle.sptrsv_forward(m, n, c["data"], c["indices"], c["indptr"], lower, unit, c["b"])
        assert_same(c["x"], x, name)
        gA, gb = oracle.sptrsv_backward(c["grad_x"], x, m, n, c["data"], c["indices"], c["indptr"], lower, unit, c["b"])
        assert_same(c["grad_A"], gA, name)
        assert_same(c["grad_b"], gb, name)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_port_matches_compiled_reference(oracle, reference_module, dtype):
    R = reference_module
    if R is None:
        pytest.skip("oracle/_ref not built on this machine")
    d, i, p, (m, n) = W.random_csr(300, 220, 0.04, seed=101, dtype=dtype)
    x, g = W.randn(n, 0, dtype), W.randn(m, 1, dtype)
    assert_same(R.spgemv_forward(m, n, d, i, p, x), oracle.spgemv_forward(m, n, d, i, p, x))
    for a, b in zip(R.spgemv_backward(g, m, n, d, i, p, x), oracle.spgemv_backward(g, m, n, d, i, p, x)):
        assert_same(a, b)
    d2, i2, p2, (m2, n2) = W.random_csr(220, 180, 0.05, seed=102, dtype=dtype)
    C = R.spgemm_forward(m, n, d, i, p, m2, n2, d2, i2, p2)
    C2 = oracle.spgemm_forward(m, n, d, i, p, m2, n2, d2, i2, p2)
    for a, b in zip(C, C2):
        assert_same(a, b)
    gc = W.randn(C[0].numel(), 3, dtype)
    for a, b in zip(R.spgemm_backward(gc, C[1], C[2], m, n, d, i, p, m2, n2, d2, i2, p2),
                    oracle.spgemm_backward(gc, C[1], C[2], m, n, d, i, p, m2, n2, d2, i2, p2)):
        assert_same(a, b)
    for a, b in zip(R.csr_transpose_forward(m, n, d, i, p), oracle.csr_transpose_forward(m, n, d, i, p)):
        assert_same(a, b)
    B, G = W.randn((n, 7), 4, dtype), W.randn((m, 7), 5, dtype)
    assert_same(R.spdmm_forward(m, n, d, i, p, B), oracle.spdmm_forward(m, n, d, i, p, B))
    for a, b in zip(R.spdmm_backward(m, n, d, i, p, B, G), oracle.spdmm_backward(m, n, d, i, p, B, G)):
        assert_same(a, b)
    for lower in (True, False):
        for unit in (True, False):
            d, i, p, (m, n) = W.random_triangular(257, 0.03, lower=lower, seed=103, dtype=dtype)
            b, gx = W.randn(m, 6, dtype), W.randn(m, 7, dtype)
            x = R.sptrsv_forward(m, n, d, i, p, lower, unit, b)
            assert_same(x, oracle.sptrsv_forward(m, n, d, i, p, lower, unit, b))
            for a, bb in zip(R.sptrsv_backward(gx, x, m, n, d, i, p, lower, unit, b),
                             oracle.sptrsv_backward(gx, x, m, n, d, i, p, lower, unit, b)):
                assert_same(a, bb)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_pattern_operators_match_the_reference(oracle, reference_module, dtype):
    """Linear combination on the union pattern against the compiled reference (forward and backward),
    and tril / triu against a restatement of the reference's Python loops."""
    d, i, p, (m, n) = W.random_csr(200, 150, 0.05, seed=201, dtype=dtype)
    d2, i2, p2, _ = W.random_csr(200, 150, 0.07, seed=202, dtype=dtype)
    C = oracle.splincomb_forward(m, n, 1.5, d, i, p, -0.25, d2, i2, p2)
    gC = W.randn(C[0].numel(), 9, dtype)
    gA, gB = oracle.splincomb_backward(m, n, 1.5, d, i, p, -0.25, d2, i2, p2, gC, C[1], C[2])
    if reference_module is not None:
        a, b = torch.tensor(1.5, dtype=dtype), torch.tensor(-0.25, dtype=dtype)
        R = reference_module.splincomb_forward(m, n, a, d, i, p, b, d2, i2, p2)
        for u, v in zip(R, C):
            assert_same(u, v)
        Rg = reference_module.splincomb_backward(m, n, a, d, i, p, b, d2, i2, p2, gC, C[1], C[2])
        assert_same(Rg[0], gA)
        assert_same(Rg[1], gB)
    # the union pattern is sorted and holds every entry of both operands
    rows = torch.repeat_interleave(torch.arange(m), C[2][1:] - C[2][:-1])
    key = rows * n + C[1]
    assert torch.all(key[1:] > key[:-1])
    for k in (-2, 0, 3):
        for lower in (True, False):
            td, ti, tp, pos = oracle.triangle(m, d, i, p, k, lower)
            ld, li, lp = [], [], [0]                       # the reference's loops, entry by entry
            for r in range(m):
                for e in range(int(p[r]), int(p[r + 1])):
                    c = int(i[e])
                    if lower and c > r + k:
                        break
                    if not lower and c < r + k:
                        continue
                    ld.append(float(d[e])); li.append(c)
                lp.append(len(ld))
            assert ti.tolist() == li and tp.tolist() == lp
            assert_same(torch.tensor(ld, dtype=dtype), td)
            assert torch.equal(d[pos], td)


def test_sparse_lu_matches_the_reference(oracle, reference_module):
    """LU without pivoting (fill pattern, factors, their transposes) and the backward of the direct
    solve, bit for bit against the compiled reference, plus L U = A."""
    import numpy as np
    import scipy.sparse as sps
    cases = [sps.random(60, 60, density=0.08, random_state=3, format="csr") + sps.eye(60) * 4,
             sps.diags([-1, 2, -1], [-1, 0, 1], shape=(40, 40), format="csr")]
    pd, pi, pp, (m, k) = W.poisson2d_5pt(8, torch.float64)
    cases.append(sps.csr_matrix((pd.numpy(), pi.numpy(), pp.numpy()), shape=(m, k)))
    for S in cases:
        S = S.tocsr()
        S.sort_indices()
        n = S.shape[0]
        d = torch.from_numpy(S.data.astype(np.float64))
        i, p = torch.from_numpy(S.indices.astype(np.int64)), torch.from_numpy(S.indptr.astype(np.int64))
        mine = oracle.splu(n, n, d, i, p)
        M = sps.csr_matrix((mine[0].numpy(), mine[1].numpy(), mine[2].numpy()), shape=(n, n))
        L, U = sps.tril(M, -1) + sps.eye(n), sps.triu(M)
        assert abs(L @ U - S).max() < 1e-12
        x, gx = W.randn(n, 1, torch.float64), W.randn(n, 2, torch.float64)
        gmine = oracle.spsolve_backward(gx, x, n, n, mine[3], mine[4], mine[5], d, i, p)
        if reference_module is not None:
            for u, v in zip(reference_module.splu(n, n, d, i, p), mine):
                assert_same(u, v)
            ref = reference_module.spsolve_backward(gx, x, n, n, mine[3], mine[4], mine[5], d, i, p)
            assert_same(ref[0], gmine[0])
            assert_same(ref[1], gmine[1])


def test_workload_sizes():
    assert W.poisson2d_5pt(256)[0].numel() == 326656
    assert W.poisson3d_7pt(16)[0].numel() == 7 * 16 ** 3 - 6 * 16 ** 2
    assert W.poisson2d_9pt_lower(64)[0].numel() == 5 * 64 * 64 - 6 * 64 + 2
    d, i, p, s = W.aggregation_2x2(8)
    assert s == (64, 16) and d.numel() == 64
    d, i, p, s = W.powerlaw_graph(1 << 12)
    assert int(p[-1]) == d.numel() and torch.all(p[1:] > p[:-1])  # every node has at least one edge
    row_sums = torch.zeros(s[0], dtype=torch.float64).index_add_(
        0, torch.repeat_interleave(torch.arange(s[0]), p[1:] - p[:-1]), d.double())
    assert torch.allclose(row_sums, torch.ones_like(row_sums), atol=1e-5)
