"""GPU parity of the hash SpGEMM (symbolic + numeric) and its masked backward: structure must be
bit-exact (sorted columns, cancelled entries kept), values within tolerance, gradients bit-exact."""
import pytest
import torch

from parity import assert_close, assert_same, case, case_names
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from numml_b200 import numml_torch_cpp
    return numml_torch_cpp


def run_case(ops, A, B, grad_C=None):
    (ad, ai, ap, (am, an)), (bd, bi, bp, (bm, bn)) = A, B
    dA = [t.cuda() for t in (ad, ai, ap)]
    dB = [t.cuda() for t in (bd, bi, bp)]
    Cd, Ci, Cp = ops.spgemm_forward(am, an, *dA, bm, bn, *dB)
    grads = None
    if grad_C is not None:
        grads = ops.spgemm_backward(grad_C.cuda(), Ci, Cp, am, an, *dA, bm, bn, *dB)
    return (Cd, Ci, Cp), grads


def test_golden_spgemm(golden_ops, ops):
    for name in case_names(golden_ops, "spgemm_"):
        c = case(golden_ops, name)
        A = (c["A_data"], c["A_indices"], c["A_indptr"], (int(c["A_shape"][0]), int(c["A_shape"][1])))
        B = (c["B_data"], c["B_indices"], c["B_indptr"], (int(c["B_shape"][0]), int(c["B_shape"][1])))
        (Cd, Ci, Cp), (gA, gB) = run_case(ops, A, B, c["grad_C"])
        assert_same(c["C_indptr"], Cp, name + " indptr")
        assert_same(c["C_indices"], Ci, name + " indices")
        assert_close(c["C_data"], Cd, name + " data") if c["C_data"].abs().sum() > 0 else assert_same(c["C_data"], Cd, name)
        assert_same(c["grad_A"], gA, name + " grad_A")
        assert_same(c["grad_B"], gB, name + " grad_B")


def test_cancelled_entry_is_kept(ops):
    one = (torch.tensor([1., 1.], dtype=torch.float64), torch.tensor([0, 1]), torch.tensor([0, 2]), (1, 2))
    col = (torch.tensor([1., -1.], dtype=torch.float64), torch.tensor([0, 0]), torch.tensor([0, 1, 2]), (2, 1))
    (Cd, Ci, Cp), _ = run_case(ops, one, col)
    assert Cp.tolist() == [0, 1] and Ci.tolist() == [0] and Cd.tolist() == [0.0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shapes,dens", [(((60, 50), (50, 70)), (0.1, 0.1)),      # small rows (8-lane bin)
                                          (((300, 400), (400, 500)), (0.04, 0.05)),  # 32-lane bin
                                          (((40, 600), (600, 3000)), (0.3, 0.05)),   # CTA bin
                                          (((6, 900), (900, 20000)), (0.9, 0.02)),   # global-memory spill bin
                                          (((1, 1), (1, 1)), (1.0, 1.0))])
def test_random_vs_oracle(oracle, ops, dtype, shapes, dens):
    (am, an), (bm, bn) = shapes
    A = W.random_csr(am, an, dens[0], seed=5, dtype=dtype)
    B = W.random_csr(bm, bn, dens[1], seed=6, dtype=dtype)
    Cd_ref, Ci_ref, Cp_ref = oracle.spgemm_forward(am, an, *A[:3], bm, bn, *B[:3])
    gC = W.randn(Cd_ref.numel(), 7, dtype)
    gA_ref, gB_ref = oracle.spgemm_backward(gC, Ci_ref, Cp_ref, am, an, *A[:3], bm, bn, *B[:3])
    (Cd, Ci, Cp), (gA, gB) = run_case(ops, A, B, gC)
    assert_same(Cp_ref, Cp, "C_indptr")
    assert_same(Ci_ref, Ci, "C_indices")
    assert_close(Cd_ref, Cd, "C_data")
    assert_same(gA_ref, gA, "grad_A")
    assert_same(gB_ref, gB, "grad_B")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_small_rows_are_bit_exact(oracle, ops, dtype):
    """Rows with at most 32 products (and at most 32 entries in the row of A) are formed by one warp
    in the reference's order of additions: values bit for bit, including duplicates-heavy rows, rows of
    A that select empty rows of B, rows with exactly 32 products, and rows just above the limit (which
    take the hash path and are compared at the tolerance)."""
    import numpy as np
    rng = np.random.default_rng(3)
    bm, bn = 500, 40                                     # few columns: many colliding products
    lens_b = rng.integers(0, 9, size=bm)
    lens_b[rng.choice(bm, 60, replace=False)] = 0        # empty rows of B
    b_ptr = np.concatenate(([0], np.cumsum(lens_b)))
    b_idx = np.concatenate([np.sort(rng.choice(bn, k, replace=False)) for k in lens_b] + [np.zeros(0, dtype=np.int64)])
    B = (torch.from_numpy(rng.standard_normal(len(b_idx))).to(dtype), torch.from_numpy(b_idx.astype(np.int64)),
         torch.from_numpy(b_ptr.astype(np.int64)), (bm, bn))
    am = 3000
    lens_a = rng.integers(0, 7, size=am)
    a_ptr = np.concatenate(([0], np.cumsum(lens_a)))
    a_idx = np.concatenate([np.sort(rng.choice(bm, k, replace=False)) for k in lens_a] + [np.zeros(0, dtype=np.int64)])
    A = (torch.from_numpy(rng.standard_normal(len(a_idx))).to(dtype), torch.from_numpy(a_idx.astype(np.int64)),
         torch.from_numpy(a_ptr.astype(np.int64)), (am, bm))
    products = np.array([lens_b[a_idx[a_ptr[r]:a_ptr[r + 1]]].sum() for r in range(am)])
    assert (products == 32).any() or (products > 32).any()
    Cd_ref, Ci_ref, Cp_ref = oracle.spgemm_forward(am, bm, *A[:3], bm, bn, *B[:3])
    (Cd, Ci, Cp), _ = run_case(ops, A, B)
    assert_same(Cp_ref, Cp, "C_indptr")
    assert_same(Ci_ref, Ci, "C_indices")
    assert_close(Cd_ref, Cd, "C_data")
    rows = torch.repeat_interleave(torch.arange(am), Cp_ref[1:] - Cp_ref[:-1])
    small = torch.from_numpy(products <= 32)[rows]
    assert int(small.sum()) > 0 and int((~small).sum()) > 0
    assert_same(Cd_ref[small], Cd.cpu()[small], "values of the rows formed by one warp")


def test_unsorted_right_factor_still_multiplies(oracle, ops):
    """The thread-per-row merge needs the rows of B sorted; with unsorted rows those rows of C are formed
    by the warp or hash kernels instead and the product is the same (structure exact, values at tolerance,
    as the order of additions within a column then follows B's storage order)."""
    import numpy as np
    A = W.random_csr(400, 300, 0.01, seed=41, dtype=torch.float64)
    bd, bi, bp, (bm, bn) = W.random_csr(300, 200, 0.03, seed=42, dtype=torch.float64)
    rng = np.random.default_rng(0)
    bd, bi = bd.clone(), bi.clone()
    for r in range(bm):                                   # reverse the entries of every second row
        if r % 2 == 0:
            a, b = int(bp[r]), int(bp[r + 1])
            bd[a:b], bi[a:b] = bd[a:b].flip(0), bi[a:b].flip(0)
    B = (bd, bi, bp, (bm, bn))
    ref = oracle.spgemm_forward(400, 300, *A[:3], bm, bn, bd, bi, bp)
    (Cd, Ci, Cp), _ = run_case(ops, A, B)
    assert_same(ref[2], Cp, "C_indptr")
    assert_same(ref[1], Ci, "C_indices")
    assert_close(ref[0], Cd, "C_data")


def test_empty_operands(ops):
    z = (torch.zeros(0, dtype=torch.float64), torch.zeros(0, dtype=torch.int64), torch.zeros(5, dtype=torch.int64), (4, 3))
    B = W.random_csr(3, 6, 0.5, seed=1, dtype=torch.float64, empty_rows=False)
    (Cd, Ci, Cp), (gA, gB) = run_case(ops, z, B, torch.zeros(0, dtype=torch.float64))
    assert Cd.numel() == 0 and Ci.numel() == 0 and Cp.tolist() == [0] * 5
    assert gA.numel() == 0 and torch.all(gB == 0)


def test_galerkin_product_vs_oracle(oracle, ops):
    """A*A and (P^T A) P on a 2-D Laplacian with 2x2 aggregation: the AMG products of the benchmark
    configuration, at a size the CPU oracle finishes quickly."""
    n = 48
    A = W.poisson2d_5pt(n, torch.float64)
    P = W.aggregation_2x2(n, torch.float64)
    am, an = A[3]
    pm, pn = P[3]
    # C = A A
    ref = oracle.spgemm_forward(am, an, *A[:3], am, an, *A[:3])
    assert ref[0].numel() == 13 * n * n - 20 * n + 4
    (Cd, Ci, Cp), _ = run_case(ops, A, A)
    assert_same(ref[2], Cp, "AA indptr"); assert_same(ref[1], Ci, "AA indices"); assert_same(ref[0], Cd, "AA data")
    # Pt = P^T, then (Pt A) P
    Pt_ref = oracle.csr_transpose_forward(pm, pn, *P[:3])
    Pt = (Pt_ref[0], Pt_ref[1], Pt_ref[2], (pn, pm))
    PtA_ref = oracle.spgemm_forward(pn, pm, *Pt[:3], am, an, *A[:3])
    PtA = (PtA_ref[0], PtA_ref[1], PtA_ref[2], (pn, an))
    Ac_ref = oracle.spgemm_forward(pn, an, *PtA[:3], pm, pn, *P[:3])
    (d1, i1, p1), _ = run_case(ops, Pt, A)
    assert_same(PtA_ref[2], p1, "PtA indptr"); assert_same(PtA_ref[1], i1, "PtA indices"); assert_close(PtA_ref[0], d1, "PtA data")
    gC = W.randn(Ac_ref[0].numel(), 3, torch.float64)
    (d2, i2, p2), (gA, gB) = run_case(ops, PtA, P, gC)
    assert_same(Ac_ref[2], p2, "Ac indptr"); assert_same(Ac_ref[1], i2, "Ac indices"); assert_close(Ac_ref[0], d2, "Ac data")
    gA_ref, gB_ref = oracle.spgemm_backward(gC, Ac_ref[1], Ac_ref[2], pn, an, *PtA[:3], pm, pn, *P[:3])
    assert_same(gA_ref, gA, "grad PtA"); assert_same(gB_ref, gB, "grad P")


def test_structure_properties_at_scale(ops):
    """Benchmark-scale A*A (2-D Laplacian, 1024^2 grid): nnz matches the closed form 13n^2-20n+4,
    every row is strictly ascending, and (A A) 1 == A (A 1)."""
    n = 1024
    A = W.poisson2d_5pt(n, torch.float64)
    m = n * n
    (Cd, Ci, Cp), _ = run_case(ops, A, A)
    assert int(Cp[-1]) == 13 * n * n - 20 * n + 4 == Ci.numel()
    rows = torch.repeat_interleave(torch.arange(m, device="cuda"), Cp[1:] - Cp[:-1])
    key = rows * m + Ci
    assert torch.all(key[1:] > key[:-1])
    ones = torch.ones(m, dtype=torch.float64, device="cuda")
    dA = [t.cuda() for t in A[:3]]
    lhs = ops.spgemv_forward(m, m, Cd, Ci, Cp, ones)
    rhs = ops.spgemv_forward(m, m, *dA, ops.spgemv_forward(m, m, *dA, ones))
    assert torch.allclose(lhs, rhs, atol=1e-12)


@pytest.mark.parametrize("case", ["stencil", "random"])
def test_kept_symbolic_phase_gives_the_same_product(oracle, ops, case):
    """A second product of the same two patterns with other values runs the numeric phase alone, on the row
    pointers and row lists kept from the first: same structure, values as the oracle's, and the same bits as with
    the keeping switched off.  The row pointers returned are a tensor of their own each time."""
    if case == "stencil":
        ad, ai, ap, (m, k) = W.poisson2d_5pt(96, torch.float64)
        bd, bi, bp, (_, n) = ad.clone(), ai, ap, (m, k)
    else:                                                   # long and short rows: hash bins and the spill path's header
        ad, ai, ap, (m, k) = W.random_csr(300, 400, 0.05, seed=3, dtype=torch.float64)
        bd, bi, bp, (_, n) = W.random_csr(400, 350, 0.08, seed=4, dtype=torch.float64)
    dA_idx, dA_ptr, dB_idx, dB_ptr = ai.cuda(), ap.cuda(), bi.cuda(), bp.cuda()
    assert ops.spgemm_keep_symbolic
    outs = []
    for rep, scale in enumerate((1.0, -0.75, 3.0, 0.5)):
        a, b = ad * scale, bd + scale
        ref = oracle.spgemm_forward(m, k, a, ai, ap, k, n, b, bi, bp)
        Cd, Ci, Cp = ops.spgemm_forward(m, k, a.cuda(), dA_idx, dA_ptr, k, n, b.cuda(), dB_idx, dB_ptr)
        assert_same(ref[2], Cp, "C_indptr")
        assert_same(ref[1], Ci, "C_indices")
        assert_close(ref[0], Cd, "C_data")
        outs.append((Cd, Ci, Cp))
        if rep > 0:                                         # kept from the second product of the pair on
            from numml_b200 import _plan
            kept = _plan.get_plan(m, k, dA_idx, dA_ptr).extra
            assert any(isinstance(key, tuple) and key[0] == "spgemm_symbolic" for key in kept)
            assert Cp.data_ptr() != outs[0][2].data_ptr()
    ops.spgemm_keep_symbolic = False
    try:
        a, b = ad * 0.5, bd + 0.5
        Cd, Ci, Cp = ops.spgemm_forward(m, k, a.cuda(), dA_idx, dA_ptr, k, n, b.cuda(), dB_idx, dB_ptr)
    finally:
        ops.spgemm_keep_symbolic = True
    if case == "stencil":                                   # register-merge rows: values reproducible bit for bit
        assert torch.equal(Cd, outs[3][0])
    assert torch.equal(Ci, outs[3][1]) and torch.equal(Cp, outs[3][2])
