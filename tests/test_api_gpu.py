"""API-level GPU tests through SparseCSRTensor and its autograd Functions, mirroring the
reference's own test modules (numml/tests/test_spmv.py, test_spdmm.py, test_spmm.py,
test_sptrsv.py, test_transpose.py) with the reference's tolerances, plus the golden vectors that
the reference's Python package produced (conjugate gradients, Galerkin product with autograd)."""
import pytest
import torch
import torch.linalg as tla

from parity import assert_close, assert_same
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu
gpu = torch.device("cuda:0")


@pytest.fixture(scope="module")
def sp():
    import numml_b200.sparse as sp
    return sp


def tridiag(sp, n, dtype=torch.float32):
    return (sp.eye(n, dtype=dtype) * 2 - sp.eye(n, k=-1, dtype=dtype) - sp.eye(n, k=1, dtype=dtype))


def relerr(x, xhat):
    return (tla.norm(x - xhat) / tla.norm(x)).item()


# ---- SpMV (reference numml/tests/test_spmv.py) ---------------------------------------------------
def test_spmv_zeros_and_unit_vectors(sp):
    n = 16
    A = tridiag(sp, n)
    A_c = A.to(gpu)
    assert torch.all((A_c @ torch.zeros(n, device=gpu)) == 0)
    for i in range(n):
        e = torch.zeros(n, device=gpu)
        e[i] = 1.
        Ae = A_c @ e
        assert Ae[i] == 2
        if i > 0:
            assert Ae[i - 1] == -1
        if i < n - 1:
            assert Ae[i + 1] == -1


@pytest.mark.parametrize("n,tol", [(16, 1e-6), (2048, 1e-7)])
def test_spmv_random(sp, n, tol):
    A = tridiag(sp, n)
    A_d = A.to_dense()
    A_c = A.to(gpu)
    for _ in range(20):
        b = torch.rand(n)
        assert relerr(A_d @ b, (A_c @ b.to(gpu)).cpu()) < tol


def test_spmv_backward(sp):
    n = 2048
    A = tridiag(sp, n)
    for _ in range(3):
        w, x = torch.rand(n), torch.rand(n)
        Ag = A.to(gpu).copy()
        Ag.requires_grad = True
        xg = x.to(gpu).requires_grad_(True)
        ((Ag @ xg) * w.to(gpu)).sum().backward()
        rows = torch.repeat_interleave(torch.arange(n), A.indptr[1:] - A.indptr[:-1])
        assert torch.allclose(Ag.data.grad.cpu(), w[rows] * x[A.indices], rtol=1e-7, atol=0)
        assert relerr(A.to_dense().T @ w, xg.grad.cpu()) < 1e-6


def test_spmv_keeps_singleton_shape_and_rejects_mismatch(sp):
    A = tridiag(sp, 8).to(gpu)
    y = A @ torch.ones((8, 1), device=gpu)
    assert y.shape == (8, 1)
    with pytest.raises(RuntimeError, match="same data type"):
        A @ torch.ones(8, dtype=torch.float64, device=gpu)
    with pytest.raises(RuntimeError, match="Number of columns"):
        A @ torch.ones(9, device=gpu)


# ---- SpMM (reference numml/tests/test_spdmm.py) --------------------------------------------------
def test_spdmm_forward_backward(sp):
    n, k = 512, 24
    A = tridiag(sp, n)
    A_d = A.to_dense()
    B = torch.randn(n, k)
    Ag = A.to(gpu).copy()
    Ag.requires_grad = True
    Bg = B.to(gpu).requires_grad_(True)
    C = Ag @ Bg
    assert torch.allclose(C.cpu(), A_d @ B, atol=1e-5)
    C.sum().backward()
    mask = A_d != 0
    gA_dense = (torch.ones(n, k) @ B.T) * mask
    assert torch.allclose(Ag.grad.to_dense().cpu(), gA_dense, atol=1e-4)
    assert torch.allclose(Bg.grad.cpu(), A_d.T @ torch.ones(n, k), atol=1e-5)


def test_batched_spdmm(sp):
    A = tridiag(sp, 32).to(gpu)
    X = torch.randn(3, 5, 32, 7, device=gpu)
    Y = A @ X
    assert Y.shape == X.shape
    assert torch.allclose(Y, torch.matmul(A.to_dense(), X), atol=1e-5)


# ---- SpGEMM (reference numml/tests/test_spmm.py) ---------------------------------------------------
@pytest.mark.parametrize("n", [16, 2048])
def test_matmat(sp, n):
    A = tridiag(sp, n)
    B = (-A).copy()
    C_c = A.to(gpu) @ B.to(gpu)
    assert torch.allclose(A.to_dense() @ B.to_dense(), C_c.to_dense().cpu())


def skinny_P(sp, n=16, blocks=4):
    P_d = torch.zeros((n, blocks))
    for i in range(blocks):
        P_d[i * (n // blocks):(i + 1) * (n // blocks), i] = 1.
    return P_d, sp.SparseCSRTensor(P_d)


def test_galerkin_skinny_with_grads(sp):
    import numml_b200.utils as utils
    A = tridiag(sp, 16)
    P_d, P = skinny_P(sp)
    A_c, P_c = A.to(gpu).copy(), P.to(gpu).copy()
    A_c.requires_grad = True
    P_c.requires_grad = True
    AH = P_c.T @ A_c @ P_c
    assert torch.allclose(AH.to_dense().cpu(), P_d.T @ A.to_dense() @ P_d)
    AH.sum().backward()

    def f_A(M):
        return (P.to(gpu).T @ M @ P.to(gpu)).sum()

    def f_P(M):
        return (M.T @ A.to(gpu) @ M).sum()

    fdA = utils.sp_fd(f_A, A.to(gpu))
    fdP = utils.sp_fd(f_P, P.to(gpu))
    assert relerr(fdA.data, A_c.grad.data) < 1e-3
    assert relerr(fdP.data, P_c.grad.data) < 1e-3


def test_spgemm_analytic_grads(sp):
    n = 256
    A = tridiag(sp, n)
    B = (-A).copy()
    Ag, Bg = A.to(gpu).copy(), B.to(gpu).copy()
    Ag.requires_grad = True
    Bg.requires_grad = True
    C = Ag @ Bg
    C.sum().backward()
    gC = sp.SparseCSRTensor((torch.ones_like(C.data), C.indices, C.indptr), C.shape).to_dense().cpu()
    maskA, maskB = A.to_dense() != 0, B.to_dense() != 0
    assert torch.allclose((gC @ B.to_dense().T) * maskA, Ag.grad.to_dense().cpu())
    assert torch.allclose((A.to_dense().T @ gC) * maskB, Bg.grad.to_dense().cpu())


# ---- transpose (reference numml/tests/test_transpose.py) ----------------------------------------
@pytest.mark.parametrize("shape", [(512, 64), (64, 512)])
def test_transpose_random_with_grad(sp, shape):
    A_d = torch.zeros(shape)
    nnz = (shape[0] * shape[1]) // 2
    A_d[torch.randint(shape[0], (nnz,)), torch.randint(shape[1], (nnz,))] = torch.randn(nnz)
    A = sp.SparseCSRTensor(A_d).to(gpu)
    A.requires_grad = True
    At = A.T
    assert torch.allclose(At.to_dense().cpu(), A_d.T)
    w = torch.randn(A.nnz, device=gpu)
    (At.data * w).sum().backward()
    # d/dA of sum(w * At.data) is w scattered back through the permutation
    ref = sp.SparseCSRTensor((w, At.indices, At.indptr), At.shape).to_dense().T
    assert torch.allclose(A.grad.to_dense(), ref)


# ---- triangular solve (reference numml/tests/test_sptrsv.py) ------------------------------------
def test_solve_triangular_identity_and_bidiagonal(sp):
    n = 32
    I_c = sp.eye(n).to(gpu)
    x = torch.randn(n, device=gpu)
    for upper in (False, True):
        for unit in (False, True):
            assert torch.allclose(I_c.solve_triangular(upper, unit, x), x)
    A = (sp.eye(n) * 2 - sp.eye(n, k=-1)).to(gpu)
    b = A @ torch.randn(n, device=gpu)
    xs = A.solve_triangular(False, False, b)
    assert relerr(b, A @ xs) < 1e-5
    U = (sp.eye(n) - sp.eye(n, k=1) * 2).to(gpu)
    b = U @ torch.randn(n, device=gpu)
    xs = U.solve_triangular(True, True, b)
    assert relerr(b, U @ xs) < 1e-5


def test_solve_triangular_grads_vs_finite_differences(sp):
    import numml_b200.utils as utils
    import numml_b200.sparse.linalg as spla
    n = 24
    A = (sp.eye(n, dtype=torch.float64) * 2 - sp.eye(n, k=-1, dtype=torch.float64)).to(gpu)
    b = (A @ torch.randn(n, dtype=torch.float64, device=gpu)).detach()
    Ag = A.copy()
    Ag.requires_grad = True
    bg = b.clone().requires_grad_(True)
    spla.spsolve_triangular(Ag, bg, lower=True).sum().backward()
    fdA = utils.fd(lambda M: M.solve_triangular(False, False, b).sum(), A, h=1e-6)
    fdb = utils.fd(lambda v: A.solve_triangular(False, False, v).sum(), b, h=1e-6)
    assert relerr(fdA.data, Ag.data.grad) < 1e-3
    assert relerr(fdb, bg.grad) < 1e-3


def test_random_lower_fp64_like_reference(sp):
    for seed in range(3):
        n = int(torch.randint(32, 2048, (1,)).item())
        d, i, p, shape = W.random_triangular(n, 0.05, lower=True, seed=seed, dtype=torch.float64)
        A = sp.SparseCSRTensor((d, i, p), shape).to(gpu)
        b = torch.randn(n, dtype=torch.float64, device=gpu)
        x = A.solve_triangular(False, False, b)
        assert relerr(b, A @ x) < 1e-5


# ---- golden vectors produced by the reference's Python package ----------------------------------
def test_golden_conjugate_gradient(sp, golden_api):
    import numml_b200.krylov as kry
    n = int(golden_api["cg_poisson3d/n"])
    d, i, p, shape = W.poisson3d_7pt(n, torch.float64)
    A = sp.SparseCSRTensor((d, i, p), shape).to(gpu)
    b = torch.from_numpy(golden_api["cg_poisson3d/b"]).to(gpu)
    x, hist = kry.conjugate_gradient(A, b, rtol=0.0, iterations=25)
    # per-operation parity is 1e-12; the 25-step Krylov recurrence amplifies rounding differences
    # of the dot products (torch reductions differ between CPU and GPU), so the trajectory is
    # compared at 1e-8
    assert_close(torch.from_numpy(golden_api["cg_poisson3d/x"]), x, "CG solution", tol=1e-8)
    assert_close(torch.from_numpy(golden_api["cg_poisson3d/res_hist"]), hist, "CG residual history", tol=1e-8)
    assert hist.numel() == 26


def test_golden_galerkin_autograd(sp, golden_api):
    n = int(golden_api["galerkin/n"])
    ad, ai, ap, ashape = W.poisson2d_5pt(n, torch.float64)
    pd, pi, pp, pshape = W.aggregation_2x2(n, torch.float64)
    A = sp.SparseCSRTensor((ad, ai, ap), ashape).to(gpu)
    P = sp.SparseCSRTensor((pd, pi, pp), pshape).to(gpu)
    A.requires_grad = True
    P.requires_grad = True
    AH = P.T @ A @ P
    w = torch.from_numpy(golden_api["galerkin/w"]).to(gpu)
    (AH.data * w).sum().backward()
    assert_same(torch.from_numpy(golden_api["galerkin/AH_indptr"]), AH.indptr, "indptr")
    assert_same(torch.from_numpy(golden_api["galerkin/AH_indices"]), AH.indices, "indices")
    assert_close(torch.from_numpy(golden_api["galerkin/AH_data"]), AH.data, "data")
    assert_close(torch.from_numpy(golden_api["galerkin/grad_A"]), A.data.grad, "grad_A")
    assert_close(torch.from_numpy(golden_api["galerkin/grad_P"]), P.data.grad, "grad_P")


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-9), (torch.float32, 2e-3)])
@pytest.mark.parametrize("with_x0", [False, True])
def test_library_cg_loop_vs_oracle(sp, oracle, dtype, tol, with_x0):
    """The in-library CG loop (one SpMV + three fused vector kernels per iteration, scalars on the
    device) against the same recurrence evaluated on CPU with the oracle SpMV."""
    import numml_b200.krylov as kry
    d, i, p, (m, n) = W.poisson3d_7pt(12, dtype)
    b = W.randn(m, 3, dtype)
    x0 = W.randn(m, 4, dtype) * 0.1 if with_x0 else None
    iters = 20
    x = torch.zeros(m, dtype=dtype) if x0 is None else x0.clone()
    r = b.clone() if x0 is None else b - oracle.spgemv_forward(m, n, d, i, p, x0)
    pv, rz = r.clone(), r @ r
    hist = [rz.sqrt()]
    for _ in range(iters):
        Ap = oracle.spgemv_forward(m, n, d, i, p, pv)
        alpha = rz / (Ap @ pv)
        x = x + alpha * pv
        r = r - alpha * Ap
        rz_new = r @ r
        pv = r + (rz_new / rz) * pv
        rz = rz_new
        hist.append(rz.sqrt())
    A = sp.SparseCSRTensor((d, i, p), (m, n)).to(gpu)
    xg, hg = kry.conjugate_gradient(A, b.to(gpu), x=None if x0 is None else x0.to(gpu), rtol=0.0, iterations=iters)
    assert hg.numel() == iters + 1
    assert_close(x, xg, "x", tol=tol)
    assert_close(torch.stack(hist), hg, "residual history", tol=tol)
    # the differentiable torch-op loop (taken when gradients are requested) agrees with it
    Ag = A.copy()
    Ag.requires_grad = True
    xt, ht = kry.conjugate_gradient(Ag, b.to(gpu), x=None if x0 is None else x0.to(gpu), rtol=0.0, iterations=iters)
    assert_close(xg, xt.detach(), "x (torch-op loop)", tol=tol)
    assert xt.requires_grad


def test_cg_exact_convergence_stops_like_the_reference(sp):
    """With rtol = 0 the reference's loop still ends when the residual reaches exactly zero.  On the
    identity CG converges in one step; the remaining iterations must not turn x into NaN, and the
    history must end at its first zero."""
    import numml_b200.krylov as kry
    n = 300
    A = sp.eye(n, dtype=torch.float64).to(gpu)
    b = W.randn(n, 5, torch.float64).to(gpu)
    x, hist = kry.conjugate_gradient(A, b, rtol=0.0, iterations=6)
    assert_same(b, x, "x")
    assert hist.numel() == 2 and float(hist[1]) == 0.0 and float(hist[0]) > 0
    Ag = A.copy()
    Ag.requires_grad = True                      # the torch-op loop
    x2, hist2 = kry.conjugate_gradient(Ag, b, rtol=0.0, iterations=6)
    assert_same(b, x2.detach(), "x (torch-op loop)")
    assert hist2.numel() == 2


def test_conjugate_residual_vs_cpu_recurrence(sp, oracle):
    """Conjugate residuals on a symmetric indefinite matrix (a shifted Laplacian), against the same
    recurrence (reference numml/krylov.py:40-80) evaluated on the CPU with the oracle SpMV."""
    import numml_b200.krylov as kry
    d, i, p, (m, n) = W.poisson3d_7pt(10, torch.float64)
    rows = torch.repeat_interleave(torch.arange(m), p[1:] - p[:-1])
    d = d - 2.5 * (rows == i).double()           # eigenvalues on both sides of zero
    b = W.randn(m, 6, torch.float64)
    mv = lambda v: oracle.spgemv_forward(m, n, d, i, p, v)  # noqa: E731
    iters = 30
    x, r = torch.zeros(m, dtype=torch.float64), b.clone()
    pv, Ar = r.clone(), mv(r)
    Ap, hist = Ar.clone(), [tla.norm(r)]
    for _ in range(iters):
        alpha = (r @ Ar) / (Ap @ Ap)
        x = x + alpha * pv
        r_new = r - alpha * Ap
        Ar_new = mv(r_new)
        beta = (r_new @ Ar_new) / (r @ Ar)
        pv = r_new + beta * pv
        Ap = Ar_new + beta * Ap
        Ar, r = Ar_new, r_new
        hist.append(tla.norm(r))
    A = sp.SparseCSRTensor((d, i, p), (m, n)).to(gpu)
    xg, hg = kry.conjugate_residual(A, b.to(gpu), rtol=0.0, iterations=iters)
    assert isinstance(hg, list) and len(hg) == iters + 1
    assert_close(x, xg, "x", tol=1e-8)
    assert_close(torch.stack(hist), torch.stack(hg), "residual history", tol=1e-8)
    # with a preconditioner (a LinearOperator, as in the reference) the loop runs and reduces the residual
    M = sp.LinearOperator((m, n), rm=lambda v: v / 4.0, lm=lambda v: v / 4.0)
    _, hp = kry.conjugate_residual(A, b.to(gpu), M=M, rtol=1e-3, iterations=200)
    assert float(hp[-1]) < float(hp[0])


# ---------------------------------------------------------------------------------------------
# Malformed structure raises instead of reading out of bounds or answering wrongly
# ---------------------------------------------------------------------------------------------
def _flags(rows, cols, indices, indptr):
    import ctypes
    from numml_b200 import _cabi
    i, p = torch.tensor(indices, dtype=torch.int64).cuda(), torch.tensor(indptr, dtype=torch.int64).cuda()
    out = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    _cabi.call("nb200_csr_check", rows, cols, i.numel(), P(i), P(p), _cabi.I64, P(out),
               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return int(out.item())


def test_structure_check_flags():
    assert _flags(3, 3, [0, 0, 1, 2], [0, 1, 3, 4]) == 0                 # lower bidiagonal: clean
    assert _flags(3, 3, [0, 1, 0, 2], [0, 1, 3, 4]) == 4                 # row 1 descending
    assert _flags(3, 3, [0, 1, 1, 2], [0, 1, 3, 4]) == 4                 # duplicate column
    assert _flags(3, 3, [0, 0, 2], [0, 1, 2, 3]) == 8                    # row 1 has no diagonal
    assert _flags(3, 3, [0, 1, 3], [0, 1, 2, 3]) == 2 | 8                # column 3 of a 3-column matrix
    assert _flags(3, 3, [0, 1, 2], [0, 1, 2, 2]) & 1                     # indptr ends before nnz
    assert _flags(3, 3, [0, 1, 2], [0, 2, 1, 3]) & 1                     # indptr decreases
    assert _flags(2, 4, [3, 0], [0, 1, 2]) == 8                          # rectangular: rows 0, 1 lack (r, r)
    assert _flags(0, 0, [], [0]) == 0


def test_malformed_matrices_raise():
    import numml_b200.numml_torch_cpp as ops
    d = torch.ones(4, dtype=torch.float64).cuda()
    x = torch.ones(3, dtype=torch.float64).cuda()
    L = lambda idx, ptr: (torch.tensor(idx).cuda(), torch.tensor(ptr).cuda())  # noqa: E731
    i, p = L([0, 1, 0, 2], [0, 1, 3, 4])                                 # unsorted row
    ops.spgemv_forward(3, 3, d, i, p, x)                                 # a product does not care
    with pytest.raises(RuntimeError, match="strictly ascending"):
        ops.sptrsv_forward(3, 3, d, i, p, True, False, x)
    i, p = L([0, 0, 2], [0, 1, 2, 3])                                    # no diagonal in row 1
    with pytest.raises(RuntimeError, match="diagonal"):
        ops.sptrsv_forward(3, 3, d[:3], i, p, True, False, x)
    y = ops.sptrsv_forward(3, 3, d[:3], i, p, True, True, x)             # unit diagonal: nothing stored is needed
    assert torch.equal(y.cpu(), torch.tensor([1., 0., 1.], dtype=torch.float64))
    i, p = L([0, 1, 3], [0, 1, 2, 3])                                    # column out of range
    with pytest.raises(RuntimeError, match="outside"):
        ops.spgemv_forward(3, 3, d[:3], i, p, x)
    i, p = L([0, 1, 2], [0, 1, 2, 2])                                    # indptr does not reach nnz
    with pytest.raises(RuntimeError, match="indptr"):
        ops.spgemv_forward(3, 3, d[:3], i, p, x)
    ops.check_status()
