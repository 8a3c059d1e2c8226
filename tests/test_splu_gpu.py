"""GPU parity of the sparse LU factorisation (fill pattern, factors, their transpose) and of the
differentiable direct solve built on it, against the CPU oracle: everything bit for bit, since the
elimination applies the reference's updates in the reference's order."""
import numpy as np
import pytest
import scipy.sparse as sps
import torch

from parity import assert_close, assert_same
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from numml_b200 import numml_torch_cpp
    yield numml_torch_cpp
    numml_torch_cpp.check_status()


def _csr(S, dtype):
    S = S.tocsr()
    S.sort_indices()
    return (torch.from_numpy(S.data.astype(np.float64)).to(dtype), torch.from_numpy(S.indices.astype(np.int64)),
            torch.from_numpy(S.indptr.astype(np.int64)), S.shape[0])


def _cases(dtype):
    out = {"random 60": _csr(sps.random(60, 60, density=0.08, random_state=3, format="csr") + sps.eye(60) * 4, dtype),
           "tridiagonal 300": _csr(sps.diags([-1, 2, -1], [-1, 0, 1], shape=(300, 300)), dtype),
           "diagonal 5": _csr(sps.eye(5) * 3, dtype),
           "random 700": _csr(sps.random(700, 700, density=0.004, random_state=5, format="csr") + sps.eye(700) * 6, dtype)}
    for g in (8, 24):
        d, i, p, (m, _) = W.poisson2d_5pt(g, dtype)
        out[f"poisson {g}x{g}"] = (d, i, p, m)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_factorisation_vs_oracle(oracle, ops, dtype):
    for name, (d, i, p, n) in _cases(dtype).items():
        ref = oracle.splu(n, n, d, i, p)
        got = ops.splu(n, n, d.cuda(), i.cuda(), p.cuda())
        for what, a, b in zip(("M data", "M indices", "M indptr", "Mt data", "Mt indices", "Mt indptr"), ref, got):
            assert_same(a, b, f"{name}: {what}")


def test_factors_reproduce_the_matrix(ops):
    d, i, p, (n, _) = W.poisson2d_5pt(40, torch.float64)
    M = ops.splu(n, n, d.cuda(), i.cuda(), p.cuda())
    Ms = sps.csr_matrix((M[0].cpu().numpy(), M[1].cpu().numpy(), M[2].cpu().numpy()), shape=(n, n))
    A = sps.csr_matrix((d.numpy(), i.numpy(), p.numpy()), shape=(n, n))
    L, U = sps.tril(Ms, -1) + sps.eye(n), sps.triu(Ms)
    assert abs(L @ U - A).max() < 1e-11
    assert M[0].numel() > 10 * d.numel() // 4            # the band fills in


def test_direct_solve_and_its_gradients(oracle, ops):
    import numml_b200.sparse as sp
    import numml_b200.sparse.linalg as spla
    d, i, p, n = _csr(sps.random(120, 120, density=0.05, random_state=9, format="csr") + sps.eye(120) * 5, torch.float64)
    A = sp.SparseCSRTensor((d, i, p), (n, n)).to("cuda")
    A.requires_grad = True
    b = W.randn(n, 1, torch.float64).cuda().requires_grad_(True)
    x = spla.spsolve(A, b)
    assert float(torch.linalg.norm(A.detach() @ x.detach() - b.detach()) / torch.linalg.norm(b.detach())) < 1e-12
    w = W.randn(n, 2, torch.float64).cuda()
    (x * w).sum().backward()
    M = oracle.splu(n, n, d, i, p)
    y = oracle.sptrsv_forward(n, n, M[0], M[1], M[2], True, True, b.detach().cpu())
    x_ref = oracle.sptrsv_forward(n, n, M[0], M[1], M[2], False, False, y)
    assert_same(x_ref, x.detach(), "x")
    gA_ref, gb_ref = oracle.spsolve_backward(w.cpu(), x_ref, n, n, M[3], M[4], M[5], d, i, p)
    assert_same(gb_ref, b.grad, "grad_b")
    assert_same(gA_ref, A.data.grad, "grad_A")
    # the factor object and the two-solve helper
    LU = spla.splu(A)
    assert_same(M[0], LU.data, "splu data")
    assert_same(x_ref, spla.splu_solve(LU, b.detach()), "splu_solve")


def test_missing_diagonal_is_refused(ops):
    d, i, p, n = _csr(sps.csr_matrix(np.array([[0.0, 1.0], [1.0, 2.0]])), torch.float64)
    with pytest.raises(RuntimeError, match="diagonal"):
        ops.splu(n, n, d.cuda(), i.cuda(), p.cuda())
