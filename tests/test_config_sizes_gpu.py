"""Parity with the CPU oracle at the sizes the benchmark configurations are quoted on.

Every case runs the operator functions (which sit directly on the C ABI) on the full-size input
and compares with the oracle on the same seeded input.  At these sizes a persistent CTA of the
pipelined SpMV kernels walks several row blocks (stage reuse, barrier phase flips, the producer
running ahead), the SpGEMM bins hold millions of rows, and the triangular solve crosses thousands of
dependency levels -- regimes the small cases never reach.

Tolerances: index arrays and every sum taken in the reference's order must match bit for bit;
warp-reduced or atomically accumulated values are compared norm-wise at 1e-12 (fp64) / 1e-5 (fp32);
the 100-step CG trajectory at 1e-8 (its dot products are reduced block-wise on the device, in another
order than on the CPU, and the recurrence amplifies the difference).
"""
import numpy as np
import pytest
import torch

from parity import assert_close, assert_same
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["auto", "stream"])
def spmv_ops(request):
    from numml_b200 import numml_torch_cpp
    old = numml_torch_cpp.spmv_kernel
    numml_torch_cpp.spmv_kernel = request.param
    yield numml_torch_cpp
    numml_torch_cpp.spmv_kernel = old
    numml_torch_cpp.check_status()


@pytest.fixture(scope="module")
def ops():
    from numml_b200 import numml_torch_cpp
    yield numml_torch_cpp
    numml_torch_cpp.check_status()


def cuda(*ts):
    return [t.cuda() for t in ts]


# ---- configuration 1: 2-D Poisson 256^2, fp32 ------------------------------------------------------
def test_c1_poisson2d_256_fp32_spmv(oracle, spmv_ops):
    d, i, p, (m, k) = W.poisson2d_5pt(256, torch.float32)
    assert (m, d.numel()) == (65536, 326656)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(k, generator=gen, dtype=torch.float32)
    g = torch.randn(m, generator=gen, dtype=torch.float32)
    dd, di, dp, dx, dg = cuda(d, i, p, x, g)
    assert_same(oracle.spgemv_forward(m, k, d, i, p, x), spmv_ops.spgemv_forward(m, k, dd, di, dp, dx), "y")
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, d, i, p, x)
    for call in range(2):                  # the second call may take the value-symmetric pass
        gA, gx = spmv_ops.spgemv_backward(dg, m, k, dd, di, dp, dx)
        assert_same(gA_ref, gA, f"grad_A (call {call})")
        assert_same(gx_ref, gx, f"grad_x (call {call})")


# ---- configuration 2: 3-D Poisson 128^3, fp64 ------------------------------------------------------
@pytest.fixture(scope="module")
def poisson128():
    d, i, p, (m, k) = W.poisson3d_7pt(128, torch.float64)
    assert (m, d.numel()) == (2097152, 14581760)
    return d, i, p, m, k


@pytest.mark.parametrize("values", ["laplacian", "random"])
def test_c2_poisson3d_128_fp64_spmv(oracle, spmv_ops, poisson128, values):
    """Forward and backward, bit for bit, with the Laplacian's values (symmetric: the second backward
    call runs the value-symmetric pass) and with random values on the same pattern (A[i,j] != A[j,i]:
    a backward that confused an entry with its mirror image would be caught)."""
    d, i, p, m, k = poisson128
    if values == "random":
        d = W.randn(d.numel(), 11, torch.float64)
    x, g = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
    dd, di, dp, dx, dg = cuda(d, i, p, x, g)
    assert_same(oracle.spgemv_forward(m, k, d, i, p, x), spmv_ops.spgemv_forward(m, k, dd, di, dp, dx), "y")
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, d, i, p, x)
    for call in range(3):
        gA, gx = spmv_ops.spgemv_backward(dg, m, k, dd, di, dp, dx)
        assert_same(gA_ref, gA, f"grad_A (call {call})")
        assert_same(gx_ref, gx, f"grad_x (call {call})")
    if spmv_ops.spmv_kernel == "auto":
        assert spmv_ops.values_symmetric_state(m, k, di, dp) is (values == "laplacian")


def test_c2_cg_100_iterations(oracle, ops, poisson128):
    """100 unpreconditioned CG iterations (b ~ N(0,1), x0 = 0, rtol = 0) through the public solver,
    against the reference's recurrence (numml/krylov.py:135-153) evaluated on the CPU in float64 with
    the oracle SpMV: the 101 residual norms and the final iterate, at 1e-8."""
    import numml_b200.sparse as sp
    import numml_b200.krylov as kry
    d, i, p, m, k = poisson128
    b = W.randn(m, 2, torch.float64)
    x = torch.zeros(m, dtype=torch.float64)
    r = b.clone()
    pvec = r.clone()
    rz = torch.dot(r, r)
    hist = [torch.sqrt(rz)]
    for _ in range(100):
        Ap = oracle.spgemv_forward(m, k, d, i, p, pvec)
        alpha = rz / torch.dot(Ap, pvec)
        x += alpha * pvec
        r -= alpha * Ap
        rz_new = torch.dot(r, r)
        pvec = r + (rz_new / rz) * pvec
        rz = rz_new
        hist.append(torch.sqrt(rz))
    hist = torch.stack(hist)
    A = sp.SparseCSRTensor((d, i, p), (m, k), clone=False).to("cuda")
    x_gpu, hist_gpu = kry.conjugate_gradient(A, b.cuda(), rtol=0.0, iterations=100)
    assert hist_gpu.numel() == 101
    assert_close(hist, hist_gpu, "residual history", tol=1e-8)
    assert_close(x, x_gpu, "iterate after 100 steps", tol=1e-8)
    assert float(torch.max(torch.abs(hist_gpu.cpu() - hist) / hist)) < 1e-8   # entry by entry, not only norm-wise


# ---- configuration 4: Galerkin products on the 2048^2 grid, fp64 -----------------------------------
def _spgemm(ops, A, B):
    (ad, ai, ap, (am, an)), (bd, bi, bp, (bm, bn)) = A, B
    return ops.spgemm_forward(am, an, ad, ai, ap, bm, bn, bd, bi, bp)


def test_c4_galerkin_2048_fp64(oracle, ops):
    n = 2048
    A = W.poisson2d_5pt(n, torch.float64)
    P = W.aggregation_2x2(n, torch.float64)
    (ad, ai, ap, (am, an)), (pd, pi, pp, (pm, pn)) = A, P
    assert (am, ad.numel()) == (4194304, 20963328)
    dA = tuple(cuda(ad, ai, ap)) + ((am, an),)
    dP = tuple(cuda(pd, pi, pp)) + ((pm, pn),)

    # C = A A: structure and values bit-exact
    ref = oracle.spgemm_forward(am, an, ad, ai, ap, am, an, ad, ai, ap)
    assert ref[0].numel() == 54484996
    Cd, Ci, Cp = _spgemm(ops, dA, dA)
    assert_same(ref[2], Cp, "A A indptr")
    assert_same(ref[1], Ci, "A A indices")
    assert_same(ref[0], Cd, "A A values")            # rows of 25 products: one warp each, reference order
    # backward of C = A A with an upstream gradient on C's values
    gC = W.randn(ref[0].numel(), 0, torch.float64)
    gA_ref, gB_ref = oracle.spgemm_backward(gC, ref[1], ref[2], am, an, ad, ai, ap, am, an, ad, ai, ap)
    gA, gB = ops.spgemm_backward(gC.cuda(), Ci, Cp, am, an, *dA[:3], am, an, *dA[:3])
    assert_same(gA_ref, gA, "grad of the left factor")
    assert_same(gB_ref, gB, "grad of the right factor")
    del Cd, Ci, Cp, gA, gB, gC, ref, gA_ref, gB_ref

    # Ac = (P^T A) P, left to right as the reference evaluates it
    Pt_ref = oracle.csr_transpose_forward(pm, pn, pd, pi, pp)
    Pt = ops.csr_transpose_forward(pm, pn, *dP[:3])
    assert_same(Pt_ref[2], Pt[2], "P^T indptr")
    assert_same(Pt_ref[1], Pt[1], "P^T indices")
    assert_same(Pt_ref[3], Pt[3], "P^T permutation")
    dPt = (Pt[0], Pt[1], Pt[2], (pn, pm))
    PtA_ref = oracle.spgemm_forward(pn, pm, Pt_ref[0], Pt_ref[1], Pt_ref[2], am, an, ad, ai, ap)
    assert PtA_ref[0].numel() == 12574720
    PtA = _spgemm(ops, dPt, dA)
    assert_same(PtA_ref[2], PtA[2], "P^T A indptr")
    assert_same(PtA_ref[1], PtA[1], "P^T A indices")
    assert_same(PtA_ref[0], PtA[0], "P^T A values")
    Ac_ref = oracle.spgemm_forward(pn, an, PtA_ref[0], PtA_ref[1], PtA_ref[2], pm, pn, pd, pi, pp)
    assert Ac_ref[0].numel() == 5238784
    dPtA = (PtA[0], PtA[1], PtA[2], (pn, an))
    Ac = _spgemm(ops, dPtA, dP)
    assert_same(Ac_ref[2], Ac[2], "Ac indptr")
    assert_same(Ac_ref[1], Ac[1], "Ac indices")
    assert_same(Ac_ref[0], Ac[0], "Ac values")
    gAc = W.randn(Ac_ref[0].numel(), 0, torch.float64)
    g1_ref, g2_ref = oracle.spgemm_backward(gAc, Ac_ref[1], Ac_ref[2], pn, an, PtA_ref[0], PtA_ref[1], PtA_ref[2],
                                            pm, pn, pd, pi, pp)
    g1, g2 = ops.spgemm_backward(gAc.cuda(), Ac[1], Ac[2], pn, an, PtA[0], PtA[1], PtA[2], pm, pn, *dP[:3])
    assert_same(g1_ref, g1, "grad of P^T A")
    assert_same(g2_ref, g2, "grad of P")


# ---- configuration 5: lower factor of the 9-point Laplacian on 1024^2, 16 right-hand sides ---------
def test_c5_sptrsv_1024_16rhs(oracle, ops):
    d, i, p, (n, _) = W.poisson2d_9pt_lower(1024, torch.float64)
    assert (n, d.numel()) == (1048576, 5236738)
    B = W.randn((n, 16), 0, torch.float64)
    G = W.randn((n, 16), 1, torch.float64)
    dd, di, dp = cuda(d, i, p)
    X = ops.sptrsv_forward(n, n, dd, di, dp, True, False, B.cuda())
    X_ref = torch.stack([oracle.sptrsv_forward(n, n, d, i, p, True, False, B[:, c].contiguous()) for c in range(16)], 1)
    assert_same(X_ref, X, "all 16 solution columns")
    gL, gB = ops.sptrsv_backward(G.cuda(), X, n, n, dd, di, dp, True, False, B.cuda())
    gL_ref = torch.zeros_like(d)
    for c in range(16):
        gl, gb = oracle.sptrsv_backward(G[:, c].contiguous(), X_ref[:, c].contiguous(), n, n, d, i, p, True, False,
                                        B[:, c].contiguous())
        assert_same(gb, gB[:, c].contiguous(), f"grad_b column {c}")
        gL_ref += gl
    assert_close(gL_ref, gL, "grad_L summed over the 16 right-hand sides")
    # two columns as single-vector calls (the reference's own signature): everything bit for bit
    for c in (0, 15):
        b, g = B[:, c].contiguous(), G[:, c].contiguous()
        x = ops.sptrsv_forward(n, n, dd, di, dp, True, False, b.cuda())
        assert_same(X_ref[:, c].contiguous(), x, f"x, single column {c}")
        gl_ref, gb_ref = oracle.sptrsv_backward(g, X_ref[:, c].contiguous(), n, n, d, i, p, True, False, b)
        gl, gb = ops.sptrsv_backward(g.cuda(), x, n, n, dd, di, dp, True, False, b.cuda())
        assert_same(gb_ref, gb, f"grad_b, single column {c}")
        assert_same(gl_ref, gl, f"grad_L, single column {c}")


# ---- configuration 3: power-law graph, 4,194,304 nodes, K = 128, fp32 ------------------------------
def _compress(rows_indptr, rows_indices):
    """Renumber the columns that a set of rows refers to as 0..u-1 (ascending, so the order of the
    entries within every row is unchanged).  Returns (new indices, the original column of each new one)."""
    cols, inv = torch.unique(rows_indices, return_inverse=True)
    return inv.contiguous(), cols


def test_c3_powerlaw_spmm_full_size(oracle, ops):
    """Y = A X forward and backward on the full graph; rows of Y and the grad_A entries of a fixed
    sample of rows (the first and last rows, every row of the maximum degree 4096, 16384 random rows),
    and grad_X rows of a sample of columns, against the oracle on the sliced matrix."""
    n, K = 4194304, 128
    d, i, p, _ = W.powerlaw_graph(n, dtype=torch.float32)
    nnz = int(d.numel())
    deg = p[1:] - p[:-1]
    assert 60_000_000 < nnz < 70_000_000 and int(deg.max()) <= 4096
    dd, di, dp = cuda(d, i, p)
    gen = torch.Generator(device="cuda").manual_seed(0)
    X = torch.randn((n, K), generator=gen, dtype=torch.float32, device="cuda")
    G = torch.randn((n, K), generator=gen, dtype=torch.float32, device="cuda")
    Y = ops.spdmm_forward(n, n, dd, di, dp, X)
    gA, gX = ops.spdmm_backward(n, n, dd, di, dp, X, G)
    torch.cuda.synchronize()

    rng = np.random.default_rng(5)
    long_rows = torch.nonzero(deg >= 4000).flatten()
    sample = torch.unique(torch.cat((torch.arange(64), torch.arange(n - 64, n), long_rows,
                                     torch.from_numpy(rng.choice(n, 16384, replace=False)))))
    assert sample.numel() >= 16384
    # rows of the sample as a CSR matrix of their own, columns renumbered to the ones they use
    starts, cnts = p[sample], deg[sample]
    sub_ptr = torch.zeros(sample.numel() + 1, dtype=torch.int64)
    sub_ptr[1:] = torch.cumsum(cnts, 0)
    pos = torch.repeat_interleave(starts - sub_ptr[:-1], cnts) + torch.arange(int(sub_ptr[-1]))
    sub_idx, cols = _compress(sub_ptr, i[pos])
    sub_d = d[pos].contiguous()
    Xs = X[cols.cuda()].cpu()
    Gs = G[sample.cuda()].cpu()
    Y_ref = oracle.spdmm_forward(sample.numel(), cols.numel(), sub_d, sub_idx, sub_ptr, Xs)
    assert_same(Y_ref, Y[sample.cuda()], "rows of Y")
    gA_ref, _ = oracle.spdmm_backward(sample.numel(), cols.numel(), sub_d, sub_idx, sub_ptr, Xs, Gs)
    assert_close(gA_ref, gA[pos.cuda()], "grad_A entries of the sampled rows")
    # entry by entry: each is a dot product of 128 terms of size ~1 reduced across lanes in another order
    worst = float(torch.max(torch.abs(gA_ref - gA[pos.cuda()].cpu())))
    assert worst < 1e-4, worst

    # grad_X = A^T G for a sample of columns: the entries of those columns from a transposed copy
    import scipy.sparse as sps
    At = sps.csr_matrix((d.numpy(), i.numpy(), p.numpy()), shape=(n, n)).T.tocsr()
    At.sort_indices()
    csample = np.unique(np.concatenate((np.arange(32), np.arange(n - 32, n), rng.choice(n, 4096, replace=False))))
    sub = At[csample]
    t_idx, t_rows = _compress(None, torch.from_numpy(sub.indices.astype(np.int64)))
    t_ptr = torch.from_numpy(sub.indptr.astype(np.int64))
    t_d = torch.from_numpy(sub.data.astype(np.float32))
    gX_ref = oracle.spdmm_forward(len(csample), t_rows.numel(), t_d, t_idx, t_ptr, G[t_rows.cuda()].cpu())
    assert_same(gX_ref, gX[torch.from_numpy(csample).cuda()], "rows of grad_X")
