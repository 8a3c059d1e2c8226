"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

Needs the reference checkout (--reference, else $NUMML_REFERENCE) and its CPU operator module compiled
unmodified by oracle/build_ref.py.  Operator-level cases call the reference's C++ functions
directly; API-level cases (autograd through SparseCSRTensor, conjugate gradients) import the
reference's Python package on top of that module.  The outputs are small .npz files that are
committed, so the parity tests can run where the reference is not available.

Usage:  python tests/golden/make_golden.py [--reference /path/to/reference]
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import build_ref  # noqa: E402
from numml_b200 import workloads as W  # noqa: E402


def npy(t):
    return t.detach().cpu().numpy()


def op_level(ref):
    out = {}

    def put(prefix, **kw):
        for k, v in kw.items():
            out[f"{prefix}/{k}"] = npy(v) if isinstance(v, torch.Tensor) else np.asarray(v)

    # ---- SpMV forward / backward ----
    cases = {
        "spmv_poisson2d_f32": W.poisson2d_5pt(8, torch.float32),
        "spmv_random_f64": W.random_csr(40, 30, 0.12, seed=11, dtype=torch.float64),
        "spmv_longrows_f64": W.random_csr(6, 300, 0.5, seed=12, dtype=torch.float64, empty_rows=False),
    }
    for name, (d, i, p, (m, n)) in cases.items():
        x = W.randn(n, 0, d.dtype)
        g = W.randn(m, 1, d.dtype)
        y = ref.spgemv_forward(m, n, d, i, p, x)
        gA, gx = ref.spgemv_backward(g, m, n, d, i, p, x)
        put(name, data=d, indices=i, indptr=p, shape=(m, n), x=x, g=g, y=y, grad_A=gA, grad_x=gx)

    # ---- SpMM forward / backward ----
    for name, dt, K in (("spdmm_f32", torch.float32, 5), ("spdmm_f64", torch.float64, 8)):
        d, i, p, (m, n) = W.random_csr(30, 20, 0.2, seed=21, dtype=dt)
        B = W.randn((n, K), 2, dt)
        G = W.randn((m, K), 3, dt)
        C = ref.spdmm_forward(m, n, d, i, p, B)
        gA, gB = ref.spdmm_backward(m, n, d, i, p, B, G)
        put(name, data=d, indices=i, indptr=p, shape=(m, n), B=B, G=G, C=C, grad_A=gA, grad_B=gB)

    # ---- SpGEMM forward / backward ----
    def spgemm_case(name, A, B, seed):
        (ad, ai, ap, (am, an)), (bd, bi, bp, (bm, bn)) = A, B
        Cd, Ci, Cp = ref.spgemm_forward(am, an, ad, ai, ap, bm, bn, bd, bi, bp)
        gC = W.randn(Cd.numel(), seed, ad.dtype)
        gA, gB = ref.spgemm_backward(gC, Ci, Cp, am, an, ad, ai, ap, bm, bn, bd, bi, bp)
        put(name, A_data=ad, A_indices=ai, A_indptr=ap, A_shape=(am, an),
            B_data=bd, B_indices=bi, B_indptr=bp, B_shape=(bm, bn),
            C_data=Cd, C_indices=Ci, C_indptr=Cp, grad_C=gC, grad_A=gA, grad_B=gB)

    spgemm_case("spgemm_random_f64", W.random_csr(30, 25, 0.15, seed=31), W.random_csr(25, 35, 0.15, seed=32), 4)
    A5 = W.poisson2d_5pt(6, torch.float32)
    spgemm_case("spgemm_laplace_sq_f32", A5, A5, 5)
    P = W.aggregation_2x2(6, torch.float32)
    spgemm_case("spgemm_AP_f32", A5, P, 6)
    # numerically cancelling product: [1 1] * [1; -1] keeps one stored entry with value 0
    one = (torch.tensor([1., 1.], dtype=torch.float64), torch.tensor([0, 1]), torch.tensor([0, 2]), (1, 2))
    col = (torch.tensor([1., -1.], dtype=torch.float64), torch.tensor([0, 0]), torch.tensor([0, 1, 2]), (2, 1))
    spgemm_case("spgemm_cancel_f64", one, col, 7)

    # ---- transpose ----
    for name, dt, shp in (("transpose_f64", torch.float64, (12, 20)), ("transpose_f32", torch.float32, (33, 7))):
        d, i, p, (m, n) = W.random_csr(shp[0], shp[1], 0.3, seed=41, dtype=dt)
        td, ti, tp, perm = ref.csr_transpose_forward(m, n, d, i, p)
        gT = W.randn(d.numel(), 8, dt)
        gA = ref.csr_transpose_backward(gT, perm)
        put(name, data=d, indices=i, indptr=p, shape=(m, n), t_data=td, t_indices=ti, t_indptr=tp,
            t_perm=perm, grad_At=gT, grad_A=gA)

    # ---- triangular solve ----
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for lower in (True, False):
            for unit in (False, True):
                d, i, p, (m, n) = W.random_triangular(40, 0.12, lower=lower, seed=51, dtype=dt)
                b = W.randn(m, 9, dt)
                gx = W.randn(m, 10, dt)
                x = ref.sptrsv_forward(m, n, d, i, p, lower, unit, b)
                gA, gb = ref.sptrsv_backward(gx, x, m, n, d, i, p, lower, unit, b)
                put(f"sptrsv_{tag}_{'lower' if lower else 'upper'}_{'unit' if unit else 'nonunit'}",
                    data=d, indices=i, indptr=p, shape=(m, n), lower=lower, unit=unit, b=b, grad_x=gx,
                    x=x, grad_A=gA, grad_b=gb)
    return out


def api_level(reference):
    """Cases that go through the reference's Python package (autograd Functions, CG)."""
    sys.modules["numml_torch_cpp"] = build_ref.load()
    sys.path.insert(0, reference)
    import numml.sparse as sp
    import numml.krylov as kry

    out = {}
    # conjugate gradients on a small 3-D Laplacian, fixed iteration count (rtol=0 never stops early)
    d, i, p, shape = W.poisson3d_7pt(6, torch.float64)
    A = sp.SparseCSRTensor((d, i, p), shape)
    b = W.randn(shape[0], 0, torch.float64)
    x, hist = kry.conjugate_gradient(A, b, rtol=0.0, iterations=25)
    out["cg_poisson3d/n"] = np.asarray(6)
    out["cg_poisson3d/b"] = npy(b)
    out["cg_poisson3d/x"] = npy(x)
    out["cg_poisson3d/res_hist"] = npy(hist)

    # Galerkin triple product P^T A P with autograd through A and P (reference tests/test_spmm.py:39-157)
    ad, ai, ap, ashape = W.poisson2d_5pt(4, torch.float64)
    pd, pi, pp, pshape = W.aggregation_2x2(4, torch.float64)
    A = sp.SparseCSRTensor((ad, ai, ap), ashape)
    P = sp.SparseCSRTensor((pd, pi, pp), pshape)
    A.requires_grad = True
    P.requires_grad = True
    AH = P.T @ A @ P
    w = W.randn(AH.data.numel(), 3, torch.float64)
    (AH.data * w).sum().backward()
    out["galerkin/n"] = np.asarray(4)
    out["galerkin/w"] = npy(w)
    out["galerkin/AH_data"] = npy(AH.data)
    out["galerkin/AH_indices"] = npy(AH.indices)
    out["galerkin/AH_indptr"] = npy(AH.indptr)
    out["galerkin/grad_A"] = npy(A.data.grad)
    out["galerkin/grad_P"] = npy(P.data.grad)

    # graph-convolution layers (reference numml/nn.py:6-168): weights set explicitly, gradients with
    # respect to the layer parameters, the stored values of A and the node features
    import numml.nn as rnn
    gd, gi, gp, gshape = W.random_csr(30, 30, 0.15, seed=61, dtype=torch.float32)
    gd = gd.abs()                                  # row sums > -1 keep the normalisation real
    out["gnn/A_data"], out["gnn/A_indices"], out["gnn/A_indptr"] = npy(gd), npy(gi), npy(gp)
    X0 = W.randn((30, 4), 62, torch.float32)
    out["gnn/X"] = npy(X0)

    def run(tag, layer, w_seed):
        with torch.no_grad():
            layer.weights.copy_(W.randn(tuple(layer.weights.shape), w_seed, torch.float32))
            layer.bias.copy_(W.randn(tuple(layer.bias.shape), w_seed + 1, torch.float32))
        A = sp.SparseCSRTensor((gd.clone(), gi, gp), gshape)
        A.requires_grad = True
        X = X0.clone().requires_grad_(True)
        Y = layer(A, X)
        w = W.randn(tuple(Y.shape), w_seed + 2, torch.float32)
        (Y * w).sum().backward()
        out[f"gnn/{tag}/weights"] = npy(layer.weights)
        out[f"gnn/{tag}/bias"] = npy(layer.bias)
        out[f"gnn/{tag}/Y"] = npy(Y)
        out[f"gnn/{tag}/w"] = npy(w)
        out[f"gnn/{tag}/grad_weights"] = npy(layer.weights.grad)
        out[f"gnn/{tag}/grad_bias"] = npy(layer.bias.grad)
        out[f"gnn/{tag}/grad_A"] = npy(A.data.grad)
        out[f"gnn/{tag}/grad_X"] = npy(X.grad)

    run("gcn_norm", rnn.GCNConv(4, 3, normalize=True), 70)
    run("gcn_plain", rnn.GCNConv(4, 3, normalize=False), 73)
    run("tag_norm", rnn.TAGConv(4, 3, k=2, normalize=True), 76)
    run("tag_plain", rnn.TAGConv(4, 3, k=3, normalize=False), 79)
    out["rowsum/values"] = npy(sp.SparseCSRTensor((gd, gi, gp), gshape).row_sum())
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=build_ref.DEFAULT_REFERENCE)
    a = ap.parse_args()
    if build_ref.build(a.reference) is None:
        raise SystemExit("reference sources not found; cannot generate golden vectors")
    ref = build_ref.load()
    torch.set_num_threads(1)
    np.savez_compressed(os.path.join(HERE, "ops_small.npz"), **op_level(ref))
    np.savez_compressed(os.path.join(HERE, "api_small.npz"), **api_level(a.reference))
    for f in ("ops_small.npz", "api_small.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
