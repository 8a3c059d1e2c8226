"""Sparse triangular solves with gradients (reference ``numml/sparse/linalg.py``).

``sptrsv`` keeps the reference's Function signature.  As an extension, ``b`` may have shape
[n, k]: the k right-hand sides are solved together, column by column equal to k single solves,
and grad_A is the sum of the k per-column gradients.  ``splu`` / ``splu_solve`` / ``spsolve`` are the
reference's sparse LU without pivoting and the differentiable direct solve built on it.
"""
import torch

from .. import numml_torch_cpp


class sptrsv(torch.autograd.Function):
    """Sparse triangular solve (reference ``numml/sparse/linalg.py:8-44``)."""

    @staticmethod
    def forward(ctx, shape, A_data, A_indices, A_indptr, lower, unit, b):
        if shape[0] != shape[1]:
            raise RuntimeError(f'Expected square matrix for triangular solve, got {shape[0]} x {shape[1]}.')
        if A_data.type() != b.type():
            raise RuntimeError(f'Matrix and vector should be same data type, got {A_data.type()} and {b.type()}, respectively.')
        x = numml_torch_cpp.sptrsv_forward(shape[0], shape[1], A_data, A_indices, A_indptr, lower, unit, b)
        ctx.save_for_backward(A_data, A_indices, A_indptr, b, x)
        ctx.lower, ctx.unit, ctx.shape = lower, unit, shape
        return x

    @staticmethod
    def backward(ctx, grad_x):
        A_data, A_indices, A_indptr, b, x = ctx.saved_tensors
        grad_A_data, grad_b = numml_torch_cpp.sptrsv_backward(grad_x, x, ctx.shape[0], ctx.shape[1],
                                                              A_data, A_indices, A_indptr, ctx.lower, ctx.unit, b)
        return None, grad_A_data, None, None, None, None, grad_b


def spsolve_triangular(A, b, lower=True, unit_diagonal=False):
    """Solve A x = b for triangular A (reference ``numml/sparse/linalg.py:116-137``)."""
    return sptrsv.apply(A.shape, A.data, A.indices, A.indptr, lower, unit_diagonal, b)


def _sparse_module():
    from . import _csr
    return _csr


def splu(A):
    """Sparse LU factorisation of an invertible matrix without pivoting (reference
    ``numml/sparse/linalg.py:47-56``): returns M = L + U on the filled pattern, L unit lower (its ones
    not stored).  No gradients flow through it; use ``spsolve`` for a solve with gradients."""
    M_data, M_indices, M_indptr = numml_torch_cpp.splu(A.shape[0], A.shape[1], A.data.detach(), A.indices, A.indptr)[:3]
    return _sparse_module().SparseCSRTensor((M_data, M_indices, M_indptr), A.shape, clone=False)


def splu_solve(A_LU, b):
    """Solve A x = b given ``A_LU = splu(A)`` (reference ``numml/sparse/linalg.py:59-78``): a unit lower
    solve followed by an upper solve."""
    y = spsolve_triangular(A_LU, b, True, True)
    return spsolve_triangular(A_LU, y, False, False)


class spsolve_fn(torch.autograd.Function):
    """Direct solve A x = b with gradients for the stored values of A and for b (reference
    ``numml/sparse/linalg.py:81-109``)."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_indices, A_indptr, b):
        if A_data.type() != b.type():
            raise RuntimeError(f'Matrix and vector should be same data type, got {A_data.type()} and {b.type()}, respectively.')
        M_data, M_indices, M_indptr, Mt_data, Mt_indices, Mt_indptr = \
            numml_torch_cpp.splu(A_shape[0], A_shape[1], A_data, A_indices, A_indptr)
        y = numml_torch_cpp.sptrsv_forward(A_shape[0], A_shape[1], M_data, M_indices, M_indptr, True, True, b)
        x = numml_torch_cpp.sptrsv_forward(A_shape[0], A_shape[1], M_data, M_indices, M_indptr, False, False, y)
        ctx.shape = A_shape
        ctx.save_for_backward(A_data, A_indices, A_indptr, Mt_data, Mt_indices, Mt_indptr, x)
        return x

    @staticmethod
    def backward(ctx, grad_x):
        A_data, A_indices, A_indptr, Mt_data, Mt_indices, Mt_indptr, x = ctx.saved_tensors
        grad_A_data, grad_b = numml_torch_cpp.spsolve_backward(grad_x.contiguous(), x, ctx.shape[0], ctx.shape[1],
                                                               Mt_data, Mt_indices, Mt_indptr, A_data, A_indices, A_indptr)
        return None, grad_A_data, None, None, grad_b


def spsolve(A, b):
    """x = A^{-1} b by sparse LU, differentiable (reference ``numml/sparse/linalg.py:112-113``)."""
    return spsolve_fn.apply(A.shape, A.data, A.indices, A.indptr, b)
