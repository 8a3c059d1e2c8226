"""Sparse triangular solves with gradients (reference ``numml/sparse/linalg.py``).

``sptrsv`` keeps the reference's Function signature.  As an extension, ``b`` may have shape
[n, k]: the k right-hand sides are solved together, column by column equal to k single solves,
and grad_A is the sum of the k per-column gradients.  Sparse LU (``splu``, ``spsolve``) is not
part of the accelerated path and raises ``NotImplementedError``.
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


def _no_lu(*_a, **_k):
    raise NotImplementedError("sparse LU factorisation is outside the accelerated CSR path of numml_b200")


splu = splu_solve = spsolve = _no_lu
