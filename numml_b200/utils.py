"""Gradient checks and small tensor helpers with the names of the reference's ``numml/utils.py``:
centred finite differences over the stored entries of a sparse tensor or over a dense tensor
(``sp_fd``, ``reg_fd``, ``fd``), autograd gradients in the same shape (``sp_grad``, ``reg_grad``,
``grad``) and ``unsqueeze_like``."""
import numpy as np
import torch


def _scalar(value):
    """Tensor / array outputs count as the sum of their entries (d sum / d entry = 1)."""
    if isinstance(value, (torch.Tensor, np.ndarray)):
        return value.sum()
    if isinstance(value, (int, float)):
        return value
    raise RuntimeError(f'Unknown type for output: {type(value)}')


def _central_differences(evaluate, flat_values, h):
    """d evaluate / d flat_values[i] by (f(v + h e_i) - f(v - h e_i)) / 2h, one entry at a time."""
    out = torch.empty_like(flat_values)
    with torch.no_grad():
        for i in range(flat_values.numel()):
            probe = flat_values.clone()
            probe[i] = flat_values[i] + h
            upper = _scalar(evaluate(probe))
            probe[i] = flat_values[i] - h
            lower = _scalar(evaluate(probe))
            out[i] = (upper - lower) / (2 * h)
    return out


def _apply(f, arg, fargs):
    return f(arg, *fargs) if fargs is not None else f(arg)


def sp_fd(f, A, fargs=None, h=1e-3):
    """Finite-difference gradient of the scalar ``f(A)`` with respect to the stored entries of the
    SparseCSRTensor ``A``, returned on A's pattern (reference ``numml/utils.py:28-61``)."""
    from . import sparse as sp

    def evaluate(values):
        return _apply(f, sp.SparseCSRTensor((values, A.indices, A.indptr), A.shape, clone=False), fargs)

    grads = _central_differences(evaluate, A.data.detach(), h)
    return sp.SparseCSRTensor((grads, A.indices, A.indptr), A.shape)


def reg_fd(f, x, fargs=None, h=1e-3):
    """Finite-difference gradient of the scalar ``f(x)`` for a dense tensor ``x`` (reference
    ``numml/utils.py:63-99``)."""
    shape = x.shape
    grads = _central_differences(lambda flat: _apply(f, flat.reshape(shape), fargs), x.detach().reshape(-1).clone(), h)
    return grads.reshape(shape)


def fd(f, X, fargs=None, h=1e-3):
    from . import sparse as sp
    if isinstance(X, sp.SparseCSRTensor):
        return sp_fd(f, X, fargs, h)
    if isinstance(X, torch.Tensor):
        return reg_fd(f, X, fargs, h)
    raise RuntimeError(f'Encountered unknown type when trying to take finite difference: {type(X)}.')


def sp_grad(f, A, fargs=None):
    """Autograd gradient of ``f(A)`` with respect to A's stored entries, on A's pattern."""
    from . import sparse as sp
    leaf = A.copy().detach()
    leaf.requires_grad = True
    (g,) = torch.autograd.grad(_scalar(_apply(f, leaf, fargs)), leaf.data)
    return sp.SparseCSRTensor((g, leaf.indices, leaf.indptr), leaf.shape)


def reg_grad(f, X, fargs=None):
    leaf = X.clone().detach().requires_grad_(True)
    (g,) = torch.autograd.grad(_scalar(_apply(f, leaf, fargs)), leaf)
    return g


def grad(f, X, fargs=None):
    from . import sparse as sp
    if isinstance(X, sp.SparseCSRTensor):
        return sp_grad(f, X, fargs)
    if isinstance(X, torch.Tensor):
        return reg_grad(f, X, fargs)
    raise RuntimeError(f'Encountered unknown type when trying to take gradient: {type(X)}.')


def unsqueeze_like(x, y):
    """Insert into 1-D ``x`` the singleton dimensions that ``y`` has (reference
    ``numml/utils.py:152-167``), so that ``A @ y`` comes back in the shape of ``y``."""
    if y.ndim <= 1:
        return x
    for dim, size in enumerate(y.shape):
        if size == 1:
            x = torch.unsqueeze(x, dim)
    return x
