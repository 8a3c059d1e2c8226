"""Gradient-checking helpers and small tensor utilities (reference ``numml/utils.py``)."""
import numpy as np
import torch


def _to_scalar(f):
    if isinstance(f, (torch.Tensor, np.ndarray)):
        return f.sum()
    if isinstance(f, (int, float)):
        return f
    raise RuntimeError(f'Unknown type for output: {type(f)}')


def _call(f, X, fargs):
    return f(X) if fargs is None else f(X, *fargs)


def sp_fd(f, A, fargs=None, h=1e-3):
    """Centred finite differences of a scalar function with respect to the stored entries of a
    SparseCSRTensor (reference ``numml/utils.py:28-61``)."""
    from . import sparse as sp
    M = A.copy()
    for i in range(M.nnz):
        fwd = torch.clone(A.data)
        fwd[i] += h
        bwd = torch.clone(A.data)
        bwd[i] -= h
        with torch.no_grad():
            f_fwd = _to_scalar(_call(f, sp.SparseCSRTensor((fwd, A.indices, A.indptr), A.shape), fargs))
            f_bwd = _to_scalar(_call(f, sp.SparseCSRTensor((bwd, A.indices, A.indptr), A.shape), fargs))
        M.data[i] = (f_fwd - f_bwd) / (2 * h)
    return M


def reg_fd(f, x, fargs=None, h=1e-3):
    """Centred finite differences with respect to a dense tensor (reference ``numml/utils.py:63-99``)."""
    dx = torch.empty_like(x).flatten()
    for i in range(len(dx)):
        fwd = x.clone().flatten()
        fwd[i] += h
        bwd = x.clone().flatten()
        bwd[i] -= h
        with torch.no_grad():
            f_fwd = _to_scalar(_call(f, fwd.reshape(x.shape), fargs))
            f_bwd = _to_scalar(_call(f, bwd.reshape(x.shape), fargs))
        dx[i] = (f_fwd - f_bwd) / (2 * h)
    return dx.reshape(x.shape)


def fd(f, X, fargs=None, h=1e-3):
    from . import sparse as sp
    if isinstance(X, sp.SparseCSRTensor):
        return sp_fd(f, X, fargs, h)
    if isinstance(X, torch.Tensor):
        return reg_fd(f, X, fargs, h)
    raise RuntimeError(f'Encountered unknown type when trying to take finite difference: {type(X)}.')


def sp_grad(f, A, fargs=None):
    """Autograd gradient of a scalar function with respect to the stored entries of A."""
    from . import sparse as sp
    A = A.copy().detach()
    A.requires_grad = True
    (g,) = torch.autograd.grad(_to_scalar(_call(f, A, fargs)), A.data)
    return sp.SparseCSRTensor((g, A.indices, A.indptr), A.shape)


def reg_grad(f, X, fargs=None):
    X = X.clone().detach()
    X.requires_grad = True
    (g,) = torch.autograd.grad(_to_scalar(_call(f, X, fargs)), X)
    return g


def grad(f, X, fargs=None):
    from . import sparse as sp
    if isinstance(X, sp.SparseCSRTensor):
        return sp_grad(f, X, fargs)
    if isinstance(X, torch.Tensor):
        return reg_grad(f, X, fargs)
    raise RuntimeError(f'Encountered unknown type when trying to take gradient: {type(X)}.')


def unsqueeze_like(x, y):
    """Give 1-D ``x`` the singleton dimensions of ``y`` (reference ``numml/utils.py:152-167``)."""
    for dim, size in enumerate(y.shape):
        if size == 1 and y.ndim > 1:
            x = torch.unsqueeze(x, dim)
    return x
