"""Krylov solvers on top of the sparse operators (reference ``numml/krylov.py``)."""
import torch
import torch.linalg as tla

from . import sparse as sp


def conjugate_gradient(A, b, x=None, M=None, rtol=1e-6, iterations=None):
    """Conjugate gradients for SPD ``A`` (reference ``numml/krylov.py:83-155``).

    Same recurrence, stopping rule and return value as the reference: ``(x, res_hist)`` with
    ``res_hist`` the stacked residual norms, one before the first iteration and one per
    iteration.  The initial guess defaults to zeros in the dtype of ``b``.
    """
    assert A.shape[0] == A.shape[1]
    if x is None:
        x = torch.zeros(A.shape[1], device=b.device, dtype=b.dtype)
        r = b.clone()
    else:
        r = b - A @ x
    if M is None:
        M = sp.LinearOperator(A.shape, rm=lambda v: v.clone(), lm=lambda v: v.clone())
    z = M @ r
    p = z.clone()
    norm_b = tla.norm(b)
    it = 0
    norm_r = tla.norm(r)
    res_hist = [norm_r]
    while norm_r / norm_b > rtol:
        Ap = A @ p
        rz = r @ z
        alpha = rz / (Ap @ p)
        x = x + alpha * p
        r = r - alpha * Ap
        z = M @ r
        beta = (r @ z) / rz
        p = z + beta * p
        norm_r = tla.norm(r)
        if torch.any(torch.isnan(norm_r)):
            return x, torch.stack(res_hist)
        res_hist.append(norm_r)
        it += 1
        if iterations is not None and it >= iterations:
            break
    return x, torch.stack(res_hist)
