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
    if rtol <= 0.0 and iterations is not None and M is None and b.is_cuda:
        return _cg_fixed_iterations(A, b, x, int(iterations))
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


def conjugate_residual(A, b, x=None, M=None, rtol=1e-6, iterations=None):
    """Conjugate residuals for symmetric, possibly indefinite ``A`` with an optional SPD
    preconditioner ``M`` (reference ``numml/krylov.py:6-80``; the method of Saad 2003, section 6.8).

    Same quantities, stopping rule and return value as the reference: the preconditioned residual
    ``r = M (b - A x)`` is driven to zero, the loop runs while ``||r|| / ||b|| > rtol`` and for at most
    ``iterations`` steps, and ``(x, res_hist)`` comes back with ``res_hist`` a Python list of the norms
    of ``r`` (one before the first step, one per step).  The initial guess defaults to zeros in the
    dtype of ``b`` (the reference creates it in torch's default dtype, which promotes or fails for a
    float64 ``b``)."""
    assert A.shape[0] == A.shape[1]
    if x is None:
        x = torch.zeros(A.shape[1], device=b.device, dtype=b.dtype)
        r = b.clone()
    else:
        r = b - A @ x
    apply_M = (lambda v: v.clone()) if M is None else (lambda v: M @ v)
    r = apply_M(r)
    p = r.clone()
    Ar = A @ p
    Ap = Ar.clone()
    rAr = r @ Ar
    norm_b = tla.norm(b)
    res_hist = [tla.norm(r)]
    steps = 0
    while res_hist[-1] / norm_b > rtol:
        MAp = apply_M(Ap)
        alpha = rAr / (Ap @ MAp)
        x = x + alpha * p
        r = r - alpha * MAp
        Ar = A @ r
        rAr_next = r @ Ar
        beta = rAr_next / rAr
        p = r + beta * p
        Ap = Ar + beta * Ap
        rAr = rAr_next
        res_hist.append(tla.norm(r))
        steps += 1
        if iterations is not None and steps >= iterations:
            break
    return x, res_hist


def _cg_fixed_iterations(A, b, x, iterations):
    """The same recurrence when the stopping rule can never fire (``rtol <= 0`` with a given
    iteration count, no preconditioner): nothing is read back to the host inside the loop, so
    the iterations queue up on the stream behind one another instead of synchronising twice per
    iteration as the tolerance test and the NaN check of the general loop do.  A NaN residual
    simply propagates to the end, where the history is cut at its first occurrence like the
    early return of the general loop.  A residual that reaches exactly zero ends the reference's
    loop even at rtol = 0; here the remaining iterations leave x unchanged (alpha = beta = 0) and the
    history is cut after its first zero, so the same x and the same history come back."""
    needs_autograd = torch.is_grad_enabled() and (getattr(A, "requires_grad", False) or b.requires_grad
                                                  or (x is not None and x.requires_grad))
    if isinstance(A, sp.SparseCSRTensor) and not needs_autograd:
        # the whole loop runs inside the library: one SpMV and three fused vector kernels per
        # iteration, scalars kept on the device
        from . import numml_torch_cpp
        x, hist = numml_torch_cpp.cg_fixed_iterations(A.shape[0], A.data.detach(), A.indices, A.indptr, b, x, iterations)
        return x, _cut_at_nan(hist)
    if x is None:
        x = torch.zeros(A.shape[1], device=b.device, dtype=b.dtype)
        r = b.clone()
    else:
        r = b - A @ x
    p = r.clone()
    rz = torch.dot(r, r)
    hist = torch.empty(iterations + 1, device=b.device, dtype=b.dtype)
    hist[0] = torch.sqrt(rz)
    for it in range(iterations):
        Ap = A @ p
        done = rz == 0
        alpha = torch.where(done, torch.zeros_like(rz), rz / torch.dot(Ap, p))
        x = x + alpha * p
        r = r - alpha * Ap
        rz_new = torch.dot(r, r)
        p = r + torch.where(done, torch.zeros_like(rz), rz_new / rz) * p
        rz = rz_new
        hist[it + 1] = torch.sqrt(rz)
    return x, _cut_at_nan(hist)


def _cut_at_nan(hist):
    """The history as the reference's loop would have returned it: cut before the first NaN (its
    early return) and after the first exact zero (its stopping test ``norm_r / norm_b > rtol``)."""
    bad = torch.nonzero(torch.isnan(hist)).flatten()
    if bad.numel() > 0:
        hist = hist[:int(bad[0])]
    zero = torch.nonzero(hist == 0).flatten()
    return hist[:int(zero[0]) + 1] if zero.numel() > 0 else hist
