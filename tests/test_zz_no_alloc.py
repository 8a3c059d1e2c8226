"""The allocation-free float32 triangular solve, called through the C ABI.

Some hosts of this library cannot give it device memory (an embedding runtime that owns the pool,
a loop that must never reach cudaMalloc), so this one entry point keeps its double-precision
working array inside the library.  The test checks it against the regular entry point, which
takes the working array from the caller: outputs must be bit-identical, on two calls in a row with
different right-hand sides (the shared array keeps the first call's contents, which the second call
must not see).  This file sorts last so that a run that stops at the first failure has already
run every other test; it passes on its own in a fresh process as well.
"""
import ctypes

import pytest
import torch

from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _problem(n, nrhs, lower, seed):
    from numml_b200 import _plan
    d, i, p, _ = W.random_triangular(n, min(1.0, 6.0 / n), lower=lower, seed=seed, dtype=torch.float32)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    plan = _plan.get_plan(n, n, di, dp)
    idx, ptr, itype = plan.csr()
    order, _ = plan.sptrsv_order(lower)
    return dd, idx, ptr, itype, order, int(d.numel())


@pytest.mark.parametrize("n,nrhs,lower", [(500, 1, True), (300, 16, False), (4096, 3, True)])
def test_noalloc_solve_matches_regular_entry_point(n, nrhs, lower):
    from numml_b200 import _cabi
    data, idx, ptr, itype, order, nnz = _problem(n, nrhs, lower, seed=n)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    shape = (n,) if nrhs == 1 else (n, nrhs)
    for call in range(2):                       # two calls in a row share the library's working array
        b = W.randn(shape, 100 + call, torch.float32).cuda()
        x_ref = torch.empty_like(b)
        xd = torch.empty(n * nrhs, dtype=torch.float64, device="cuda")
        _cabi.call("nb200_sptrsv_solve", n, nnz, nrhs, P(data), P(idx), P(ptr), None, P(order), int(lower), 0,
                   P(b), P(x_ref), P(xd), P(status), 0, 0, _cabi.F32, itype, stream)
        x = torch.full_like(b, float("nan"))
        _cabi.call("nb200_sptrsv_solve_f32_noalloc", n, nnz, nrhs, P(data), P(idx), P(ptr), None, P(order),
                   int(lower), 0, P(b), P(x), P(status), 0, itype, stream)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.isfinite(x_ref).all()
        assert torch.equal(x, x_ref), f"call {call}: outputs differ"


def test_noalloc_solve_rejects_oversized_problems():
    from numml_b200 import _cabi
    cap = _cabi.lib().nb200_sptrsv_solve_f32_noalloc_capacity()
    assert cap == 1 << 20
    with pytest.raises(_cabi.NB200Error) as err:
        _cabi.call("nb200_sptrsv_solve_f32_noalloc", cap // 8 + 1, 0, 8, None, None, None, None, None, 1, 0,
                   None, None, None, 0, _cabi.I32, None)
    assert err.value.status == 3                # NB200_ERR_TOO_LARGE, before anything is launched
