"""GPU parity of the sparse triangular solve and its backward.  The solve reproduces the
reference's arithmetic order, so results are compared bit for bit with the golden vectors and
the CPU oracle; k right-hand sides are checked column by column against k single solves."""
import ctypes

import pytest
import torch

from parity import assert_close, assert_same, case, case_names
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["auto", "cluster"])
def ops(request):
    """The operator shim with its default solve kernel (grid-wide, sync-free) and with the optional cluster
    kernel (taken whenever its ring of recent rows fits)."""
    from numml_b200 import numml_torch_cpp
    before = numml_torch_cpp.sptrsv_kernel
    numml_torch_cpp.sptrsv_kernel = request.param
    yield numml_torch_cpp
    numml_torch_cpp.sptrsv_kernel = before


def test_golden_sptrsv(golden_ops, ops):
    names = case_names(golden_ops, "sptrsv_")
    assert len(names) == 8
    for name in names:
        c = case(golden_ops, name)
        n = int(c["shape"][0])
        lower, unit = bool(c["lower"]), bool(c["unit"])
        d, i, p, b, gx = [c[k].cuda() for k in ("data", "indices", "indptr", "b", "grad_x")]
        x = ops.sptrsv_forward(n, n, d, i, p, lower, unit, b)
        assert_same(c["x"], x, name + " x")
        gA, gb = ops.sptrsv_backward(gx, x, n, n, d, i, p, lower, unit, b)
        assert_same(c["grad_b"], gb, name + " grad_b")
        assert_same(c["grad_A"], gA, name + " grad_A")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("lower", [True, False])
@pytest.mark.parametrize("unit", [False, True])
@pytest.mark.parametrize("n,density", [(1, 1.0), (33, 0.3), (700, 0.02), (2047, 0.004)])
def test_random_vs_oracle(oracle, ops, dtype, lower, unit, n, density):
    d, i, p, _ = W.random_triangular(n, density, lower=lower, seed=n, dtype=dtype)
    b, gx = W.randn(n, 1, dtype), W.randn(n, 2, dtype)
    x_ref = oracle.sptrsv_forward(n, n, d, i, p, lower, unit, b)
    gA_ref, gb_ref = oracle.sptrsv_backward(gx, x_ref, n, n, d, i, p, lower, unit, b)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    x = ops.sptrsv_forward(n, n, dd, di, dp, lower, unit, b.cuda())
    assert_same(x_ref, x, "x")
    gA, gb = ops.sptrsv_backward(gx.cuda(), x, n, n, dd, di, dp, lower, unit, b.cuda())
    assert_same(gb_ref, gb, "grad_b")
    assert_same(gA_ref, gA, "grad_A")


def test_missing_diagonal_entries(oracle, ops):
    """With `unit` the diagonal need not be stored at all (same result as the reference); without
    `unit` a row that stores no diagonal is refused by the structure check before any kernel runs
    (the reference divides by an uninitialised value there)."""
    d, i, p, _ = W.random_triangular(50, 0.2, lower=True, seed=3, dtype=torch.float64, with_diag=False)
    b = W.randn(50, 1, torch.float64)
    x_ref = oracle.sptrsv_forward(50, 50, d, i, p, True, True, b)
    assert_same(x_ref, ops.sptrsv_forward(50, 50, d.cuda(), i.cuda(), p.cuda(), True, True, b.cuda()), "unit, no diagonal")
    with pytest.raises(RuntimeError, match="diagonal"):
        ops.sptrsv_forward(50, 50, d.cuda(), i.cuda(), p.cuda(), True, False, b.cuda())


@pytest.mark.parametrize("nrhs", [1, 2, 3, 16, 40])
@pytest.mark.parametrize("lower", [True, False])
def test_multiple_right_hand_sides(oracle, ops, nrhs, lower):
    n = 300
    d, i, p, _ = W.random_triangular(n, 0.03, lower=lower, seed=8, dtype=torch.float64)
    B, GX = W.randn((n, nrhs), 1, torch.float64), W.randn((n, nrhs), 2, torch.float64)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    X = ops.sptrsv_forward(n, n, dd, di, dp, lower, False, B.cuda())
    gA, gB = ops.sptrsv_backward(GX.cuda(), X, n, n, dd, di, dp, lower, False, B.cuda())
    gA_sum = torch.zeros_like(d)
    for c in range(nrhs):
        x_ref = oracle.sptrsv_forward(n, n, d, i, p, lower, False, B[:, c].contiguous())
        assert_same(x_ref, X[:, c].contiguous(), f"x[:, {c}]")
        gA_c, gb_c = oracle.sptrsv_backward(GX[:, c].contiguous(), x_ref, n, n, d, i, p, lower, False, B[:, c].contiguous())
        assert_same(gb_c, gB[:, c].contiguous(), f"grad_b[:, {c}]")
        gA_sum = gA_sum + gA_c            # the oracle's grad_A for k right-hand sides is the sum of k calls
    assert_same(gA_sum, gA, "grad_A")


def test_nine_point_lower_factor(oracle, ops):
    """The benchmark's matrix family at a size the oracle finishes quickly: lower triangle of the
    2-D 9-point Laplacian (3n-2 dependency levels), 16 right-hand sides."""
    n = 96
    d, i, p, (m, _) = W.poisson2d_9pt_lower(n, torch.float64)
    B, GX = W.randn((m, 16), 0, torch.float64), W.randn((m, 16), 1, torch.float64)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    X = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B.cuda())
    gA, gB = ops.sptrsv_backward(GX.cuda(), X, m, m, dd, di, dp, True, False, B.cuda())
    from numml_b200 import _plan
    assert _plan.get_plan(m, m, di, dp).sptrsv_order(True)[1] == 3 * n - 2
    for c in (0, 7, 15):
        x_ref = oracle.sptrsv_forward(m, m, d, i, p, True, False, B[:, c].contiguous())
        assert_same(x_ref, X[:, c].contiguous(), f"x[:, {c}]")
        _, gb_ref = oracle.sptrsv_backward(GX[:, c].contiguous(), x_ref, m, m, d, i, p, True, False, B[:, c].contiguous())
        assert_same(gb_ref, gB[:, c].contiguous(), f"grad_b[:, {c}]")
    # residual and gradient identities that hold at any size
    L = torch.sparse_csr_tensor(p, i, d, size=(m, m)).to_dense()
    assert torch.linalg.norm(L @ X.cpu() - B) / torch.linalg.norm(B) < 1e-13


def test_residual_at_scale(ops):
    """Benchmark-scale solve (1024^2 grid, 16 right-hand sides): ||L x - b|| / ||b|| is tiny, and
    the backward solve satisfies L^T grad_b = grad_x."""
    n = 1024
    d, i, p, (m, _) = W.poisson2d_9pt_lower(n, torch.float64)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    B = torch.randn((m, 16), dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    X = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B)
    R = ops.spdmm_forward(m, m, dd, di, dp, X) - B
    assert (torch.linalg.norm(R) / torch.linalg.norm(B)).item() < 1e-13
    GX = torch.randn((m, 16), dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    gA, gB = ops.sptrsv_backward(GX, X, m, m, dd, di, dp, True, False, B)
    td, ti, tp, _ = ops.csr_transpose_forward(m, m, dd, di, dp)
    Rt = ops.spdmm_forward(m, m, td, ti, tp, gB) - GX
    assert (torch.linalg.norm(Rt) / torch.linalg.norm(GX)).item() < 1e-13
    assert gA.shape == dd.shape and torch.isfinite(gA).all()


def test_wait_budget_expires_cleanly(ops):
    """A schedule in which a needed row is never solved: the bounded wait must run out, record
    NB200_ERR_WAIT_BUDGET in the status word, poison the output with NaN and leave the context
    usable (no fault, no endless spin)."""
    from numml_b200 import _cabi
    n = 64
    d, i, p, _ = W.random_triangular(n, 0.3, lower=True, seed=1, dtype=torch.float64)
    i32, p32 = i.to(torch.int32).cuda(), p.to(torch.int32).cuda()
    dd, b = d.cuda(), torch.ones(n, dtype=torch.float64, device="cuda")
    x = torch.zeros(n, dtype=torch.float64, device="cuda")
    order = torch.full((n,), n - 1, dtype=torch.int32, device="cuda")   # every team takes the last row
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    _cabi.call("nb200_sptrsv_solve", n, d.numel(), 1, P(dd), P(i32), P(p32), None, P(order), 1, 0, P(b), P(x),
               None, P(status), 2_000_000, 0, _cabi.F64, _cabi.I32,
               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(status.item()) == 5          # NB200_ERR_WAIT_BUDGET
    assert torch.isnan(x[n - 1])
    # the device is still healthy: a regular solve works afterwards
    x2 = ops.sptrsv_forward(n, n, dd, i.cuda(), p.cuda(), True, False, b)
    assert torch.isfinite(x2).all()


def test_shape_checks(ops):
    d, i, p, _ = W.random_triangular(10, 0.3, seed=1)
    with pytest.raises(RuntimeError, match="square"):
        ops.sptrsv_forward(10, 11, d.cuda(), i.cuda(), p.cuda(), True, False, torch.ones(10, dtype=torch.float64, device="cuda"))
    with pytest.raises(RuntimeError, match="right-hand side"):
        ops.sptrsv_forward(10, 10, d.cuda(), i.cuda(), p.cuda(), True, False, torch.ones(9, dtype=torch.float64, device="cuda"))


@pytest.mark.parametrize("nrhs,ctas", [(16, 8), (1, 8), (3, 4), (16, 16), (40, 8)])
def test_cluster_kernel_matches_syncfree_at_scale(nrhs, ctas):
    """512^2 grid (1534 narrow levels): the cluster kernel and the grid-wide kernel give the same bits,
    forward and backward, for cluster sizes 4 / 8 / 16 and right-hand-side counts below, at and above
    the lanes of a team."""
    from numml_b200 import numml_torch_cpp as ops
    n = 512
    d, i, p, (m, _) = W.poisson2d_9pt_lower(n, torch.float64)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    gen = torch.Generator("cuda").manual_seed(nrhs)
    shape = (m,) if nrhs == 1 else (m, nrhs)
    B = torch.randn(shape, dtype=torch.float64, device="cuda", generator=gen)
    GX = torch.randn(shape, dtype=torch.float64, device="cuda", generator=gen)
    before = ops.sptrsv_kernel, ops.sptrsv_cluster_ctas
    try:
        ops.sptrsv_kernel = "syncfree"
        X0 = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B)
        gA0, gB0 = ops.sptrsv_backward(GX, X0, m, m, dd, di, dp, True, False, B)
        ops.sptrsv_kernel, ops.sptrsv_cluster_ctas = "cluster", ctas
        X1 = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B)
        gA1, gB1 = ops.sptrsv_backward(GX, X1, m, m, dd, di, dp, True, False, B)
    finally:
        ops.sptrsv_kernel, ops.sptrsv_cluster_ctas = before
    assert torch.equal(X0, X1) and torch.equal(gB0, gB1) and torch.equal(gA0, gA1)
    from numml_b200 import _plan
    levels = _plan.get_plan(m, m, di, dp).sptrsv_level_plan(True)
    assert levels["nlevels"] == 3 * n - 2 and levels["longest_row"] == 5 and levels["reach"] <= 5 * n
