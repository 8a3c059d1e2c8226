"""GPU parity of SpMV forward/backward and the CSR transpose, called through the operator
functions that sit directly on the C ABI.  Checked against the committed golden vectors (made by
the reference itself) and against the CPU oracle on seeded inputs."""
import pytest
import torch

from parity import assert_close, assert_same, case, case_names
from numml_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["auto", "stream", "auto, python shim"])
def ops(request):
    """The operator module, with automatic kernel choice (TMA-pipelined kernels where the pattern
    allows) through the compiled shim and through the Python one, and forced onto the register-staged
    streaming kernels."""
    from numml_b200 import numml_torch_cpp, _plan
    old = (numml_torch_cpp.spmv_kernel, numml_torch_cpp.use_compiled_shim)
    numml_torch_cpp.spmv_kernel = request.param.split(",")[0]
    numml_torch_cpp.use_compiled_shim = "python" not in request.param
    yield numml_torch_cpp
    numml_torch_cpp.spmv_kernel, numml_torch_cpp.use_compiled_shim = old
    numml_torch_cpp.check_status()


def dev(*ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("mode", ["transpose", "atomic"])
def test_golden_spmv(golden_ops, ops, mode):
    ops.spmv_backward_mode = mode
    try:
        for name in case_names(golden_ops, "spmv_"):
            c = case(golden_ops, name)
            m, n = int(c["shape"][0]), int(c["shape"][1])
            d, i, p, x, g = dev(c["data"], c["indices"], c["indptr"], c["x"], c["g"])
            y = ops.spgemv_forward(m, n, d, i, p, x)
            gA, gx = ops.spgemv_backward(g, m, n, d, i, p, x)
            if "longrows" in name:       # warp-per-row kernel: different summation order
                assert_close(c["y"], y, name)
            else:                        # row-streaming kernel keeps the reference's order
                assert_same(c["y"], y, name)
            assert_same(c["grad_A"], gA, name)
            if mode == "transpose" and "longrows" not in name:
                assert_same(c["grad_x"], gx, name)
            else:
                assert_close(c["grad_x"], gx, name)
    finally:
        ops.spmv_backward_mode = "transpose"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("mode", ["transpose", "atomic"])
@pytest.mark.parametrize("shape,density", [((1, 1), 1.0), ((5, 3), 0.5), ((1000, 777), 0.01), ((3000, 3000), 0.002),
                                           ((257, 4100), 0.2), ((4099, 300), 0.01)])
def test_random_vs_oracle(oracle, ops, dtype, mode, shape, density):
    ops.spmv_backward_mode = mode
    try:
        d, i, p, (m, n) = W.random_csr(shape[0], shape[1], density, seed=7, dtype=dtype)
        x, g = W.randn(n, 0, dtype), W.randn(m, 1, dtype)
        y_ref = oracle.spgemv_forward(m, n, d, i, p, x)
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, n, d, i, p, x)
        dd, di, dp, dx, dg = dev(d, i, p, x, g)
        y = ops.spgemv_forward(m, n, dd, di, dp, dx)
        gA, gx = ops.spgemv_backward(dg, m, n, dd, di, dp, dx)
        assert_close(y_ref, y, "y")
        assert_same(gA_ref, gA, "grad_A")
        assert_close(gx_ref, gx, "grad_x")
    finally:
        ops.spmv_backward_mode = "transpose"


def test_empty_matrix_and_empty_rows(ops):
    z = torch.zeros(0, dtype=torch.float64).cuda()
    zi = torch.zeros(0, dtype=torch.int64).cuda()
    p = torch.zeros(6, dtype=torch.int64).cuda()
    x = torch.ones(4, dtype=torch.float64).cuda()
    y = ops.spgemv_forward(5, 4, z, zi, p, x)
    assert y.shape == (5,) and torch.all(y == 0)
    gA, gx = ops.spgemv_backward(torch.ones(5, dtype=torch.float64).cuda(), 5, 4, z, zi, p, x)
    assert gA.numel() == 0 and torch.all(gx == 0)


@pytest.mark.parametrize("n,dtype", [(64, torch.float32), (40, torch.float64)])
def test_stencils_bit_exact(oracle, ops, n, dtype):
    """Stencil matrices go through the row-streaming kernels, whose sums are taken in the
    reference's order: everything must be bit-identical to the CPU oracle."""
    gen = W.poisson2d_5pt if dtype == torch.float32 else W.poisson3d_7pt
    d, i, p, (m, k) = gen(n, dtype)
    x, g = W.randn(k, 0, dtype), W.randn(m, 1, dtype)
    dd, di, dp, dx, dg = dev(d, i, p, x, g)
    assert_same(oracle.spgemv_forward(m, k, d, i, p, x), ops.spgemv_forward(m, k, dd, di, dp, dx), "y")
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, d, i, p, x)
    gA, gx = ops.spgemv_backward(dg, m, k, dd, di, dp, dx)
    assert_same(gA_ref, gA, "grad_A")
    assert_same(gx_ref, gx, "grad_x")


def _symmetric_pattern_case(kind, dtype):
    """A matrix whose PATTERN equals its transpose while its VALUES do not (they are random), so that
    a backward pass that confused an entry with its mirror image would be caught."""
    import numpy as np
    import scipy.sparse as sps
    if kind == "stencil7":                      # every row has at most 7 entries
        _, i, p, (n, _) = W.poisson3d_7pt(20, dtype)
        S = sps.csr_matrix((np.ones(i.numel()), i.numpy(), p.numpy()), shape=(n, n))
    elif kind == "stencil9":                    # interior rows have 9 entries
        _, i, p, (n, _) = W.poisson2d_9pt_lower(70, dtype)
        L = sps.csr_matrix((np.ones(i.numel()), i.numpy(), p.numpy()), shape=(n, n))
        S = (L + L.T).tocsr()
    else:                                       # short random rows plus a few rows of 60+ entries
        n = 6000
        rng = np.random.default_rng(5)
        B = sps.random(n, n, density=2.0 / n, random_state=7, format="lil")
        for h in rng.choice(n, 12, replace=False):
            B[h, rng.choice(n, 60, replace=False)] = 1.0
        B = B.tocsr()
        S = (B + B.T + sps.eye(n)).tocsr()
    S.sort_indices()
    indices = torch.from_numpy(S.indices.astype(np.int64))
    indptr = torch.from_numpy(S.indptr.astype(np.int64))
    data = W.randn(indices.numel(), 3, dtype)
    return data, indices, indptr, S.shape


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("kind", ["stencil7", "stencil9", "hubs"])
def test_symmetric_pattern_random_values_bit_exact(oracle, ops, kind, dtype):
    """The one-pass backward for patterns that equal their transpose, on values that are not
    symmetric: rows short enough for the asynchronous gathers, rows just beyond them, and blocks
    that mix short rows with long ones."""
    from numml_b200 import _plan
    d, i, p, (m, k) = _symmetric_pattern_case(kind, dtype)
    x, g = W.randn(k, 0, dtype), W.randn(m, 1, dtype)
    dd, di, dp, dx, dg = dev(d, i, p, x, g)
    plan = _plan.get_plan(m, k, di, dp)
    assert plan.pattern_symmetric() and plan.spmv_block_rows() > 0
    assert_same(oracle.spgemv_forward(m, k, d, i, p, x), ops.spgemv_forward(m, k, dd, di, dp, dx), "y")
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, d, i, p, x)
    gA, gx = ops.spgemv_backward(dg, m, k, dd, di, dp, dx)
    assert_same(gA_ref, gA, "grad_A")
    assert_same(gx_ref, gx, "grad_x")


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_int64_index_path(oracle, ops, dtype):
    """The kernels also read the int64 arrays exactly as the reference stores them."""
    from numml_b200 import _plan
    _plan.force_int64 = True
    _plan.clear_plan_cache()
    try:
        d, i, p, (m, n) = W.poisson3d_7pt(24, dtype)
        x, g = W.randn(n, 0, dtype), W.randn(m, 1, dtype)
        dd, di, dp, dx, dg = dev(d, i, p, x, g)
        assert_same(oracle.spgemv_forward(m, n, d, i, p, x), ops.spgemv_forward(m, n, dd, di, dp, dx), "y")
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, n, d, i, p, x)
        gA, gx = ops.spgemv_backward(dg, m, n, dd, di, dp, dx)
        assert_same(gA_ref, gA, "grad_A")
        assert_same(gx_ref, gx, "grad_x")
    finally:
        _plan.force_int64 = False
        _plan.clear_plan_cache()


def test_golden_transpose(golden_ops, ops):
    for name in case_names(golden_ops, "transpose_"):
        c = case(golden_ops, name)
        m, n = int(c["shape"][0]), int(c["shape"][1])
        d, i, p = dev(c["data"], c["indices"], c["indptr"])
        td, ti, tp, perm = ops.csr_transpose_forward(m, n, d, i, p)
        for k, v in (("t_data", td), ("t_indices", ti), ("t_indptr", tp), ("t_perm", perm)):
            assert_same(c[k], v, f"{name}/{k}")
        assert_same(c["grad_A"], ops.csr_transpose_backward(c["grad_At"].cuda(), perm), name)


@pytest.mark.parametrize("shape,density", [((512, 64), 0.5), ((64, 512), 0.5), ((20000, 30000), 0.0005),
                                           ((3, 100000), 0.3), ((70000, 2), 0.5), ((1, 1), 1.0)])
def test_transpose_vs_oracle(oracle, ops, shape, density):
    d, i, p, (m, n) = W.random_csr(shape[0], shape[1], density, seed=3, dtype=torch.float64)
    ref = oracle.csr_transpose_forward(m, n, d, i, p)
    got = ops.csr_transpose_forward(m, n, *dev(d, i, p))
    for a, b, what in zip(ref, got, ("t_data", "t_indices", "t_indptr", "t_perm")):
        assert_same(a, b, what)


def test_transpose_full_size_property(ops):
    """At a benchmark-scale size: transposing twice gives the matrix back, and the permutation
    is a bijection (size-independent properties, no oracle needed)."""
    d, i, p, (m, n) = W.poisson3d_7pt(96, torch.float64)
    d = W.randn(d.numel(), 5, torch.float64)
    dd, di, dp = dev(d, i, p)
    td, ti, tp, perm = ops.csr_transpose_forward(m, n, dd, di, dp)
    assert torch.equal(torch.sort(perm).values, torch.arange(d.numel(), device="cuda"))
    d2, i2, p2, _ = ops.csr_transpose_forward(n, m, td, ti, tp)
    assert torch.equal(d2, dd) and torch.equal(i2, di) and torch.equal(p2, dp)


def test_pipelined_kernels_are_chosen_for_stencils(ops):
    from numml_b200 import _plan
    d, i, p, (m, n) = W.poisson3d_7pt(24, torch.float64)
    plan = _plan.get_plan(m, n, i.cuda(), p.cuda())
    assert plan.spmv_block_rows() == 256 and plan.spmv_block_rows(transposed=True) == 256
    d, i, p, (m, n) = W.random_csr(600, 5000, 0.02, seed=1)       # about 100 entries per row
    assert _plan.get_plan(m, n, i.cuda(), p.cuda()).spmv_block_rows() == 0


@pytest.mark.parametrize("n", [127, 255])
def test_full_size_properties(ops, n):
    """At benchmark scale (n^3 rows): A applied to the all-ones vector gives the row sums, which
    for the Dirichlet Laplacian are the number of missing neighbours; forward and backward are
    consistent: <A x, g> == <x, A^T g>; grad_A is the masked outer product."""
    d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    ones = torch.ones(k, dtype=torch.float64, device="cuda")
    y = ops.spgemv_forward(m, k, dd, di, dp, ones)
    counts = (dp[1:] - dp[:-1]).double()
    assert torch.equal(y, 7.0 - counts)
    x = torch.randn(k, dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    g = torch.randn(m, dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    Ax = ops.spgemv_forward(m, k, dd, di, dp, x)
    gA, gx = ops.spgemv_backward(g, m, k, dd, di, dp, x)
    lhs, rhs = torch.dot(Ax, g).item(), torch.dot(x, gx).item()
    assert abs(lhs - rhs) <= 1e-11 * abs(lhs)
    rows = torch.repeat_interleave(torch.arange(m, device="cuda"), dp[1:] - dp[:-1])
    assert torch.equal(gA, g[rows] * x[di])


def test_cpu_tensors_are_rejected(ops):
    d, i, p, (m, n) = W.poisson2d_5pt(4, torch.float32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.spgemv_forward(m, n, d, i, p, torch.ones(n))


def _cabi_ptr(t):
    import ctypes
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def test_row_range_entry_points(oracle):
    """The pieces the row-partitioned driver schedules by hand, called through the C ABI:
    nb200_csr_block_profile, nb200_spgemv_grad_A and nb200_spgemv_backward_symmetric_rows on two
    row ranges that together cover the matrix."""
    import ctypes
    from numml_b200 import _cabi, _plan
    d, i, p, (m, k) = W.poisson3d_7pt(20, torch.float64)
    d = W.randn(d.numel(), 9, torch.float64)
    x, g = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, d, i, p, x)
    dd, di, dp, dx, dg = [t.cuda() for t in (d, i, p, x, g)]
    plan = _plan.get_plan(m, k, di, dp)
    idx, ptr, itype = plan.csr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    prof = torch.empty(4, dtype=torch.int64, device="cuda")
    _cabi.call("nb200_csr_block_profile", m, _cabi_ptr(ptr), itype, _cabi_ptr(prof), stream)
    lens = (p[1:] - p[:-1])
    expect = [int(torch.stack([lens[b:b + R].sum() for b in range(0, m, R)]).max()) for R in (256, 128, 64, 32)]
    assert prof.tolist() == expect
    assert _cabi.lib().nb200_spmv_pipeline_tile() >= expect[0]

    for block_rows in (0, 256):
        gA = torch.full_like(dd, float("nan"))
        _cabi.call("nb200_spgemv_grad_A", m, k, d.numel(), _cabi_ptr(idx), _cabi_ptr(ptr), _cabi_ptr(dx), _cabi_ptr(dg),
                   _cabi_ptr(gA), block_rows, _cabi_ptr(status), _cabi.F64, itype, stream)
        assert_same(gA_ref, gA, f"grad_A (block_rows={block_rows})")

    assert plan.pattern_symmetric()
    _, _, t_perm, _ = plan.transpose()
    cut = 4096                                  # two launches: rows [cut, m) first, then [0, cut)
    # once with values that differ from their mirror images (general pass), once with values made
    # symmetric (d[k] + d[mirror of k]: the same bits on both sides) and the value-symmetric pass
    d_sym = d + d[t_perm.cpu().long()]
    for values_symmetric, vals in ((0, d), (1, d_sym)):
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, vals, i, p, x)
        dv = vals.cuda()
        word = torch.zeros(1, dtype=torch.int32, device="cuda")
        _cabi.call("nb200_csr_values_symmetric", d.numel(), _cabi_ptr(dv), _cabi_ptr(t_perm), _cabi_ptr(word),
                   _cabi.F64, itype, stream)
        assert int(word.item()) == (0 if values_symmetric else 1)
        gA = torch.full_like(dd, float("nan"))
        gx = torch.full_like(dx, float("nan"))
        for lo, hi in ((cut, m), (0, cut)):
            _cabi.call("nb200_spgemv_backward_symmetric_rows", m, d.numel(), lo, hi, _cabi_ptr(dv), _cabi_ptr(idx),
                       _cabi_ptr(ptr), _cabi_ptr(t_perm), _cabi_ptr(dx), _cabi_ptr(dg), _cabi_ptr(gA), _cabi_ptr(gx),
                       values_symmetric, 256, _cabi_ptr(status), _cabi.F64, itype, stream)
        assert_same(gA_ref, gA, f"grad_A (fused, two row ranges, values_symmetric={values_symmetric})")
        assert_same(gx_ref, gx, f"grad_x (fused, two row ranges, values_symmetric={values_symmetric})")
    assert int(status.item()) == 0

    # the forward on a short sub-range of rows (as the row-partitioned driver launches its boundary and ghost rows):
    # block_rows = -1 names the row-streaming kernel, whose sums are the oracle's bit for bit; with 0 the library
    # would go by nnz / rows, which for 300 of 8000 rows says "long rows" and picks the warp-per-row kernel
    y_ref = oracle.spgemv_forward(m, k, d, i, p, x)
    for lo, hi, perm in ((0, 300, None), (4099, 4400, None), (m - 257, m, None), (4099, 4400, t_perm)):
        y = torch.full((m,), float("nan"), dtype=torch.float64, device="cuda")
        ptr_lo = ctypes.c_void_p(ptr.data_ptr() + lo * ptr.element_size())
        y_lo = ctypes.c_void_p(y.data_ptr() + lo * 8)
        vals = dd if perm is None else d_sym.cuda()        # through the mirror permutation symmetric values are themselves
        ref = y_ref if perm is None else oracle.spgemv_forward(m, k, d_sym, i, p, x)
        _cabi.call("nb200_spgemv_forward", hi - lo, k, d.numel(), _cabi_ptr(vals), _cabi_ptr(idx), ptr_lo,
                   _cabi_ptr(perm) if perm is not None else None, _cabi_ptr(dx), y_lo, -1, _cabi_ptr(status), _cabi.F64, itype, stream)
        assert_same(ref[lo:hi], y[lo:hi], f"forward on rows [{lo}, {hi})")
        assert torch.isnan(y[:lo]).all() and torch.isnan(y[hi:]).all()
    assert _cabi.lib().nb200_spgemv_forward(m, k, d.numel(), _cabi_ptr(dd), _cabi_ptr(idx), _cabi_ptr(ptr), None, _cabi_ptr(dx),
                                            _cabi_ptr(y), -2, None, _cabi.F64, itype, stream) == 1      # NB200_ERR_BAD_ARG


@pytest.mark.parametrize("compiled", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_value_symmetric_backward_is_chosen_only_when_it_applies(oracle, dtype, compiled):
    """The operator switches to the value-symmetric pass on the second call with unchanged values, and
    only if the device-side test finds the matrix equal to its transpose bit for bit; an in-place
    change of one value (version bump) sends it back to the general pass.  Results are bit-exact
    against the oracle in every state."""
    from numml_b200 import numml_torch_cpp as ops
    old_shim = ops.use_compiled_shim
    ops.use_compiled_shim = compiled
    if compiled and ops.compiled_shim() is None:
        ops.use_compiled_shim = old_shim
        pytest.skip("the compiled shim has not been built")
    gen = W.poisson2d_5pt if dtype == torch.float32 else W.poisson3d_7pt
    d, i, p, (m, k) = gen(48 if dtype == torch.float32 else 24, dtype)
    x, g = W.randn(k, 0, dtype), W.randn(m, 1, dtype)
    dd, di, dp, dx, dg = [t.cuda() for t in (d, i, p, x, g)]

    def check(vals_cpu, vals_dev, expect_symmetric):
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, k, vals_cpu, i, p, x)
        gA, gx = ops.spgemv_backward(dg, m, k, vals_dev, di, dp, dx)
        assert_same(gA_ref, gA, "grad_A")
        assert_same(gx_ref, gx, "grad_x")
        assert ops.values_symmetric_state(m, k, di, dp) is expect_symmetric

    check(d, dd, None)            # first sighting of these values: general pass, nothing tested yet
    check(d, dd, True)            # second sighting: tested, symmetric -> value-symmetric pass from now on
    check(d, dd, True)
    with torch.no_grad():         # break the symmetry of one off-diagonal pair in place
        dd[1] += 0.5
    d2 = dd.cpu()
    check(d2, dd, None)
    check(d2, dd, False)          # tested, not symmetric: stays on the general pass
    check(d2, dd, False)
    ops.check_status()
    ops.use_compiled_shim = old_shim
