"""The peer-memory halo exchange kernels on one GPU, called through the C ABI.  The "neighbour" is a
second buffer on the same device, so the packing, the step counting, the double-buffered halves, the
ordered additions and the bounded waits can all be checked without a second process.  (Waiting kernels
of different ranks must not share a GPU; here nothing waits for a kernel that has not run yet, except in
the time-out case, where nothing ever sets the flag and the wait is made to run out.)"""
import ctypes

import pytest
import torch

from numml_b200 import _cabi

pytestmark = pytest.mark.gpu
P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
ERR_WAIT_BUDGET = 5


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype,code", [(torch.float64, _cabi.F64), (torch.float32, _cabi.F32)])
def test_publish_pull_and_pull_add_round_trip(dtype, code):
    dev = "cuda"
    n_local, count = 1000, 300
    es = torch.empty(0, dtype=dtype).element_size()
    # the neighbour's exchange buffer: [flag_x, flag_g, ...][x area: 2 halves][g area: 2 halves]
    buf = torch.zeros(256 + 2 * count * es + 2 * count * es, dtype=torch.uint8, device=dev)
    x_area, g_area = buf.data_ptr() + 256, buf.data_ptr() + 256 + 2 * count * es
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    idx = torch.randperm(n_local, device=dev)[:count].contiguous()
    x_desc = torch.tensor([x_area, count, 40, 200, 5, buf.data_ptr(), 0, 0], dtype=torch.int64, device=dev)
    g_desc = torch.tensor([g_area, count, 0, 0, 0, buf.data_ptr() + 4, 0, 0], dtype=torch.int64, device=dev)
    # gradient targets: 150 distinct indices, each receiving two elements of the packed area
    targets = torch.sort(torch.randperm(n_local, device=dev)[:150]).values.contiguous()
    tptr = (2 * torch.arange(151, device=dev)).contiguous()
    src_peer = torch.zeros(300, dtype=torch.int32, device=dev)
    src_elem = torch.randperm(count, device=dev).contiguous()
    for t in (1, 2, 3):                                   # three steps: both halves get reused
        src = torch.randn(n_local, dtype=dtype, device=dev)
        _cabi.call("nb200_halo_publish", count, P(src), P(idx), ctypes.c_void_p(x_area), P(buf), P(step), 1, P(arrivals),
                   code, _stream())
        dst = torch.full((400,), -7.0, dtype=dtype, device=dev)
        _cabi.call("nb200_halo_pull", 1, P(x_desc), 200, P(dst), P(step), P(status), 0, code, _stream())
        assert int(step.item()) == t and buf[:4].view(torch.int32).item() == t
        assert torch.equal(dst[5:205], src[idx][40:240])
        assert torch.all(dst[:5] == -7.0) and torch.all(dst[205:] == -7.0)
        part = torch.randn(count, dtype=dtype, device=dev)
        _cabi.call("nb200_halo_publish", count, P(part), None, ctypes.c_void_p(g_area), ctypes.c_void_p(buf.data_ptr() + 4),
                   P(step), 0, P(arrivals), code, _stream())
        grad = torch.randn(n_local, dtype=dtype, device=dev)
        expect = grad.clone()
        expect[targets] = (grad[targets] + part[src_elem[0::2]]) + part[src_elem[1::2]]      # in the listed order
        _cabi.call("nb200_halo_pull_add", 1, P(g_desc), 150, P(targets), P(tptr), P(src_peer), P(src_elem), P(grad), P(step),
                   P(status), 0, code, _stream())
        assert torch.equal(grad, expect)
        assert int(step.item()) == t and buf[4:8].view(torch.int32).item() == t
    assert int(status.item()) == 0 and int(arrivals.item()) == 0


def test_wait_budget_runs_out_cleanly():
    """A flag that nobody sets: both pulling kernels give up after the cycle budget, report
    NB200_ERR_WAIT_BUDGET in the status word, copy nothing, and the context stays usable."""
    dev = "cuda"
    buf = torch.zeros(256 + 2 * 64 * 8, dtype=torch.uint8, device=dev)
    step = torch.full((1,), 3, dtype=torch.int32, device=dev)       # the current step is 3; the flag stays 0
    desc = torch.tensor([buf.data_ptr() + 256, 64, 0, 64, 0, buf.data_ptr(), 0, 0], dtype=torch.int64, device=dev)
    dst = torch.full((64,), -1.0, dtype=torch.float64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _cabi.call("nb200_halo_pull", 1, P(desc), 64, P(dst), P(step), P(status), 2_000_000, _cabi.F64, _stream())
    torch.cuda.synchronize()
    assert int(status.item()) == ERR_WAIT_BUDGET and torch.all(dst == -1.0)
    status.zero_()
    grad = torch.ones(8, dtype=torch.float64, device=dev)
    targets = torch.arange(8, device=dev)
    tptr = torch.arange(9, device=dev)
    _cabi.call("nb200_halo_pull_add", 1, P(desc), 8, P(targets), P(tptr), P(torch.zeros(8, dtype=torch.int32, device=dev)),
               P(torch.arange(8, device=dev)), P(grad), P(step), P(status), 2_000_000, _cabi.F64, _stream())
    torch.cuda.synchronize()
    assert int(status.item()) == ERR_WAIT_BUDGET and torch.all(grad == 1.0)
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0      # the device still answers


@pytest.mark.parametrize("dtype,code,width", [(torch.float64, _cabi.F64, 6), (torch.float32, _cabi.F32, 128)])
def test_rows_publish_pull_and_pull_add(dtype, code, width):
    """Rows of a dense operand: the neighbour publishes its whole block, this rank gathers the rows it needs by
    index; partial gradient rows are added to their targets in the listed order.  Three steps reuse both halves."""
    dev = "cuda"
    n_peer, n_halo, n_local = 500, 220, 400
    es = torch.empty(0, dtype=dtype).element_size()
    row_bytes = width * es
    buf = torch.zeros(256 + 2 * n_peer * row_bytes + 2 * n_halo * row_bytes, dtype=torch.uint8, device=dev)
    x_area, g_area = buf.data_ptr() + 256, buf.data_ptr() + 256 + 2 * n_peer * row_bytes
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    row_of_slot = torch.cat((torch.zeros(7, dtype=torch.int64, device=dev),          # slots of another neighbour
                             torch.sort(torch.randperm(n_peer, device=dev)[:n_halo]).values)).contiguous()
    x_desc = torch.tensor([x_area, n_peer, 7, n_halo, n_local, buf.data_ptr(), 0, 0], dtype=torch.int64, device=dev)
    g_desc = torch.tensor([g_area, n_halo, 0, 0, 0, buf.data_ptr() + 4, 0, 0], dtype=torch.int64, device=dev)
    targets = torch.sort(torch.randperm(n_local, device=dev)[:110]).values.contiguous()
    tptr = (2 * torch.arange(111, device=dev)).contiguous()
    src_peer = torch.zeros(220, dtype=torch.int32, device=dev)
    src_elem = torch.randperm(n_halo, device=dev).contiguous()
    for t in (1, 2, 3):
        block = torch.randn((n_peer, width), dtype=dtype, device=dev)
        _cabi.call("nb200_halo_publish", n_peer * width, P(block), None, ctypes.c_void_p(x_area), P(buf), P(step), 1,
                   P(arrivals), code, _stream())
        x_ext = torch.full((n_local + n_halo + 3, width), -7.0, dtype=dtype, device=dev)
        _cabi.call("nb200_halo_pull_rows", 1, P(x_desc), P(row_of_slot), n_halo, row_bytes, P(x_ext), P(step), P(status),
                   0, _stream())
        assert int(step.item()) == t
        assert torch.equal(x_ext[n_local:n_local + n_halo], block[row_of_slot[7:]])
        assert torch.all(x_ext[:n_local] == -7.0) and torch.all(x_ext[n_local + n_halo:] == -7.0)
        part = torch.randn((n_halo, width), dtype=dtype, device=dev)
        _cabi.call("nb200_halo_publish", n_halo * width, P(part), None, ctypes.c_void_p(g_area),
                   ctypes.c_void_p(buf.data_ptr() + 4), P(step), 0, P(arrivals), code, _stream())
        grad = torch.randn((n_local, width), dtype=dtype, device=dev)
        expect = grad.clone()
        expect[targets] = (grad[targets] + part[src_elem[0::2]]) + part[src_elem[1::2]]
        _cabi.call("nb200_halo_pull_add_rows", 1, P(g_desc), 110, P(targets), P(tptr), P(src_peer), P(src_elem), row_bytes,
                   P(grad), P(step), P(status), 0, code, _stream())
        assert torch.equal(grad, expect)
    assert int(status.item()) == 0 and int(arrivals.item()) == 0
    # a flag that nothing sets: the row kernels give up and leave their outputs alone
    step.fill_(9)
    x_ext = torch.full((n_local + n_halo, width), -1.0, dtype=dtype, device=dev)
    _cabi.call("nb200_halo_pull_rows", 1, P(x_desc), P(row_of_slot), n_halo, row_bytes, P(x_ext), P(step), P(status),
               2_000_000, _stream())
    torch.cuda.synchronize()
    assert int(status.item()) == ERR_WAIT_BUDGET and torch.all(x_ext == -1.0)
    # a row that is not a multiple of 16 bytes is refused
    with pytest.raises(RuntimeError):
        _cabi.call("nb200_halo_pull_rows", 1, P(x_desc), P(row_of_slot), n_halo, 24, P(x_ext), P(step), P(status), 0, _stream())


@pytest.mark.parametrize("dtype,code", [(torch.float64, _cabi.F64), (torch.float32, _cabi.F32)])
def test_publish_rowsums_matches_row_sums_then_publish(dtype, code):
    """The fused launch (row sums through a permutation, written straight into the packed area, flag raised) gives
    the bits of the two-launch path: the row-streaming forward kernel over the same rows, then nb200_halo_publish."""
    dev = "cuda"
    from numml_b200 import workloads as W
    d, i, p, (m, k) = W.random_csr(700, 900, 0.01, seed=5, dtype=dtype)
    rows0 = 123                                           # the published rows are rows [rows0, m)
    nrows = m - rows0
    es = torch.empty(0, dtype=dtype).element_size()
    perm = torch.randperm(d.numel())
    dd, di, dp, dperm = d.cuda(), i.cuda().to(torch.int32), p.cuda().to(torch.int32), perm.cuda().to(torch.int32)
    x = torch.randn(k, dtype=dtype, device=dev)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
    ptr_lo = ctypes.c_void_p(dp.data_ptr() + rows0 * 4)
    for t in (1, 2, 3):
        buf = torch.zeros(256 + 2 * nrows * es, dtype=torch.uint8, device=dev)
        area = ctypes.c_void_p(buf.data_ptr() + 256)
        y = torch.empty(m, dtype=dtype, device=dev)
        _cabi.call("nb200_spgemv_forward", nrows, k, d.numel(), P(dd), P(di), ptr_lo, P(dperm), P(x),
                   ctypes.c_void_p(y.data_ptr() + rows0 * es), -1, None, code, _cabi.I32, _stream())
        _cabi.call("nb200_halo_publish_rowsums", nrows, P(dd), P(di), ptr_lo, P(dperm), P(x), area, P(buf), P(step), 1,
                   P(arrivals), code, _cabi.I32, _stream())
        assert int(step.item()) == t and buf[:4].view(torch.int32).item() == t
        half = buf[256:].view(dtype)[(t & 1) * nrows:(t & 1) * nrows + nrows]
        assert torch.equal(half, y[rows0:])
        other = buf[256:].view(dtype)[(1 - (t & 1)) * nrows:(1 - (t & 1)) * nrows + nrows]
        assert torch.all(other == 0)
    assert int(arrivals.item()) == 0
