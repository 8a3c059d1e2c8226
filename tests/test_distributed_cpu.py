"""Host logic of the row-block partitioned operators, run as gloo ranks on CPU (world sizes 2
and 3).  The local compute is the CPU oracle injected as the operator module, so what is under
test is the partitioner, the column renumbering, the halo plans and the exchanges: results must
equal the single-partition oracle result."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, init_file, case):
    for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import csr_oracle as oracle
    from numml_b200 import distributed as nd, workloads as W
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        if case == "stencil":
            d, i, p, (m, n) = W.poisson3d_7pt(6, torch.float64, nz=6 * world)
            bounds = nd.partition_rows(m, world)
        else:
            d, i, p, (m, n) = W.random_csr(157, 157, 0.06, seed=4, dtype=torch.float64)
            bounds = nd.partition_rows(m, world, indptr=p)          # balanced by nonzeros
        lo, hi = bounds[rank], bounds[rank + 1]
        sl = slice(int(p[lo]), int(p[hi]))
        A = nd.DistSparseCSR(d[sl].clone(), i[sl].clone(), (p[lo:hi + 1] - p[lo]).clone(), (m, n), bounds, ops=oracle)

        # ---- SpMV forward / backward through autograd --------------------------------------
        x, g = W.randn(n, 1, torch.float64), W.randn(m, 2, torch.float64)
        y_ref = oracle.spgemv_forward(m, n, d, i, p, x)
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, n, d, i, p, x)
        A.requires_grad = True
        xl = x[lo:hi].clone().requires_grad_(True)
        y = A @ xl
        y.backward(g[lo:hi])
        assert torch.allclose(y.detach(), y_ref[lo:hi], rtol=1e-13, atol=1e-13)
        assert torch.equal(A.data.grad, gA_ref[sl])
        assert torch.allclose(xl.grad, gx_ref[lo:hi], rtol=1e-13, atol=1e-13)

        # ---- SpMM forward / backward ----------------------------------------------------------
        X, G = W.randn((n, 5), 3, torch.float64), W.randn((m, 5), 4, torch.float64)
        Y_ref = oracle.spdmm_forward(m, n, d, i, p, X)
        gA2_ref, gX_ref = oracle.spdmm_backward(m, n, d, i, p, X, G)
        A.data.grad = None
        Xl = X[lo:hi].clone().requires_grad_(True)
        Y = A @ Xl
        Y.backward(G[lo:hi])
        assert torch.allclose(Y.detach(), Y_ref[lo:hi], rtol=1e-13, atol=1e-13)
        assert torch.allclose(A.data.grad, gA2_ref[sl], rtol=1e-13, atol=1e-13)
        assert torch.allclose(Xl.grad, gX_ref[lo:hi], rtol=1e-13, atol=1e-13)

        # ---- SpGEMM: rows concatenate to the single-partition product ---------------------------
        C_ref = oracle.spgemm_forward(m, n, d, i, p, m, n, d, i, p)
        Cd, Ci, Cp = A @ A
        a, b = int(C_ref[2][lo]), int(C_ref[2][hi])
        assert torch.equal(Cp, C_ref[2][lo:hi + 1] - C_ref[2][lo])
        assert torch.equal(Ci, C_ref[1][a:b])
        assert torch.allclose(Cd, C_ref[0][a:b], rtol=1e-13, atol=1e-13)

        # ---- SpGEMM backward: grad_A local, grad_B of fetched rows sent home and added ---------
        gC = W.randn(C_ref[0].numel(), 6, torch.float64)
        gA3_ref, gB3_ref = oracle.spgemm_backward(gC, C_ref[1], C_ref[2], m, n, d, i, p, m, n, d, i, p)
        Bm = nd.DistSparseCSR(d[sl].clone(), i[sl].clone(), (p[lo:hi + 1] - p[lo]).clone(), (m, n), bounds, ops=oracle)
        Bm.requires_grad = True
        A.data.grad = None
        Cd2, _, _ = A @ Bm
        assert torch.equal(Cd2.detach(), Cd.detach())
        Cd2.backward(gC[a:b])
        assert torch.allclose(A.data.grad, gA3_ref[sl], rtol=1e-13, atol=1e-13)
        assert torch.allclose(Bm.data.grad, gB3_ref[sl], rtol=1e-12, atol=1e-13)
        # second product on the cached structure of the fetched rows, with other values in B
        with torch.no_grad():
            Bm.data.mul_(-0.5)
        Cd3, Ci3, Cp3 = A @ Bm
        C3_ref = oracle.spgemm_forward(m, n, d, i, p, m, n, -0.5 * d, i, p)
        assert torch.equal(Cp3, Cp) and torch.equal(Ci3, Ci)
        assert torch.allclose(Cd3.detach(), C3_ref[0][a:b], rtol=1e-13, atol=1e-13)
        assert len(Bm._fetched_rows) == 1

        # ---- CG with all-reduced dots (SPD case only) -----------------------------------------
        if case == "stencil":
            import numpy as np
            A.requires_grad = False
            bvec = W.randn(m, 5, torch.float64)
            xs, hist = nd.dist_conjugate_gradient(A, bvec[lo:hi].clone(), 15)
            # single-partition CG with the oracle
            xr = torch.zeros(m, dtype=torch.float64)
            r = bvec.clone()
            pv = r.clone()
            rz = r @ r
            h = [rz.sqrt()]
            for _ in range(15):
                Ap = oracle.spgemv_forward(m, n, d, i, p, pv)
                alpha = rz / (Ap @ pv)
                xr = xr + alpha * pv
                r = r - alpha * Ap
                rz_new = r @ r
                pv = r + (rz_new / rz) * pv
                rz = rz_new
                h.append(rz.sqrt())
            assert torch.allclose(xs, xr[lo:hi], rtol=1e-9, atol=1e-12)
            assert torch.allclose(hist, torch.stack(h), rtol=1e-9)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("case", ["stencil", "random"])
def test_partitioned_operators_match_single_partition(world, case):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import csr_oracle
    csr_oracle.build()                                   # build once before the ranks race for it
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(world, os.path.join(tmp, "rendezvous"), case), nprocs=world, join=True)


def test_partition_rows():
    from numml_b200 import distributed as nd
    assert nd.partition_rows(10, 3) == [0, 3, 6, 10]
    indptr = torch.tensor([0, 100, 100, 101, 102, 103, 200])
    b = nd.partition_rows(6, 2, indptr=indptr)
    assert b[0] == 0 and b[-1] == 6 and b == sorted(b)
    assert abs(int(indptr[b[1]]) - 100) <= 3


def test_rows_with_halo_columns_handles_empty_rows():
    """Rows are classified by their own entries only: empty rows (leading, middle, trailing) hold no
    halo column, and the first non-empty row after them is not confused with the running total."""
    sys.path.insert(0, ROOT)
    from numml_b200 import distributed as nd
    nl = 3
    ptr = torch.tensor([0, 0, 2, 3], dtype=torch.int64)
    idx = torch.tensor([0, 5, 1], dtype=torch.int64)
    assert nd.rows_with_halo_columns(idx, ptr, nl).tolist() == [False, True, False]
    ptr = torch.tensor([0, 0, 0, 1, 1, 3, 3], dtype=torch.int64)
    idx = torch.tensor([2, 1, 4], dtype=torch.int64)
    assert nd.rows_with_halo_columns(idx, ptr, nl).tolist() == [False, False, False, False, True, False]
    ptr = torch.zeros(4, dtype=torch.int64)
    assert nd.rows_with_halo_columns(torch.zeros(0, dtype=torch.int64), ptr, nl).tolist() == [False] * 3


def test_ghost_row_extension_reproduces_the_backward():
    """The index logic behind the one-pass distributed backward, emulated on CPU: for each of two
    row blocks of a 3-D stencil, build the ghost-row extension and the mirror positions (transposed
    structure from the oracle), evaluate the kernel's formulas with plain loops and check that
    grad_A and the exchanged grad_x equal the single-partition oracle."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import csr_oracle as oracle
    from numml_b200 import distributed as nd, workloads as W
    d, i, p, (m, n) = W.poisson3d_7pt(5, torch.float64, nz=10)
    d = W.randn(d.numel(), 3, torch.float64)
    x, g = W.randn(n, 1, torch.float64), W.randn(m, 2, torch.float64)
    gA_ref, gx_ref = oracle.spgemv_backward(g, m, n, d, i, p, x)
    bounds = [0, m // 2, m]
    parts = []
    for rank in range(2):
        lo, hi = bounds[rank], bounds[rank + 1]
        sl = slice(int(p[lo]), int(p[hi]))
        data, gi, ptr = d[sl], i[sl], p[lo:hi + 1] - p[lo]
        remote = (gi < lo) | (gi >= hi)
        needed = torch.unique(gi[remote])
        nl = hi - lo
        n_ext = nl + needed.numel()
        idx = torch.where(remote, nl + torch.searchsorted(needed, gi), gi - lo)
        idx_ext, ptr_ext, in_halo = nd.ghost_row_extension(idx, ptr, nl, n_ext)
        assert ptr_ext.numel() == n_ext + 1 and int(ptr_ext[-1]) == idx_ext.numel()
        _, t_idx, t_ptr, t_perm = oracle.csr_transpose_forward(n_ext, n_ext, torch.zeros(idx_ext.numel(), dtype=torch.float64), idx_ext, ptr_ext)
        perm = nd.mirror_positions(idx_ext, ptr_ext, in_halo, t_ptr, t_idx, t_perm)
        assert perm is not None                         # the stencil block is pattern-symmetric
        x_ext = torch.cat((x[lo:hi], x[needed]))
        g_ext = torch.cat((g[lo:hi], torch.zeros(needed.numel(), dtype=torch.float64)))
        gA = torch.zeros(idx_ext.numel(), dtype=torch.float64)
        gx = torch.zeros(n_ext, dtype=torch.float64)
        for r in range(n_ext):                          # what spmv_pipe_kernel mode 3 computes per row
            acc = 0.0
            for k in range(int(ptr_ext[r]), int(ptr_ext[r + 1])):
                c = int(idx_ext[k])
                gA[k] = g_ext[r] * x_ext[c]
                acc += data[int(perm[k])] * g_ext[c]
            gx[r] = acc
        assert torch.equal(gA[:data.numel()], gA_ref[sl])
        parts.append((lo, hi, needed, gx))
    for rank in range(2):
        lo, hi, _, gx = parts[rank]
        total = gx[:hi - lo].clone()
        olo, ohi, oneeded, ogx = parts[1 - rank]
        sel = (oneeded >= lo) & (oneeded < hi)
        total.index_add_(0, oneeded[sel] - lo, ogx[ohi - olo:][sel])
        assert torch.allclose(total, gx_ref[lo:hi], rtol=1e-13, atol=1e-13)

    # a block whose pattern is not symmetric is refused
    idx, ptr = torch.tensor([1, 1]), torch.tensor([0, 1, 2])          # entries (0,1) and (1,1): (1,0) is missing
    _, t_idx, t_ptr, t_perm = oracle.csr_transpose_forward(2, 2, torch.zeros(2, dtype=torch.float64), idx, ptr)
    assert nd.mirror_positions(idx, ptr, torch.zeros(2, dtype=torch.bool), t_ptr, t_idx, t_perm) is None


def _leaving_worker(rank, world, init_file, out_file):
    """Rank 1 leaves right after the rendezvous; rank 0 then starts an exchange that needs it."""
    import datetime
    import time
    for p in (ROOT, os.path.join(ROOT, "oracle")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import csr_oracle as oracle
    from numml_b200 import distributed as nd, workloads as W
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=10))
    if rank == 1:
        os._exit(0)                                    # gone without a word, nothing of its own in flight
    time.sleep(1.0)
    d, i, p, (m, n) = W.poisson3d_7pt(4, torch.float64, nz=8)
    bounds = nd.partition_rows(m, world)
    sl = slice(int(p[bounds[0]]), int(p[bounds[1]]))
    t0 = time.time()
    try:
        A = nd.DistSparseCSR(d[sl].clone(), i[sl].clone(), p[:bounds[1] + 1].clone(), (m, n), bounds, ops=oracle)
        A @ torch.ones(bounds[1], dtype=torch.float64)
        outcome = "completed"
    except Exception as e:                             # noqa: BLE001  (any error is the expected outcome)
        outcome = "error:" + type(e).__name__
    with open(out_file, "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")
    os._exit(0)                                        # the process group cannot be torn down cleanly


def test_a_rank_that_leaves_ends_the_exchange_with_an_error():
    """Failure on the host, no GPU involved: the surviving rank must get an exception from its next
    exchange within the process-group timeout instead of waiting forever."""
    with tempfile.TemporaryDirectory() as tmp:
        init_file, out_file = os.path.join(tmp, "rendezvous"), os.path.join(tmp, "outcome")
        ctx = mp.spawn(_leaving_worker, args=(2, init_file, out_file), nprocs=2, join=False)
        import time
        deadline = time.time() + 90
        while not ctx.join(timeout=2):                 # join() returns as soon as any one process ends
            if time.time() > deadline:
                for proc in ctx.processes:
                    if proc.is_alive():
                        proc.kill()
                pytest.fail("a rank was still waiting after 90 s")
        outcome, seconds = open(out_file).read().split()
        assert outcome.startswith("error:"), outcome
        assert float(seconds) < 60
