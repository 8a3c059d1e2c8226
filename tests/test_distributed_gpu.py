"""Two NCCL ranks on two GPUs (skipped when fewer are visible): partitioned SpMV forward/backward
with the CUDA kernels as local compute must equal the single-partition CPU oracle."""
import os
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, init_file):
    for p in (ROOT, os.path.join(ROOT, "oracle")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import csr_oracle as oracle
    from numml_b200 import distributed as nd, workloads as W
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    # a short collective timeout: if one rank fails an assertion the other must not wait for long
    dist.init_process_group("nccl", init_method="file://" + init_file, rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    try:
        d, i, p, (m, n) = W.poisson3d_7pt(12, torch.float64, nz=12 * world)
        bounds = nd.partition_rows(m, world)
        lo, hi = bounds[rank], bounds[rank + 1]
        sl = slice(int(p[lo]), int(p[hi]))
        A = nd.DistSparseCSR(d[sl].to(dev), i[sl].to(dev), (p[lo:hi + 1] - p[lo]).to(dev), (m, n), bounds)
        x, g = W.randn(n, 1, torch.float64), W.randn(m, 2, torch.float64)
        y_ref = oracle.spgemv_forward(m, n, d, i, p, x)
        gA_ref, gx_ref = oracle.spgemv_backward(g, m, n, d, i, p, x)
        A.requires_grad = True
        xl = x[lo:hi].to(dev).requires_grad_(True)
        y = A @ xl
        y.backward(g[lo:hi].to(dev))
        assert torch.equal(y.detach().cpu(), y_ref[lo:hi])
        assert torch.equal(A.data.grad.cpu(), gA_ref[sl])
        assert torch.allclose(xl.grad.cpu(), gx_ref[lo:hi], rtol=1e-13, atol=1e-13)
        # the pre-planned engine (overlapped exchange, sub-range launches) gives the same results, with the
        # halo values exchanged by NCCL and read from the neighbour's memory by the library's own kernels
        results = {}
        for exchange in ("nccl", "peer"):
            eng = nd.DistSpMVEngine(A, exchange=exchange)
            assert eng.fused                  # symmetric stencil block: one-pass backward over ghost rows
            assert (eng.peer is not None) == (exchange == "peer")
            eng.set_inputs(x[lo:hi].to(dev), g[lo:hi].to(dev))
            dist.barrier()
            for _ in range(3):                # both halves of the exchange buffers get reused
                eng.step()
            replay = eng.capture()
            replay()
            torch.cuda.synchronize()
            assert torch.equal(eng.y.cpu(), y_ref[lo:hi])
            assert torch.equal(eng.grad_A.cpu(), gA_ref[sl])
            assert torch.allclose(eng.grad_x.cpu(), gx_ref[lo:hi], rtol=1e-13, atol=1e-13)
            assert int(eng.status.item()) == 0
            results[exchange] = eng.grad_x.clone()
            if exchange == "peer":            # CG through the same engine against the CPU recurrence
                b = W.randn(m, 5, torch.float64)
                xs, hist = nd.DistCG(eng).solve(b[lo:hi].to(dev), 15)
                xr, r = torch.zeros(m, dtype=torch.float64), b.clone()
                pv, rz, ref = r.clone(), r @ r, []
                ref.append(rz.sqrt())
                for _ in range(15):
                    Ap = oracle.spgemv_forward(m, n, d, i, p, pv)
                    alpha = rz / (Ap @ pv)
                    xr, r = xr + alpha * pv, r - alpha * Ap
                    rz_new = r @ r
                    pv, rz = r + (rz_new / rz) * pv, rz_new
                    ref.append(rz.sqrt())
                assert torch.allclose(hist.cpu(), torch.stack(ref), rtol=1e-9)
                assert torch.allclose(xs.cpu(), xr[lo:hi], rtol=1e-8, atol=1e-10)
                assert int(eng.status.item()) == 0
            eng.close()
        # both exchanges add the neighbours' partial sums in the same order
        assert torch.equal(results["nccl"], results["peer"])
        # SpMM: rows of the dense operand gathered from the neighbour's memory (forward) and partial gradient
        # rows added by their owners (backward) equal the send/recv path bit for bit, and the oracle
        X, G = W.randn((n, 6), 3, torch.float64), W.randn((m, 6), 4, torch.float64)
        Y_ref = oracle.spdmm_forward(m, n, d, i, p, X)
        gA2_ref, gX_ref = oracle.spdmm_backward(m, n, d, i, p, X, G)
        got = {}
        for exchange in ("nccl", "peer", "peer"):              # twice: both halves of the buffers
            os.environ["NB200_EXCHANGE"] = "nccl" if exchange == "nccl" else "auto"
            A.data.grad = None
            Xl = X[lo:hi].to(dev).requires_grad_(True)
            Y = A @ Xl
            Y.backward(G[lo:hi].to(dev))
            assert torch.equal(Y.detach().cpu(), Y_ref[lo:hi])
            assert torch.allclose(A.data.grad.cpu(), gA2_ref[sl], rtol=1e-13, atol=1e-13)
            assert torch.allclose(Xl.grad.cpu(), gX_ref[lo:hi], rtol=1e-13, atol=1e-13)
            got[exchange] = (A.data.grad.clone(), Xl.grad.clone())
        rows = A.halo._row_exchanges[(torch.float64, 6)]
        assert rows is not None and rows.usable
        rows.check()
        assert torch.equal(got["nccl"][0], got["peer"][0]) and torch.equal(got["nccl"][1], got["peer"][1])
        os.environ.pop("NB200_EXCHANGE", None)
        Cd, Ci, Cp = A @ A
        C_ref = oracle.spgemm_forward(m, n, d, i, p, m, n, d, i, p)
        assert torch.equal(Cp.cpu(), C_ref[2][lo:hi + 1] - C_ref[2][lo])
        assert torch.equal(Ci.cpu(), C_ref[1][int(C_ref[2][lo]):int(C_ref[2][hi])])
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_spmv_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import csr_oracle
    csr_oracle.build()
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, os.path.join(tmp, "rendezvous")), nprocs=2, join=True)
