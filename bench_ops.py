"""Per-operator measurements for the five benchmark configurations, with the reference CPU path
timed beside each one.

    python bench_ops.py [--configs 1,2,3,4,5] [--no-cpu]        (6 = one GCN layer on the C3 graph)

Prints a Markdown table: CUDA-event time of each operator through the operator functions (plan
cached, median of the repetitions), its algorithmic bytes and effective bandwidth as a fraction of
the measured copy bandwidth (MEASURED_PEAKS.json), and the time of the reference's CPU
implementation (the compiled reference in oracle/_ref when present, else the C port) on one host
thread, on the bounded sample stated in the last column.  The CPU leg is the only part that
touches oracle/; it is a reported baseline, not a code path of the library.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))


def peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except OSError:
        return 6650.0, "fallback"


def gpu_ms(fn, reps=10, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def cpu_ms(fn, reps=1):
    fn()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps * 1e3


def cpu_module():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import build_ref
        return build_ref.load(), "reference (oracle/_ref)"
    except ImportError:
        import csr_oracle
        csr_oracle.build()
        return csr_oracle, "C port"


class Report:
    def __init__(self, peak):
        self.peak = peak
        self.rows = []

    def add(self, config, op, ms, bytes_, cpu=None, cpu_note="", extra=""):
        gbs = bytes_ / (ms * 1e-3) / 1e9 if bytes_ else None
        self.rows.append((config, op, ms, bytes_, gbs, cpu, cpu_note, extra))

    def render(self):
        out = ["| config | operator | GPU ms | algorithmic MB | GB/s | of peak | CPU ms (1 thread) | CPU/GPU | notes |",
               "|---|---|---|---|---|---|---|---|---|"]
        for config, op, ms, b, gbs, cpu, note, extra in self.rows:
            out.append("| {} | {} | {:.3f} | {} | {} | {} | {} | {} | {} |".format(
                config, op, ms, f"{b / 1e6:.1f}" if b else "-", f"{gbs:.0f}" if gbs else "-",
                f"{gbs / self.peak:.2f}" if gbs else "-", f"{cpu:.1f}" if cpu is not None else "-",
                f"{cpu / ms:.0f}x" if cpu is not None else "-", "; ".join(x for x in (extra, note) if x)))
        return "\n".join(out)


def spmv_bytes(rows, cols, nnz, s, w):
    fwd = nnz * (s + w) + (rows + 1) * w + cols * s + rows * s
    bwd = fwd + nnz * s + cols * s
    return fwd, bwd


def config12(rep, ops, W, cpu, which):
    if which == 1:
        d, i, p, (m, k) = W.poisson2d_5pt(256, torch.float32)
        name, dt, s = "C1 2-D Poisson 256^2 fp32", torch.float32, 4
    else:
        d, i, p, (m, k) = W.poisson3d_7pt(128, torch.float64)
        name, dt, s = "C2 3-D Poisson 128^3 fp64", torch.float64, 8
    nnz = d.numel()
    x, g = W.randn(k, 0, dt), W.randn(m, 0 + 1, dt)
    dd, di, dp, dx, dg = [t.cuda() for t in (d, i, p, x, g)]
    fb, bb = spmv_bytes(m, k, nnz, s, 4)
    c_f = c_b = None
    if cpu:
        c_f = cpu_ms(lambda: cpu.spgemv_forward(m, k, d, i, p, x), 5)
        c_b = cpu_ms(lambda: cpu.spgemv_backward(g, m, k, d, i, p, x), 5)
    note = "fits in L2: time only" if which == 1 else ""
    rep.add(name, "SpMV forward", gpu_ms(lambda: ops.spgemv_forward(m, k, dd, di, dp, dx), 200, 20), fb, c_f, "full size", note)
    rep.add(name, "SpMV backward", gpu_ms(lambda: ops.spgemv_backward(dg, m, k, dd, di, dp, dx), 200, 20), bb, c_b, "full size", note)
    if which == 2:
        import numml_b200.krylov as kry
        import numml_b200.sparse as sp
        A = sp.SparseCSRTensor((dd, di, dp), (m, k), clone=False)
        b = W.randn(m, 2, dt).cuda()
        ms = gpu_ms(lambda: kry.conjugate_gradient(A, b, rtol=0.0, iterations=100), 3, 1)
        c_cg = None
        if cpu:
            def cpu_cg(iters=5):
                xr = torch.zeros(m, dtype=dt)
                r = b.cpu().clone()
                pv = r.clone()
                rz = r @ r
                for _ in range(iters):
                    Ap = cpu.spgemv_forward(m, k, d, i, p, pv)
                    alpha = rz / (Ap @ pv)
                    xr = xr + alpha * pv
                    r = r - alpha * Ap
                    rzn = r @ r
                    pv = r + (rzn / rz) * pv
                    rz = rzn
            c_cg = cpu_ms(cpu_cg, 1) * 20
        rep.add(name, "100 CG iterations", ms, 100 * (fb + 7 * m * s), c_cg, "5 iterations x 20", "SpMV + 7 vector passes per iteration")


def config3(rep, ops, W, cpu, n=1 << 22):
    d, i, p, (m, k) = W.powerlaw_graph(n, scale=4, seed=0, dtype=torch.float32)
    nnz, K, s, w = d.numel(), 128, 4, 4
    name = f"C3 power-law graph {n} nodes, {nnz} nnz, K=128 fp32"
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    X = torch.randn((k, K), dtype=torch.float32, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    G = torch.randn((m, K), dtype=torch.float32, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    fb = nnz * (s + w) + (m + 1) * w + k * K * s + m * K * s
    gather = nnz * K * s + m * K * s + nnz * (s + w)
    bb = nnz * (s + w) + 2 * m * K * s + k * K * s + nnz * s
    c_f = c_b = None
    sample = 1 << 14
    if cpu:
        Xh, Gh = X.cpu(), G[:sample].cpu().contiguous()
        ps = p[:sample + 1].clone()
        ds, is_ = d[:int(ps[-1])].clone(), i[:int(ps[-1])].clone()
        scale = nnz / float(ds.numel())
        c_f = cpu_ms(lambda: cpu.spdmm_forward(sample, k, ds, is_, ps, Xh)) * scale
        c_b = cpu_ms(lambda: cpu.spdmm_backward(sample, k, ds, is_, ps, Xh, Gh)) * scale
    t_f = gpu_ms(lambda: ops.spdmm_forward(m, k, dd, di, dp, X), 5, 2)
    t_b = gpu_ms(lambda: ops.spdmm_backward(m, k, dd, di, dp, X, G), 5, 2)
    cn = f"first {sample} rows, scaled by nnz"
    rep.add(name, "SpMM forward", t_f, fb, c_f, cn, f"gather model {gather / 1e9:.1f} GB = {gather / (t_f * 1e-3) / 1e9:.0f} GB/s")
    rep.add(name, "SpMM backward", t_b, bb, c_b, cn, "")


def config4(rep, ops, W, cpu, n=2048):
    A = W.poisson2d_5pt(n, torch.float64)
    P = W.aggregation_2x2(n, torch.float64)
    m, (pm, pn) = n * n, P[3]
    name = f"C4 Galerkin, 2-D Poisson {n}^2 fp64"
    dA = [t.cuda() for t in A[:3]]
    dP = [t.cuda() for t in P[:3]]
    s, w = 8, 4
    C = ops.spgemm_forward(m, m, *dA, m, m, *dA)
    nnzA, nnzC = A[0].numel(), C[0].numel()
    fb = 2 * nnzA * (s + w) + nnzC * (s + 8) + 3 * (m + 1) * 8
    gC = torch.randn(nnzC, dtype=torch.float64, device="cuda")
    ops.spgemm_keep_symbolic = False        # the whole product: planning, symbolic and numeric phases
    try:
        t_f = gpu_ms(lambda: ops.spgemm_forward(m, m, *dA, m, m, *dA), 5, 1)
    finally:
        ops.spgemm_keep_symbolic = True
    t_rep = gpu_ms(lambda: ops.spgemm_forward(m, m, *dA, m, m, *dA), 5, 1)
    t_b = gpu_ms(lambda: ops.spgemm_backward(gC, C[1], C[2], m, m, *dA, m, m, *dA), 5, 1)
    c_f = c_b = None
    if cpu:
        c_f = cpu_ms(lambda: cpu.spgemm_forward(m, m, *A[:3], m, m, *A[:3]))
        small = W.poisson2d_5pt(256, torch.float64)
        sm = 256 * 256
        Cs = cpu.spgemm_forward(sm, sm, *small[:3], sm, sm, *small[:3])
        gs = torch.randn(Cs[0].numel(), dtype=torch.float64)
        c_b = cpu_ms(lambda: cpu.spgemm_backward(gs, Cs[1], Cs[2], sm, sm, *small[:3], sm, sm, *small[:3])) * (nnzA / small[0].numel())
    rep.add(name, "SpGEMM A*A forward", t_f, fb, c_f, "full size", f"{nnzC} output nnz = {nnzC / (t_f * 1e-3) / 1e9:.2f} G nnz/s")
    rep.add(name, "SpGEMM A*A forward, same patterns again", t_rep, fb, None, "",
            f"the symbolic phase's results kept from the previous call (the library's default): numeric phase only, {nnzC / (t_rep * 1e-3) / 1e9:.2f} G nnz/s")
    bb = 2 * nnzA * (s + w) + nnzC * (s + 8) + 2 * nnzA * s
    rep.add(name, "SpGEMM A*A backward", t_b, bb, c_b, "256^2 grid, scaled by nnz", "")

    def galerkin():
        Pt = ops.csr_transpose_forward(pm, pn, *dP)
        PtA = ops.spgemm_forward(pn, pm, Pt[0], Pt[1], Pt[2], m, m, *dA)
        return ops.spgemm_forward(pn, m, *PtA, pm, pn, *dP)
    Ac = galerkin()
    c_g = None
    if cpu:
        def cpu_galerkin():
            Pt = cpu.csr_transpose_forward(256 * 256, 128 * 128, *W.aggregation_2x2(256, torch.float64)[:3])
            sm = 256 * 256
            PtA = cpu.spgemm_forward(128 * 128, sm, Pt[0], Pt[1], Pt[2], sm, sm, *W.poisson2d_5pt(256, torch.float64)[:3])
            return cpu.spgemm_forward(128 * 128, sm, *PtA, sm, 128 * 128, *W.aggregation_2x2(256, torch.float64)[:3])
        c_g = cpu_ms(cpu_galerkin) * (n * n / (256.0 * 256.0))
    rep.add(name, "P^T, (P^T A), (P^T A) P", gpu_ms(galerkin, 8, 4), None, c_g, "256^2 grid, scaled by rows",
            f"Ac has {Ac[0].numel()} nnz")


def config5(rep, ops, W, cpu, n=1024):
    d, i, p, (m, _) = W.poisson2d_9pt_lower(n, torch.float64)
    nnz, R, s, w = d.numel(), 16, 8, 4
    name = f"C5 lower 9-point factor {n}^2 fp64, 16 right-hand sides"
    dd, di, dp = d.cuda(), i.cuda(), p.cuda()
    B = torch.randn((m, R), dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    G = torch.randn((m, R), dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    X = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B)      # first call: structure check, index copies,
    torch.cuda.synchronize()                                       # transposed structure, level analysis, solve
    first_ms = (time.perf_counter() - t0) * 1e3
    fb = nnz * (s + w) + (m + 1) * w + 2 * m * R * s
    bb = fb + nnz * (w + s) + 2 * m * R * s + nnz * s
    c_f = c_b = None
    if cpu:
        b1, g1 = B[:, 0].cpu().contiguous(), G[:, 0].cpu().contiguous()
        x1 = X[:, 0].cpu().contiguous()
        c_f = cpu_ms(lambda: cpu.sptrsv_forward(m, m, d, i, p, True, False, b1), 2) * R
        t0 = time.perf_counter()
        cpu.sptrsv_backward(g1, x1, m, m, d, i, p, True, False, b1)
        c_b = (time.perf_counter() - t0) * 1e3 * R
    from numml_b200 import _plan
    levels = _plan.get_plan(m, m, di, dp).sptrsv_order(True)[1]
    rep.add(name, "SpTRSV forward", gpu_ms(lambda: ops.sptrsv_forward(m, m, dd, di, dp, True, False, B), 5, 1), fb, c_f,
            "one right-hand side x 16", f"{levels} dependency levels: latency-bound; first call with the one-off analysis {first_ms:.1f} ms")
    rep.add(name, "SpTRSV backward", gpu_ms(lambda: ops.sptrsv_backward(G, X, m, m, dd, di, dp, True, False, B), 5, 1), bb, c_b,
            "one right-hand side x 16 (the reference transposes per call)", "")
    # the optional cluster kernel (levels inside one thread-block cluster, unknowns through distributed shared memory)
    before = ops.sptrsv_kernel, ops.sptrsv_cluster_ctas
    try:
        for ctas in (8, 16):
            ops.sptrsv_kernel, ops.sptrsv_cluster_ctas = "cluster", ctas
            Xc = ops.sptrsv_forward(m, m, dd, di, dp, True, False, B)
            same = "same bits as the sync-free kernel" if torch.equal(Xc, X) else "DIFFERS from the sync-free kernel"
            rep.add(name, f"SpTRSV forward, cluster kernel ({ctas} CTAs)",
                    gpu_ms(lambda: ops.sptrsv_forward(m, m, dd, di, dp, True, False, B), 5, 1), fb, None, "",
                    f"opt-in (sptrsv_kernel = 'cluster'); {same}")
    finally:
        ops.sptrsv_kernel, ops.sptrsv_cluster_ctas = before


def config6(rep, W, n=1 << 22):
    """One graph-convolution layer (the caller of the C3 SpMM): GCNConv(128 -> 128) with degree
    normalisation on the power-law graph, forward alone and a full training step (forward + backward
    with gradients for the layer parameters, the stored values of A and the node features)."""
    import numml_b200.nn as gnn
    import numml_b200.sparse as sp
    d, i, p, (m, k) = W.powerlaw_graph(n, scale=4, seed=0, dtype=torch.float32)
    K = 128
    name = f"C3 graph, GCNConv({K}->{K}, normalised), {n} nodes, {d.numel()} nnz, fp32"
    A = sp.SparseCSRTensor((d.cuda(), i.cuda(), p.cuda()), (m, k), clone=False)
    A.requires_grad = True
    torch.manual_seed(0)
    layer = gnn.GCNConv(K, K).cuda()
    X = torch.randn((m, K), dtype=torch.float32, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    G = torch.randn((m, K), dtype=torch.float32, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    X.requires_grad_(True)

    def forward_only():
        with torch.no_grad():
            return layer(A, X)

    def step():
        A.data.grad = None
        X.grad = None
        layer.zero_grad(set_to_none=True)
        layer(A, X).backward(G)

    t_f = gpu_ms(forward_only, 5, 2)
    t_s = gpu_ms(step, 5, 2)
    # one row-sum pass over A, one SpMM, one 128x128 GEMM over the features and 5 element-wise passes
    rep.add(name, "layer forward", t_f, None, None, "", "row sums + X W + SpMM + scaling; no CPU column (the reference layer is Python over its operators)")
    rep.add(name, "layer forward + backward", t_s, None, None, "", "gradients for weights, bias, A.data and X")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="1,2,3,4,5")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--small", action="store_true", help="reduced sizes (quick check)")
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from numml_b200 import numml_torch_cpp as ops, workloads as W
    torch.set_num_threads(1)
    cpu, cpu_kind = (None, "not timed") if a.no_cpu else cpu_module()
    peak, kind = peak_gbs()
    rep = Report(peak)
    # a fresh process finds the GPU at idle clocks, which shows in the microsecond-sized calls measured first
    # (C1 forward 16 us instead of 12 us): half a second of copies brings the clocks up before anything is timed
    spin = torch.empty(1 << 26, dtype=torch.float32, device="cuda")
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:
        spin.add_(1.0)
        torch.cuda.synchronize()
    del spin
    for c in [int(x) for x in a.configs.split(",")]:
        if c in (1, 2):
            config12(rep, ops, W, cpu, c)
        elif c == 3:
            config3(rep, ops, W, cpu, (1 << 18) if a.small else (1 << 22))
        elif c == 4:
            config4(rep, ops, W, cpu, 512 if a.small else 2048)
        elif c == 5:
            config5(rep, ops, W, cpu, 256 if a.small else 1024)
        elif c == 6:
            config6(rep, W, (1 << 18) if a.small else (1 << 22))
        torch.cuda.empty_cache()
    print(f"GPU: {torch.cuda.get_device_name(0)}; peak = {peak:.1f} GB/s ({kind} copy bandwidth); "
          f"CPU baseline: {cpu_kind}, 1 thread of {os.cpu_count()} host cores; index width read by the kernels: int32 plan copy\n")
    print(rep.render())


if __name__ == "__main__":
    main()
