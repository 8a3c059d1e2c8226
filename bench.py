"""Benchmark of the differentiable-CSR hot path on B200.

Headline (one JSON line, rank 0): one step = SpMV forward (y = A x) followed by SpMV backward
(grad_A.data = g_i x_j on the pattern, grad_x = A^T g) on the 3-D Poisson 7-point Laplacian of a
128^3 grid in fp64 (2,097,152 rows, 14,581,760 nonzeros).  With N > 1 GPUs every rank owns one 128^3
slab of a 128 x 128 x 128N grid (row-block partition, weak scaling) and exchanges one 128^2 halo plane
of x (forward) and of the grad_x partial sums (backward) with each z-neighbour.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--grid n] [--no-extras]

`value` is effective GB/s over the whole job with everything resident in HBM: algorithmic bytes of
forward + backward (4-byte indices credited in both arms) divided by the CUDA-event time of K steps,
max over ranks; the K-step block is repeated until at least --min-timed-s seconds have been timed and
the median block is reported.  Before anything is timed one step is compared with the CPU oracle on
every rank; a mismatch aborts the run.  `e2e` is the same metric through the public SparseCSRTensor API
with x and g starting in pinned host memory and y, grad_x, grad_A copied back to the host inside the
timed region (the matrix stays resident, as it does for a reference user after `A.to(device)`).

`extra` holds the other partitioned operators of the hot path, each timed on the same N GPUs after the
headline and each checked against the oracle on a sample first:
  strong  the fixed 128^3 matrix split N ways (SpMV forward + backward)
  cg      100 unpreconditioned CG iterations on the fixed 128^3 matrix split N ways
  spgemm  C = A A on the 2-D Poisson 2048^2 grid (symbolic + numeric, allocation included), row
          partitioned; output nnz per second; backward
  spmm    Y = A X on the power-law graph (4,194,304 nodes, K = 128, fp32), rows balanced by nnz;
          forward and backward, with and without the exchange of the dense rows

`--impl reference` times the reference's own CPU implementation (oracle/_ref, else the C port) of the
headline step on the host cores.
"""
import argparse
import ctypes
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "spmv_fwd_bwd_effective_GBps"
UNIT = "GB/s"
INDEX_BYTES_CREDITED = 4     # both arms credit the narrowed index width, whatever each of them reads


def algorithmic_bytes(rows, cols, nnz, s, w):
    """Bytes that forward and backward must move (value size s, index size w)."""
    fwd = nnz * (s + w) + (rows + 1) * w + cols * s + rows * s
    bwd = nnz * (s + w) + (rows + 1) * w + cols * s + rows * s + nnz * s + cols * s
    return fwd, bwd


def workload_config(n, rows, nnz):
    """The `config` object: identical in both arms."""
    return {"workload": f"poisson3d_7pt_{n}^3_fp64_spmv_fwd_bwd", "rows_per_gpu": rows, "nnz_per_gpu": nnz,
            "index_bytes_credited": INDEX_BYTES_CREDITED,
            "l2": "working set per step (>= 350 MB) is larger than the 126 MB L2; no explicit flush"}


def ncu_traffic(kernel_key, nnz):
    """DRAM bytes per launch of the named kernel from the committed ncu capture (taken on the
    128^3 workload; scaled by nnz for other grid sizes, traffic being proportional to it)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            t = json.load(f)[kernel_key]
        return int((t["read"] + t["write"]) * (nnz / 14581760.0))
    except (OSError, KeyError, ValueError):
        return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, val in zip(names, p[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "samples": len(sm), "reasons": sorted(reasons)}


# -------------------------------------------------------------------------------------------------
# CPU side: the oracle as checker, and the reference's CPU path as the timed baseline
# -------------------------------------------------------------------------------------------------
def oracle_port():
    """The C restatement of the reference CPU algorithms (bit-identical to the compiled reference;
    used here only to check results)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import csr_oracle
    csr_oracle.build()
    return csr_oracle


def reference_cpu_module():
    """(module, kind): the reference's own CPU operator module when oracle/_ref is built, else the port."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import build_ref
        return build_ref.load(), "reference"
    except ImportError:
        return oracle_port(), "port"


def cpu_steps(n, warmup, steps=None, budget_s=None):
    """Times the reference CPU path on the headline step, one host thread (its kernels are serial loops
    and its own protocol pins one thread, demos/timing.py:15).  Runs `steps` steps, or as many as fit
    `budget_s` seconds (at most 100).  Returns (median ms per step, steps run, kind, rows, nnz)."""
    from numml_b200 import workloads as W
    mod, kind = reference_cpu_module()
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
    x, g = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)

    def step():
        mod.spgemv_forward(m, k, d, i, p, x)
        mod.spgemv_backward(g, m, k, d, i, p, x)

    for _ in range(warmup):
        step()
    times, t_start = [], time.perf_counter()
    while True:
        t0 = time.perf_counter()
        step()
        times.append((time.perf_counter() - t0) * 1e3)
        if steps is not None and len(times) >= steps:
            break
        if steps is None and (time.perf_counter() - t_start > budget_s or len(times) >= 100):
            break
    torch.set_num_threads(threads)
    return statistics.median(times), len(times), kind, m, int(d.numel())


def reference_arm(args, rank):
    """The reference's CPU implementation of the same step on the host cores (rank 0 only)."""
    if rank != 0:
        return
    n = args.grid
    ms, steps, kind, m, nnz = cpu_steps(n, args.warmup, steps=args.steps)
    fwd_b, bwd_b = algorithmic_bytes(m, m, nnz, 8, INDEX_BYTES_CREDITED)
    value = (fwd_b + bwd_b) / (ms * 1e-3) / 1e9
    sample = f"{steps} full steps (forward+backward) of the {n}^3 workload, 1 thread, median step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(n, m, nnz),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline(n, budget_s=12.0):
    """Reference CPU path on a bounded sample of the same workload (rank 0, N=1 only)."""
    ms, steps, kind, m, nnz = cpu_steps(n, 2, budget_s=budget_s)
    fwd_b, bwd_b = algorithmic_bytes(m, m, nnz, 8, INDEX_BYTES_CREDITED)
    return {"value": (fwd_b + bwd_b) / (ms * 1e-3) / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
            "ms_per_step": ms, "host_cores": os.cpu_count(),
            "sample": f"{steps} full steps (forward+backward) of the {n}^3 workload, 1 thread, median step"}


# -------------------------------------------------------------------------------------------------
# Timing helpers
# -------------------------------------------------------------------------------------------------
class Ctx:
    """What every measurement needs: rank, world, device, the process group (or None)."""

    def __init__(self, rank, world, dev, dist):
        self.rank, self.world, self.dev, self.dist = rank, world, dev, dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.dist is None:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def sum_over_ranks(self, v):
        if self.dist is None:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t.item()

    def all_true(self, ok):
        return self.sum_over_ranks(0.0 if ok else 1.0) == 0.0


def timed_block(ctx, step, steps):
    """CUDA-event time (ms) of `steps` calls of `step`, barrier + synchronize on both sides, max over ranks."""
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    ctx.barrier()
    return ms


def timed_blocks(ctx, step, steps, warmup, min_timed_s, max_blocks=2000):
    """Warm up, then time blocks of exactly `steps` steps until `min_timed_s` seconds have been timed;
    returns the median block and what it was taken from."""
    for _ in range(warmup):
        step()
    first = timed_block(ctx, step, steps)
    blocks = [first]
    want = int(min(max_blocks, max(1, -(-min_timed_s * 1e3 // max(first, 1e-6)))))
    for _ in range(want - 1):
        blocks.append(timed_block(ctx, step, steps))
    med = statistics.median(blocks)
    return {"ms_per_step": med / steps, "blocks": len(blocks), "timed_region_s": sum(blocks) * 1e-3,
            "block_ms_min": min(blocks), "block_ms_max": max(blocks)}


def median_ms(ctx, fn, reps=5, warm=2):
    """Median over `reps` single calls (each bracketed like a block), max over ranks per call."""
    for _ in range(warm):
        fn()
    return statistics.median(timed_block(ctx, fn, 1) for _ in range(reps))


def count_library_kernels(step):
    """Kernels of this library (namespace nb200) launched by one call of `step`, counted from the
    profiler's record of the device activity.  None if no record can be had."""
    try:
        from torch.profiler import profile, ProfilerActivity
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        names = [e.name for e in prof.events() if "nb200::" in e.name]
        return len(names) if names else None
    except Exception:
        return None


def relerr(ref, got):
    ref, got = ref.double().flatten(), got.detach().double().cpu().flatten()
    den = torch.linalg.norm(ref).item()
    return torch.linalg.norm(ref - got).item() / (den if den > 0 else 1.0)


def compare(name, ref, got, tol, report):
    """Record how `got` agrees with the oracle's `ref`; returns False beyond `tol`."""
    if ref.shape == got.shape and torch.equal(ref, got.detach().cpu()):
        report[name] = "bit-exact"
        return True
    e = relerr(ref, got) if ref.shape == got.shape else float("inf")
    report[name] = f"relative error {e:.1e}"
    return e <= tol


# -------------------------------------------------------------------------------------------------
# Headline: SpMV forward + backward
# -------------------------------------------------------------------------------------------------
P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731


def raw_stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def single_gpu_spmv(n, dev, ops):
    """Step closures and bookkeeping for one GPU: the C-ABI entry points on resident buffers."""
    from numml_b200 import _cabi, _plan, workloads as W
    import numml_b200.sparse as sp
    d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
    x_h, g_h = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
    A = sp.SparseCSRTensor((d, i, p), (m, k), clone=False).to(dev)
    nnz = A.nnz
    plan = _plan.get_plan(m, k, A.indices, A.indptr)
    idx, ptr, itype = plan.csr()
    transposed = ops.spmv_backward_mode == "transpose"
    t_indptr = t_indices = t_perm = None
    if transposed:
        t_indptr, t_indices, t_perm, _ = plan.transpose()
    x, g = x_h.to(dev), g_h.to(dev)
    y = torch.empty(m, dtype=torch.float64, device=dev)
    grad_A = torch.empty(nnz, dtype=torch.float64, device=dev)
    grad_x = torch.empty(k, dtype=torch.float64, device=dev)
    data = A.data

    pipelined = ops.spmv_kernel == "auto"
    br = plan.spmv_block_rows() if pipelined else 0
    tbr = plan.spmv_block_rows(transposed=True) if (pipelined and transposed) else 0
    sym = int(bool(br) and transposed and plan.pattern_symmetric())
    if sym and ops.spmv_value_symmetry:
        plan.values_symmetric(data)                 # first sighting of these values
        if plan.values_symmetric(data):             # second: the device-side test runs once, its answer is cached
            sym |= 2
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def fwd():
        _cabi.call("nb200_spgemv_forward", m, k, nnz, P(data), P(idx), P(ptr), None, P(x), P(y), br, P(status),
                   _cabi.F64, itype, raw_stream())

    def bwd_with(symmetry):
        def bwd():
            _cabi.call("nb200_spgemv_backward", m, k, nnz, P(data), P(idx), P(ptr), P(x), P(g),
                       P(t_indptr), P(t_indices), P(t_perm), P(grad_A), P(grad_x), br, tbr, symmetry, P(status),
                       _cabi.F64, itype, raw_stream())
        return bwd

    bwd = bwd_with(sym)

    def step_dev():
        fwd()
        bwd()

    # end-to-end through the public API: x and g start in pinned host memory, results end there
    x_pin, g_pin = x_h.pin_memory(), g_h.pin_memory()
    y_pin = torch.empty(m, dtype=torch.float64).pin_memory()
    gx_pin = torch.empty(k, dtype=torch.float64).pin_memory()
    gA_pin = torch.empty(nnz, dtype=torch.float64).pin_memory()
    A.requires_grad = True

    def step_e2e():
        xd = x_pin.to(dev, non_blocking=True).requires_grad_(True)
        gd = g_pin.to(dev, non_blocking=True)
        A.data.grad = None
        yd = A @ xd
        yd.backward(gd)
        y_pin.copy_(yd.detach(), non_blocking=True)
        gx_pin.copy_(xd.grad, non_blocking=True)
        gA_pin.copy_(A.data.grad, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def verify(report):
        oracle = oracle_port()
        y.fill_(float("nan")); grad_A.fill_(float("nan")); grad_x.fill_(float("nan"))
        step_dev()
        torch.cuda.synchronize()
        ok = compare("y", oracle.spgemv_forward(m, k, d, i, p, x_h), y, 0.0, report)
        gA_ref, gx_ref = oracle.spgemv_backward(g_h, m, k, d, i, p, x_h)
        ok &= compare("grad_A", gA_ref, grad_A, 0.0, report)
        ok &= compare("grad_x", gx_ref, grad_x, 0.0, report)
        step_e2e()                                 # the public-API path lands in the pinned buffers
        ok &= compare("e2e_y", oracle.spgemv_forward(m, k, d, i, p, x_h), y_pin, 0.0, report)
        ok &= compare("e2e_grad_A", gA_ref, gA_pin, 0.0, report)
        ok &= compare("e2e_grad_x", gx_ref, gx_pin, 0.0, report)
        return ok

    def kernel_us(f, reps=200):
        for _ in range(10):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def name_of(symmetry):
        if symmetry & 2:
            return "spmv_pipe_kernel mode 4 (one fused pass, pattern and values symmetric)"
        if symmetry & 1:
            return "spmv_pipe_kernel mode 3 (one fused pass, symmetric pattern)"
        return "grad_A pass + grad_x pass over the transposed structure" if transposed else "one pass with atomics"

    def roofline(peak, peak_kind):
        fwd_b, bwd_b = algorithmic_bytes(m, k, nnz, 8, INDEX_BYTES_CREDITED)
        t_f, t_b = kernel_us(fwd), kernel_us(bwd)
        dominant = ("spmv_backward: " + name_of(sym)) if t_b >= t_f else "spmv_forward"
        bytes_, t = (bwd_b, t_b) if t_b >= t_f else (fwd_b, t_f)
        ach = bytes_ / (t * 1e-6) / 1e9
        if t_b >= t_f:
            key = ("spmv_backward_fused_symmetric_values" if sym & 2 else "spmv_backward_fused_symmetric") if sym else \
                  ("spmv_backward_two_pass_stream" if not br else None)
        else:
            key = "spmv_forward_pipelined" if br else "spmv_forward_stream"
        out = {"bound": "hbm", "kernel": dominant, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
               "peak_source": peak_kind + " (copy bandwidth)", "traffic": ncu_traffic(key, nnz) if key else None,
               "launch_us": t, "algorithmic_bytes": bytes_,
               "forward": {"us": t_f, "GBps": fwd_b / (t_f * 1e-6) / 1e9, "frac": fwd_b / (t_f * 1e-6) / 1e9 / peak},
               "backward": {"us": t_b, "GBps": bwd_b / (t_b * 1e-6) / 1e9, "frac": bwd_b / (t_b * 1e-6) / 1e9 / peak,
                            "kernel": name_of(sym)}}
        if sym & 2:
            # the pass a matrix with unsymmetric values takes (same pattern, same bytes credited)
            t_g = kernel_us(bwd_with(1))
            out["backward_general_values"] = {"us": t_g, "GBps": bwd_b / (t_g * 1e-6) / 1e9,
                                              "frac": bwd_b / (t_g * 1e-6) / 1e9 / peak, "kernel": name_of(1)}
        return out

    info = {"nnz": nnz, "rows": m, "cols": k, "status_word": status,
            "kernels": "tma-pipelined" if br else "register-staged", "backward": name_of(sym),
            "schedule": "eager launches", "launches_formula": (2 if sym else 3) if transposed else 2,
            "h2d_bytes": (m + k) * 8, "d2h_bytes": (m + k + nnz) * 8, "roofline": roofline, "verify": verify}
    return step_dev, step_e2e, info


def slab_engine(n, nz_total, ctx, ops, exchange="auto"):
    """A DistSpMVEngine over this rank's slab of the n x n x nz_total grid (z-planes split evenly)."""
    from numml_b200 import distributed as nd, workloads as W
    plane = n * n
    bounds = [plane * ((nz_total * r) // ctx.world) for r in range(ctx.world + 1)]
    lo, hi = bounds[ctx.rank], bounds[ctx.rank + 1]
    d, i, p, _ = W.poisson3d_7pt(n, torch.float64, nz=nz_total, row_range=(lo, hi))
    A = nd.DistSparseCSR(d.to(ctx.dev), i.to(ctx.dev), p.to(ctx.dev), (plane * nz_total,) * 2, bounds, ops=ops)
    return nd.DistSpMVEngine(A, exchange=exchange), A, bounds, (d, i, p)


def checked_slab_engine(n, nz_total, ctx, ops, x_seed, g_seed):
    """slab_engine whose first step has been compared with the oracle on every rank.  The peer-memory
    exchange is tried first; if a step over it does not reproduce the oracle (or a wait runs out) on any
    rank, every rank falls back to the NCCL exchange together and the check is repeated.  Returns
    (engine, A, bounds, csr, report) or raises SystemExit when neither exchange verifies."""
    report = {}
    for exchange in ("auto", "nccl"):
        engine, A, bounds, csr = slab_engine(n, nz_total, ctx, ops, exchange)
        engine.set_inputs(slab_vectors(bounds, ctx.rank, x_seed).to(ctx.dev), slab_vectors(bounds, ctx.rank, g_seed).to(ctx.dev))
        report = {}
        ok = verify_slab(ctx, n, nz_total, bounds, engine, x_seed, g_seed, report)
        ok = ok and int(engine.status.item()) == 0
        if ctx.all_true(ok):
            return engine, A, bounds, csr, report
        print(f"rank {ctx.rank}: a step with exchange {engine.exchange!r} does not match the oracle: {report}", file=sys.stderr)
        was_peer = engine.peer is not None
        engine.status.zero_()
        engine.close()
        if not was_peer:
            break
    raise SystemExit(f"rank {ctx.rank}: one step does not match the CPU oracle: {report}")


def slab_vectors(bounds, rank, seed_base):
    """This rank's block of a global vector whose blocks are seeded per rank (so that any rank can
    rebuild a neighbour's block for checking)."""
    from numml_b200 import workloads as W
    return W.randn(bounds[rank + 1] - bounds[rank], seed_base + rank, torch.float64)


def verify_slab(ctx, n, nz_total, bounds, engine, x_seed, g_seed, report):
    """One engine step against the oracle run on this rank's rows plus one plane of rows on either side
    (every row that contributes to the rank's block of grad_x), with the neighbours' blocks of x and g
    rebuilt from their seeds."""
    from numml_b200 import workloads as W
    oracle = oracle_port()
    plane, total = n * n, n * n * nz_total
    lo, hi = bounds[ctx.rank], bounds[ctx.rank + 1]
    a, b = max(0, lo - plane), min(total, hi + plane)
    d, i, p, _ = W.poisson3d_7pt(n, torch.float64, nz=nz_total, row_range=(a, b))
    xg, gg = torch.zeros(total, dtype=torch.float64), torch.zeros(total, dtype=torch.float64)
    for r in range(max(0, ctx.rank - 1), min(ctx.world, ctx.rank + 2)):
        xg[bounds[r]:bounds[r + 1]] = slab_vectors(bounds, r, x_seed)
        gg[bounds[r]:bounds[r + 1]] = slab_vectors(bounds, r, g_seed)
    y_ref = oracle.spgemv_forward(b - a, total, d, i, p, xg)[lo - a:hi - a]
    gA_all, gx_all = oracle.spgemv_backward(gg[a:b].contiguous(), b - a, total, d, i, p, xg)
    ea, eb = int(p[lo - a]), int(p[hi - a])
    engine.y.fill_(float("nan")); engine.grad_A.fill_(float("nan"))
    ctx.barrier()                                  # the ranks step together: a neighbour's wait is bounded
    engine.step()
    torch.cuda.synchronize()
    ok = compare("y", y_ref, engine.y, 0.0, report)
    ok &= compare("grad_A", gA_all[ea:eb], engine.grad_A, 0.0, report)
    # partial sums from the neighbours are added after the local ones: same terms, another order
    ok &= compare("grad_x", gx_all[lo:hi], engine.grad_x, 1e-12, report)
    return ok


def multi_gpu_spmv(n, ctx, ops, nz_total=None):
    """Step closures for N > 1: every rank owns a slab of the n x n x nz_total grid (default: n planes
    per rank, i.e. one n^3 slab each).  The engine comes back verified against the oracle."""
    nz_total = n * ctx.world if nz_total is None else nz_total
    engine, A, bounds, (d, i, p), verified = checked_slab_engine(n, nz_total, ctx, ops, 100, 200)
    rows = bounds[ctx.rank + 1] - bounds[ctx.rank]
    x_h, g_h = slab_vectors(bounds, ctx.rank, 100), slab_vectors(bounds, ctx.rank, 200)
    A.requires_grad = True
    step_dev, mode = engine.step, engine.schedule
    if os.environ.get("NB200_BENCH_GRAPH", "1") == "1":
        try:
            ctx.barrier()
            step_dev, mode = engine.capture(), engine.schedule + ", one CUDA graph per step"
        except Exception as e:          # capture is an optimisation; the eager schedule is always valid
            print(f"rank {ctx.rank}: CUDA graph capture failed ({type(e).__name__}: {e}); running eager launches", file=sys.stderr)
            step_dev = engine.step
    captured = ctx.all_true(step_dev is not engine.step)
    if not captured:                    # every rank runs the same schedule
        step_dev, mode = engine.step, engine.schedule

    x_pin, g_pin = x_h.pin_memory(), g_h.pin_memory()
    y_pin = torch.empty(rows, dtype=torch.float64).pin_memory()
    gx_pin = torch.empty(rows, dtype=torch.float64).pin_memory()
    gA_pin = torch.empty(d.numel(), dtype=torch.float64).pin_memory()
    dev = ctx.dev

    def step_e2e():
        xd = x_pin.to(dev, non_blocking=True).requires_grad_(True)
        gd = g_pin.to(dev, non_blocking=True)
        A.data.grad = None
        yd = A @ xd
        yd.backward(gd)
        y_pin.copy_(yd.detach(), non_blocking=True)
        gx_pin.copy_(xd.grad, non_blocking=True)
        gA_pin.copy_(A.data.grad, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def verify(report):
        report.update(verified)
        return True

    info = {"nnz": int(d.numel()), "rows": rows, "cols": engine.n_ext, "status_word": engine.status, "schedule": mode,
            "kernels": ("tma-pipelined, fused backward over ghost rows" if engine.fused else "tma-pipelined") if engine.br else "register-staged",
            "backward": ("spmv_pipe_kernel over the ghost-row extension: local rows mode "
                         + ("4 (pattern and values symmetric)" if engine.values_symmetric else "3 (symmetric pattern)")
                         + ", ghost rows mode 3") if engine.fused else "grad_A pass + transposed pass",
            "launches_formula": engine.launches_per_step, "exchange": engine.exchange,
            "h2d_bytes": 2 * rows * 8, "d2h_bytes": (2 * rows + int(d.numel())) * 8, "roofline": None, "verify": verify,
            "engine": engine}
    return step_dev, step_e2e, info


# -------------------------------------------------------------------------------------------------
# Extras: the other partitioned operators, on the same N GPUs
# -------------------------------------------------------------------------------------------------
def extra_strong(ctx, ops, n, peak, steps, min_timed_s):
    """The fixed n^3 matrix split N ways (north-star C2 as stated): SpMV forward + backward."""
    if ctx.world == 1:
        return None                                # identical to the headline at one GPU
    if n % ctx.world != 0:
        return {"skipped": f"{n} planes do not split evenly over {ctx.world} ranks"}
    step_dev, _, info = multi_gpu_spmv(n, ctx, ops, nz_total=n)
    report = {}
    info["verify"](report)
    t = timed_blocks(ctx, step_dev, steps, 5, min_timed_s)
    rows, nnz = n ** 3, 7 * n ** 3 - 6 * n ** 2
    fwd_b, bwd_b = algorithmic_bytes(rows, rows, nnz, 8, INDEX_BYTES_CREDITED)
    gbs = (fwd_b + bwd_b) / (t["ms_per_step"] * 1e-3) / 1e9
    try:
        phases = info["engine"].phase_times()
    except Exception as e:  # the timing above stands without the breakdown
        phases = {"error": f"{type(e).__name__}: {e}"}
    info["engine"].close()
    return {"workload": f"poisson3d_7pt_{n}^3_fp64 split over {ctx.world} GPUs", "ms_per_step": t["ms_per_step"], "GBps": gbs,
            "frac_of_aggregate_peak": gbs / (peak * ctx.world), "blocks": t["blocks"], "schedule": info["schedule"],
            "exchange": info["exchange"], "phases_us": phases, "verified": report}


def extra_cg(ctx, ops, n, peak):
    """100 unpreconditioned CG iterations on the fixed n^3 matrix (b ~ N(0,1), x0 = 0, rtol = 0), split
    N ways; the residual history is compared with the reference's recurrence on the oracle SpMV."""
    from numml_b200 import workloads as W
    iters = 100
    rows, nnz = n ** 3, 7 * n ** 3 - 6 * n ** 2
    b_h = W.randn(rows, 2, torch.float64)
    if ctx.world == 1:
        import numml_b200.sparse as sp
        import numml_b200.krylov as kry
        d, i, p, _ = W.poisson3d_7pt(n, torch.float64)
        A = sp.SparseCSRTensor((d, i, p), (rows, rows), clone=False).to(ctx.dev)
        b = b_h.to(ctx.dev)
        solve = lambda: kry.conjugate_gradient(A, b, rtol=0.0, iterations=iters)  # noqa: E731
        how = "in-library loop: 1 SpMV + 3 fused vector kernels per iteration, scalars on the device"
    else:
        from numml_b200 import distributed as nd
        if n % ctx.world != 0:
            return {"skipped": f"{n} planes do not split evenly over {ctx.world} ranks"}
        engine, A, bounds, _, _ = checked_slab_engine(n, n, ctx, ops, 100, 200)
        b = b_h[bounds[ctx.rank]:bounds[ctx.rank + 1]].to(ctx.dev)
        solver = nd.DistCG(engine)
        solve = lambda: solver.solve(b, iters)  # noqa: E731
        how = solver.schedule
    x, hist = solve()
    torch.cuda.synchronize()
    report, ok = {}, True
    if ctx.rank == 0:
        oracle = oracle_port()
        d, i, p, _ = W.poisson3d_7pt(n, torch.float64)
        xr, r = torch.zeros(rows, dtype=torch.float64), b_h.clone()
        pv, rz = r.clone(), torch.dot(r, r)
        ref = [torch.sqrt(rz)]
        for _ in range(iters):
            Ap = oracle.spgemv_forward(rows, rows, d, i, p, pv)
            alpha = rz / torch.dot(Ap, pv)
            xr += alpha * pv
            r -= alpha * Ap
            rz_new = torch.dot(r, r)
            pv = r + (rz_new / rz) * pv
            rz = rz_new
            ref.append(torch.sqrt(rz))
        ok = compare("residual_history_101", torch.stack(ref), hist, 1e-8, report)
        report["tolerance"] = "1e-8 (dot products reduced in another order than on the CPU)"
    if not ctx.all_true(ok):
        if ctx.world > 1:
            engine.close()
        return {"error": "mismatch against the oracle recurrence", "verified": report}
    ms = median_ms(ctx, solve, reps=5, warm=1)
    if ctx.world > 1:
        engine.close()
    fwd_b, _ = algorithmic_bytes(rows, rows, nnz, 8, INDEX_BYTES_CREDITED)
    bytes_ = iters * (fwd_b + 7 * rows * 8)
    return {"workload": f"100 CG iterations, poisson3d_7pt_{n}^3_fp64" + (f" split over {ctx.world} GPUs" if ctx.world > 1 else ""),
            "cg100_ms": ms, "us_per_iteration": ms * 1e3 / iters, "GBps": bytes_ / (ms * 1e-3) / 1e9,
            "frac_of_aggregate_peak": bytes_ / (ms * 1e-3) / 1e9 / (peak * ctx.world),
            "algorithmic_bytes": "SpMV forward + 7 vector passes per iteration", "schedule": how, "verified": report}


def extra_spgemm(ctx, ops, n, peak):
    """C = A A on the 2-D Poisson n^2 grid, rows split evenly over the ranks; rows of A that a rank's
    columns refer to are fetched from their owners.  Output nnz per second over the whole product."""
    from numml_b200 import workloads as W
    m = n * n
    bounds = [(m * r) // ctx.world for r in range(ctx.world + 1)]
    lo, hi = bounds[ctx.rank], bounds[ctx.rank + 1]
    d, i, p, _ = W.poisson2d_5pt(n, torch.float64, row_range=(lo, hi))
    dd, di, dp = d.to(ctx.dev), i.to(ctx.dev), p.to(ctx.dev)
    if ctx.world == 1:
        fwd = lambda: ops.spgemm_forward(m, m, dd, di, dp, m, m, dd, di, dp)  # noqa: E731
        C = fwd()
        gC = torch.randn(C[0].numel(), dtype=torch.float64, device=ctx.dev, generator=torch.Generator(ctx.dev).manual_seed(0))
        bwd = lambda: ops.spgemm_backward(gC, C[1], C[2], m, m, dd, di, dp, m, m, dd, di, dp)  # noqa: E731
        how = "single GPU"
    else:
        from numml_b200 import distributed as nd
        A = nd.DistSparseCSR(dd, di, dp, (m, m), bounds, ops=ops)
        A.requires_grad = True
        fwd = lambda: nd.dist_spgemm(A, A)  # noqa: E731
        C = fwd()
        gC = torch.randn(C[0].numel(), dtype=torch.float64, device=ctx.dev, generator=torch.Generator(ctx.dev).manual_seed(ctx.rank))

        def bwd():
            A.data.grad = None
            Cd, _, _ = nd.dist_spgemm(A, A)
            Cd.backward(gC)
        how = "rows of the right factor fetched point to point (lengths, then indices + values)"
    torch.cuda.synchronize()
    # oracle check: the first and last 2048 rows of this rank's block against the full right factor
    oracle = oracle_port()
    report = {}
    fd, fi, fp, _ = W.poisson2d_5pt(n, torch.float64)
    take = min(2048, hi - lo)
    sample = torch.unique(torch.cat((torch.arange(take), torch.arange(hi - lo - take, hi - lo))))
    sd, si, sp_, _ = W.rows_subset(d, i, p, sample)
    ref = oracle.spgemm_forward(sample.numel(), m, sd, si, sp_, m, m, fd, fi, fp)
    Cd, Ci, Cp = [t.cpu() for t in C[:3]]
    gd_, gi_, gp_, _ = W.rows_subset(Cd, Ci, Cp, sample)
    ok = compare("C_indptr_rows", ref[2], gp_, 0.0, report)
    ok &= compare("C_indices_rows", ref[1], gi_, 0.0, report)
    ok &= compare("C_values_rows", ref[0], gd_, 0.0, report)
    report["sample"] = f"{sample.numel()} rows per rank (first and last of the block)"
    if not ctx.all_true(ok):
        return {"error": "mismatch against the oracle", "verified": report}
    nnz_c = ctx.sum_over_ranks(float(C[0].numel()))
    # the whole product (planning, symbolic and numeric phases) with nothing kept from an earlier call, then the
    # same product again with the symbolic phase's results kept by the library (its default: numeric phase only)
    keep = ops.spgemm_keep_symbolic
    ops.spgemm_keep_symbolic = False
    try:
        t_f = median_ms(ctx, fwd, reps=7, warm=2)
    finally:
        ops.spgemm_keep_symbolic = keep
    t_rep = median_ms(ctx, fwd, reps=7, warm=2)
    if ctx.world == 1:
        t_b = median_ms(ctx, bwd, reps=5, warm=1)
    else:
        t_fb = median_ms(ctx, bwd, reps=5, warm=1)
        t_b = max(t_fb - t_rep, 0.0)               # its forward is a repeat of the same patterns
    nnz_a = 5 * n * n - 4 * n
    s, w = 8, INDEX_BYTES_CREDITED
    fwd_bytes = 2 * nnz_a * (s + w) + nnz_c * (s + 8) + 3 * (m + 1) * 8
    return {"workload": f"A*A, poisson2d_5pt_{n}^2_fp64" + (f" split over {ctx.world} GPUs" if ctx.world > 1 else ""),
            "out_nnz": int(nnz_c), "forward_ms": t_f, "spgemm_out_nnz_per_s": nnz_c / (t_f * 1e-3),
            "forward_GBps": fwd_bytes / (t_f * 1e-3) / 1e9, "frac_of_aggregate_peak": fwd_bytes / (t_f * 1e-3) / 1e9 / (peak * ctx.world),
            "algorithmic_bytes": "read A and B once, write C (int64 indices), three row-pointer arrays",
            "repeat_forward_ms": t_rep, "repeat_spgemm_out_nnz_per_s": nnz_c / (t_rep * 1e-3),
            "repeat": "the same patterns with the symbolic phase's results kept from the previous call: numeric phase and allocation of C only",
            "backward_ms": t_b, "includes": "planning, symbolic and numeric phases, allocation of C, one host read of nnz(C)"
                                            + ("; the fetch of remote rows" if ctx.world > 1 else ""),
            "exchange": how, "verified": report}


def extra_spmm(ctx, ops, n, K, peak):
    """Y = A X on the power-law graph, fp32, rows of A (and of X, Y) split by nonzero count."""
    from numml_b200 import workloads as W
    d, i, p, _ = W.powerlaw_graph(n, dtype=torch.float32)
    nnz_total = int(d.numel())
    dev = ctx.dev
    gen = torch.Generator(dev).manual_seed(0)
    X_full = torch.randn((n, K), dtype=torch.float32, device=dev, generator=gen)     # the same on every rank
    report = {}
    oracle = oracle_port()
    rng_rows = torch.from_numpy(__import__("numpy").random.default_rng(7).choice(n, 4096, replace=False)).sort().values
    s, w = 4, INDEX_BYTES_CREDITED
    if ctx.world == 1:
        dd, di, dp = d.to(dev), i.to(dev), p.to(dev)
        G = torch.randn((n, K), dtype=torch.float32, device=dev, generator=gen)
        fwd = lambda: ops.spdmm_forward(n, n, dd, di, dp, X_full)  # noqa: E731
        bwd = lambda: ops.spdmm_backward(n, n, dd, di, dp, X_full, G)  # noqa: E731
        Y = fwd()
        rows_here, row0 = rng_rows, 0
        bounds = [0, n]
        exchanged = 0
        fwd_local = bwd_local = None
        how = "single GPU"
    else:
        from numml_b200 import distributed as nd
        bounds = nd.partition_rows(n, ctx.world, indptr=p)
        lo, hi = bounds[ctx.rank], bounds[ctx.rank + 1]
        bd, bi, bp = W.row_block(d, i, p, lo, hi)
        A = nd.DistSparseCSR(bd.to(dev), bi.to(dev), bp.to(dev), (n, n), bounds, ops=ops)
        A.requires_grad = True
        X_loc = X_full[lo:hi].clone().requires_grad_(True)
        G = torch.randn((hi - lo, K), dtype=torch.float32, device=dev, generator=torch.Generator(dev).manual_seed(10 + ctx.rank))
        fwd = lambda: A @ X_loc.detach()  # noqa: E731

        def bwd():
            A.data.grad = None
            X_loc.grad = None
            (A @ X_loc).backward(G)
        Y = fwd()
        rows_here, row0 = rng_rows[(rng_rows >= lo) & (rng_rows < hi)], lo
        halo = A.halo
        exchanged = halo.n_halo * K * s                   # bytes this rank receives per forward
        n_ext = halo.n_local + halo.n_halo
        X_ext = halo.extend(X_loc.detach())
        fwd_local = lambda: ops.spdmm_forward(A.n_rows, n_ext, A.data.detach(), A.indices, A.indptr, X_ext)  # noqa: E731
        bwd_local = lambda: ops.spdmm_backward(A.n_rows, n_ext, A.data.detach(), A.indices, A.indptr, X_ext, G)  # noqa: E731
        rows = getattr(halo, "_row_exchanges", {}).get((torch.float32, K))
        if rows is not None:
            how = ("peer memory: every rank publishes its block of dense rows once, neighbours gather the rows they need over "
                   "NVLink with this library's kernels; partial gradient rows added by their owners in peer order; no NCCL call")
        else:
            how = "dense rows packed per peer and sent point to point; gradient rows sent back and added in peer order"
    torch.cuda.synchronize()
    ok = True
    if rows_here.numel() > 0:
        sd, si, sp_, _ = W.rows_subset(d, i, p, rows_here)
        cols, inv = torch.unique(si, return_inverse=True)
        Y_ref = oracle.spdmm_forward(rows_here.numel(), cols.numel(), sd, inv.contiguous(), sp_, X_full[cols.to(dev)].cpu())
        ok = compare("Y_rows", Y_ref, Y[(rows_here - row0).to(dev)], 0.0, report)
    report["sample"] = "4096 random rows of the graph, each checked by the rank that owns it"
    if ctx.world > 1:
        X_full = None                               # only this rank's block (a copy) is used from here on
    if not ctx.all_true(ok):
        return {"error": "mismatch against the oracle", "verified": report}
    t_f = median_ms(ctx, fwd, reps=5, warm=2)
    if ctx.world == 1:
        t_b = median_ms(ctx, bwd, reps=5, warm=1)
    else:
        t_b = max(median_ms(ctx, bwd, reps=5, warm=1) - t_f, 0.0)
    out = {"workload": f"powerlaw graph {n} nodes, {nnz_total} nnz, K={K}, fp32" + (f" split by nnz over {ctx.world} GPUs" if ctx.world > 1 else ""),
           "forward_ms": t_f, "backward_ms": t_b, "exchange": how, "verified": report}
    compulsory = nnz_total * (s + w) + (n + 1) * w + 2 * n * K * s
    gather = nnz_total * K * s + n * K * s + nnz_total * (s + w)
    bwd_bytes = nnz_total * (s + w) + 3 * n * K * s + nnz_total * s
    out["forward_GBps_compulsory"] = compulsory / (t_f * 1e-3) / 1e9
    out["forward_frac_compulsory"] = out["forward_GBps_compulsory"] / (peak * ctx.world)
    out["forward_GBps_gather_model"] = gather / (t_f * 1e-3) / 1e9
    out["forward_frac_gather_model"] = out["forward_GBps_gather_model"] / (peak * ctx.world)
    out["backward_GBps_compulsory"] = bwd_bytes / (t_b * 1e-3) / 1e9 if t_b > 0 else None
    if ctx.world > 1:
        t_fl = median_ms(ctx, fwd_local, reps=5, warm=2)
        t_bl = median_ms(ctx, bwd_local, reps=5, warm=1)
        recv = ctx.max_over_ranks(float(exchanged))
        out.update({"forward_ms_without_exchange": t_fl, "backward_ms_without_exchange": t_bl,
                    "exchanged_bytes_per_rank_max": int(recv), "exchanged_bytes_total": int(ctx.sum_over_ranks(float(exchanged))),
                    "nvlink_bound_ms": recv / 770e9 * 1e3,
                    "nvlink_bound": "bytes a rank must receive / 770 GB/s (measured peer copy bandwidth per direction)",
                    "exchange_frac_of_nvlink_bound": (recv / 770e9 * 1e3) / max(t_f - t_fl, 1e-9)})
    return out


def run_extras(ctx, ops, args, peak):
    extras = {}
    plan = [("strong", lambda: extra_strong(ctx, ops, args.grid, peak, args.steps, args.min_timed_s)),
            ("cg", lambda: extra_cg(ctx, ops, args.grid, peak)),
            ("spgemm", lambda: extra_spgemm(ctx, ops, args.spgemm_grid, peak)),
            ("spmm", lambda: extra_spmm(ctx, ops, args.graph_nodes, 128, peak))]
    for name, fn in plan:
        try:
            out = fn()
        except Exception as e:  # an extra must not take the headline down with it
            import traceback
            traceback.print_exc(file=sys.stderr)
            out = {"error": f"{type(e).__name__}: {e}"}
        if out is not None:
            extras[name] = out
        torch.cuda.empty_cache()
        if ctx.dist is not None:
            # every rank moves on together, whatever happened on any of them
            ctx.barrier()
    return extras


# -------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--grid", type=int, default=128, help="grid extent n (the workload is n^3 rows per GPU)")
    ap.add_argument("--spgemm-grid", type=int, default=2048, help="grid extent of the SpGEMM extra")
    ap.add_argument("--graph-nodes", type=int, default=4194304, help="nodes of the SpMM extra's graph")
    ap.add_argument("--backward", default=None, choices=["transpose", "atomic"])
    ap.add_argument("--spmv-kernel", default=None, choices=["auto", "stream"])
    ap.add_argument("--general-values", action="store_true", help="do not use the value-symmetric backward pass")
    ap.add_argument("--min-timed-s", type=float, default=0.5, help="repeat the K-step block until this much has been timed")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # a bounded collective timeout: a rank that fails must not leave the others waiting for long
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    from numml_b200 import numml_torch_cpp as ops
    if args.backward:
        ops.spmv_backward_mode = args.backward
    if args.spmv_kernel:
        ops.spmv_kernel = args.spmv_kernel
    if args.general_values:
        ops.spmv_value_symmetry = False

    ctx = Ctx(rank, world, dev, dist)
    peak, peak_kind = load_peaks()
    result = run(args, ctx, ops, peak, peak_kind)
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run(args, ctx, ops, peak, peak_kind):
    n, K, Wm = args.grid, args.steps, args.warmup
    if ctx.world == 1:
        step_dev, step_e2e, info = single_gpu_spmv(n, ctx.dev, ops)
    else:
        step_dev, step_e2e, info = multi_gpu_spmv(n, ctx, ops)
    nnz, m = info["nnz"], info["rows"]
    fwd_b, bwd_b = algorithmic_bytes(m, m, nnz, 8, INDEX_BYTES_CREDITED)
    bytes_per_step = (fwd_b + bwd_b) * ctx.world  # every rank moves the same amount (weak scaling)

    verified = {}
    if not ctx.all_true(info["verify"](verified)):
        raise SystemExit(f"rank {ctx.rank}: one step does not match the CPU oracle: {verified}")

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else 0)
    if ctx.rank == 0:
        sampler.start()
    t_dev = timed_blocks(ctx, step_dev, K, Wm, args.min_timed_s)
    clocks = sampler.stop() if ctx.rank == 0 else None
    e2e_steps = max(3, min(K, 20))
    t_e2e = None if args.no_e2e else timed_blocks(ctx, step_e2e, e2e_steps, 3, 0.0)

    if info.get("status_word") is not None and int(info["status_word"].item()) != 0:
        raise SystemExit("a bounded device-side wait ran out during the benchmark; results are invalid")
    per_step = count_library_kernels(step_dev)
    counted = per_step is not None
    if not counted:
        per_step = info["launches_formula"]
    value = bytes_per_step / (t_dev["ms_per_step"] * 1e-3) / 1e9

    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": ctx.world, "steps": K, "warmup": Wm,
        "ms_per_step": t_dev["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": workload_config(n, m, nnz),
        "timing": {"blocks_of_K_steps": t_dev["blocks"], "reported": "median block", "timed_region_s": t_dev["timed_region_s"],
                   "block_ms_min": t_dev["block_ms_min"], "block_ms_max": t_dev["block_ms_max"]},
        "details": {"index_bytes_read": 4, "kernels": info.get("kernels"), "backward": info.get("backward"),
                    "schedule": info.get("schedule"), "exchange": info.get("exchange"),
                    "partition": "z-slabs, one halo plane per neighbour" if ctx.world > 1 else "single GPU"},
        "verified": verified,
        "gpu_launches": per_step * K * t_dev["blocks"],
        "gpu_launches_per_step": per_step,
        "gpu_launches_how": "kernels of this library in the profiler's record of one step" if counted else "launch schedule (no profiler record)",
        "clocks": clocks,
    }
    if t_e2e is not None:
        result["e2e"] = {"value": bytes_per_step / (t_e2e["ms_per_step"] * 1e-3) / 1e9, "unit": UNIT,
                         "ms_per_step": t_e2e["ms_per_step"],
                         "h2d_bytes_per_step": info["h2d_bytes"] * ctx.world, "d2h_bytes_per_step": info["d2h_bytes"] * ctx.world,
                         "steps": e2e_steps}
    if ctx.world == 1:
        result["roofline"] = info["roofline"](peak, peak_kind)
        if not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(n)
    engine = info.pop("engine", None)
    if engine is not None:
        engine.close()
    if not args.no_extras:
        result["extra"] = run_extras(ctx, ops, args, peak)
    return result


if __name__ == "__main__":
    main()
