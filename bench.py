"""Benchmark of the differentiable-CSR hot path on B200.

One step = SpMV forward (y = A x) followed by SpMV backward (grad_A.data = g_i x_j on the
pattern, grad_x = A^T g) on the 3-D Poisson 7-point Laplacian of a 128^3 grid in fp64
(2,097,152 rows, 14,581,760 nonzeros).  With N > 1 GPUs every rank owns one 128^3 slab of a
128 x 128 x 128N grid (row-block partition, weak scaling) and exchanges one 128^2 halo plane
of x (forward) and of the grad_x partial sums (backward) with each z-neighbour over NCCL.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--grid n]

Prints ONE JSON line (rank 0).  `value` is effective GB/s over the whole job with everything
resident in HBM: algorithmic bytes of forward + backward (index width as read by the kernels)
divided by the CUDA-event time of the K steps, max over ranks.  `e2e` is the same metric
through the public SparseCSRTensor API with x and g starting in pinned host memory and y,
grad_x, grad_A copied back to the host inside the timed region (the matrix stays resident, as
it does for a reference user after `A.to(device)`).  `--impl reference` times the reference's
own CPU implementation (oracle/_ref, else the C port) on the host cores.
"""
import argparse
import ctypes
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


def algorithmic_bytes(rows, cols, nnz, s, w):
    """Bytes that forward and backward must move (value size s, index size w)."""
    fwd = nnz * (s + w) + (rows + 1) * w + cols * s + rows * s
    bwd = nnz * (s + w) + (rows + 1) * w + cols * s + rows * s + nnz * s + cols * s
    return fwd, bwd


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


def reference_arm(args, rank, world):
    """The reference's CPU implementation of the same step on the host cores (rank 0 only)."""
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from numml_b200 import workloads as W
    kind = "reference"
    try:
        import build_ref
        mod = build_ref.load()
    except ImportError:
        import csr_oracle as mod
        mod.build()
        kind = "port"
    torch.set_num_threads(1)  # the reference CPU kernels are serial loops (its own protocol: demos/timing.py:15)
    n = args.grid
    d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
    x, g = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
    nnz = d.numel()
    fwd_b, bwd_b = algorithmic_bytes(m, k, nnz, 8, 8)  # the reference reads int64 indices

    def step():
        mod.spgemv_forward(m, k, d, i, p, x)
        mod.spgemv_backward(g, m, k, d, i, p, x)

    for _ in range(min(args.warmup, 3)):
        step()
    steps = max(1, min(args.steps, 60))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = (fwd_b + bwd_b) * steps / dt / 1e9
    sample = f"{steps} full steps (forward+backward) of the {n}^3 workload, 1 thread"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"poisson3d_7pt_{n}^3_fp64_spmv_fwd_bwd", "rows": m, "nnz": nnz, "index_bytes": 8},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample,
                         "host_cores": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline(n, budget_s=12.0):
    """Reference CPU path on a bounded sample of the same workload (rank 0, N=1 only)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from numml_b200 import workloads as W
    kind = "reference"
    try:
        import build_ref
        mod = build_ref.load()
    except ImportError:
        import csr_oracle as mod
        mod.build()
        kind = "port"
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
    x, g = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
    fwd_b, bwd_b = algorithmic_bytes(m, k, d.numel(), 8, 8)
    mod.spgemv_forward(m, k, d, i, p, x)
    mod.spgemv_backward(g, m, k, d, i, p, x)
    steps, t0 = 0, time.perf_counter()
    while True:
        mod.spgemv_forward(m, k, d, i, p, x)
        mod.spgemv_backward(g, m, k, d, i, p, x)
        steps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or steps >= 100:
            break
    torch.set_num_threads(threads)
    return {"value": (fwd_b + bwd_b) * steps / dt / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
            "ms_per_step": dt / steps * 1e3, "host_cores": os.cpu_count(),
            "sample": f"{steps} full steps (forward+backward) of the {n}^3 workload, 1 thread"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--grid", type=int, default=128, help="grid extent n (the workload is n^3 rows per GPU)")
    ap.add_argument("--backward", default=None, choices=["transpose", "atomic"])
    ap.add_argument("--spmv-kernel", default=None, choices=["auto", "stream"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a bounded collective timeout: a rank that fails must not leave the others waiting for long
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    from numml_b200 import numml_torch_cpp as ops
    if args.backward:
        ops.spmv_backward_mode = args.backward
    if args.spmv_kernel:
        ops.spmv_kernel = args.spmv_kernel

    n = args.grid
    peak, peak_kind = load_peaks()

    result = run(args, rank, world, dev, dist, n, peak, peak_kind)
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run(args, rank, world, dev, dist, n, peak, peak_kind):
    from numml_b200 import _cabi, _plan, numml_torch_cpp as ops, workloads as W
    import numml_b200.sparse as sp

    K, Wm = args.steps, args.warmup
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
    P = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731

    if world == 1:
        d, i, p, (m, k) = W.poisson3d_7pt(n, torch.float64)
        x_h, g_h = W.randn(k, 0, torch.float64), W.randn(m, 1, torch.float64)
        A = sp.SparseCSRTensor((d, i, p), (m, k), clone=False).to(dev)
        step_dev, step_e2e, info = single_gpu_steps(A, x_h, g_h, dev, ops, _plan, _cabi, P, stream)
    else:
        from numml_b200 import distributed as nd
        step_dev, step_e2e, info = nd.bench_steps(n, rank, world, dev, ops)

    nnz, m, k, w = info["nnz"], info["rows"], info["cols"], info["index_bytes"]
    fwd_b, bwd_b = algorithmic_bytes(m, k, nnz, 8, w)
    bytes_per_step = (fwd_b + bwd_b) * world  # every rank moves the same amount (weak scaling)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step, steps, warm):
        for _ in range(warm):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        barrier()
        return ms

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else 0)
    if rank == 0:
        sampler.start()
    ms_dev = timed(step_dev, K, Wm)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(step_e2e, max(3, min(K, 20)), 3)
    e2e_steps = max(3, min(K, 20))

    if info.get("status_word") is not None and int(info["status_word"].item()) != 0:
        raise SystemExit("a bounded device-side wait ran out during the benchmark; results are invalid")
    value = bytes_per_step * K / (ms_dev * 1e-3) / 1e9
    e2e_value = bytes_per_step * e2e_steps / (ms_e2e * 1e-3) / 1e9

    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"poisson3d_7pt_{n}^3_per_gpu_fp64_spmv_fwd_bwd", "rows_per_gpu": m, "nnz_per_gpu": nnz,
                   "index_bytes": w, "backward": ops.spmv_backward_mode, "kernels": info.get("kernels"), "schedule": info.get("schedule", "eager launches"),
                   "partition": "z-slabs, one halo plane per neighbour" if world > 1 else "single GPU",
                   "l2": "working set per step (>= 350 MB) is larger than the 126 MB L2; no explicit flush"},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / e2e_steps,
                "h2d_bytes_per_step": info["h2d_bytes"] * world, "d2h_bytes_per_step": info["d2h_bytes"] * world,
                "steps": e2e_steps},
        "gpu_launches": info["launches_per_step"] * K,
        "clocks": clocks,
    }
    if world == 1 and rank == 0:
        result["roofline"] = info["roofline"](peak, peak_kind)
        if not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(n)
    return result


def single_gpu_steps(A, x_h, g_h, dev, ops, _plan, _cabi, P, stream):
    m, k = A.shape
    nnz = A.nnz
    plan = _plan.get_plan(m, k, A.indices, A.indptr)
    idx, ptr, itype = plan.csr()
    w = 4 if itype == _cabi.I32 else 8
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
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def fwd():
        _cabi.call("nb200_spgemv_forward", m, k, nnz, P(data), P(idx), P(ptr), None, P(x), P(y), br, P(status),
                   _cabi.F64, itype, stream())

    def bwd():
        _cabi.call("nb200_spgemv_backward", m, k, nnz, P(data), P(idx), P(ptr), P(x), P(g),
                   P(t_indptr), P(t_indices), P(t_perm), P(grad_A), P(grad_x), br, tbr, sym, P(status),
                   _cabi.F64, itype, stream())

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

    def kernel_us(f, reps=100):
        for _ in range(5):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def roofline(peak, peak_kind):
        fwd_b, bwd_b = algorithmic_bytes(m, k, nnz, 8, w)
        t_f, t_b = kernel_us(fwd), kernel_us(bwd)
        bwd_name = "spmv_backward (one fused pass, symmetric pattern)" if sym else "spmv_backward (grad_A pass + grad_x pass)"
        dominant = bwd_name if t_b >= t_f else "spmv_forward"
        bytes_, t = (bwd_b, t_b) if t_b >= t_f else (fwd_b, t_f)
        ach = bytes_ / (t * 1e-6) / 1e9
        if t_b >= t_f:
            key = "spmv_backward_fused_symmetric" if sym else ("spmv_backward_two_pass_stream" if not br else None)
        else:
            key = "spmv_forward_pipelined" if br else "spmv_forward_stream"
        return {"bound": "hbm", "kernel": dominant, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "peak_source": peak_kind + " (copy bandwidth)", "traffic": ncu_traffic(key, nnz) if key else None,
                "launch_us": t, "algorithmic_bytes": bytes_,
                "forward": {"us": t_f, "GBps": fwd_b / (t_f * 1e-6) / 1e9, "frac": fwd_b / (t_f * 1e-6) / 1e9 / peak},
                "backward": {"us": t_b, "GBps": bwd_b / (t_b * 1e-6) / 1e9, "frac": bwd_b / (t_b * 1e-6) / 1e9 / peak}}

    info = {"nnz": nnz, "rows": m, "cols": k, "index_bytes": w, "kernels": "tma-pipelined" if br else "register-staged",
            "status_word": status,
            "launches_per_step": (2 if sym else 3) if transposed else 2,
            "h2d_bytes": (m + k) * 8, "d2h_bytes": (m + k + nnz) * 8, "roofline": roofline}
    return step_dev, step_e2e, info


if __name__ == "__main__":
    main()
