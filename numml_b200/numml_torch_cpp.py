"""Operator functions with the names, argument order and return shapes of the reference's
``numml_torch_cpp`` extension module (reference ``cpp/sparse_csr.cpp:307-319``; prototypes
``cpp/sparse_csr.hpp:32-105``), implemented on top of the C ABI in ``include/numml_b200.h``.

This layer does what the reference's dispatch stubs and ATen glue do: argument checks, output
and workspace allocation through torch's caching allocator, current-stream lookup, and turning a
non-zero status into a ``RuntimeError``.  All tensors must be CUDA tensors on one device: there
is no CPU implementation behind these functions.
"""
import ctypes

import torch

from . import _cabi, _plan

# How grad_x = A^T g is formed in spgemv_backward: "transpose" (gather over the cached transposed
# structure: atomic-free, deterministic, bit-identical to the reference CPU loop) or "atomic"
# (one fused pass over A with floating-point atomics).
spmv_backward_mode = "transpose"
# Which SpMV kernels run: "auto" picks the TMA-pipelined persistent kernels whenever the pattern is
# regular enough (every block of 256 or 128 rows fits one pipeline stage) and the register-staged
# streaming kernels otherwise; "stream" forces the latter.  Results are identical.
spmv_kernel = "auto"
# Whether the one-pass backward may use the value-symmetric variant (the matrix equals its transpose
# in value too, established by a cached device-side test; see PatternPlan.values_symmetric).
spmv_value_symmetry = True
# Whether SpMV / SpMM calls go through the compiled torch extension (numml_b200/csrc_ext/ops_ext.cpp:
# argument checks, allocation, plan lookup and the C-ABI call in C++) when it has been built.  The
# functions below do the same work in Python and are what runs otherwise; results are identical.
use_compiled_shim = True


def _dtype_code(t):
    if t.dtype == torch.float32:
        return _cabi.F32
    if t.dtype == torch.float64:
        return _cabi.F64
    raise RuntimeError(f"numml_b200 kernels support float32 and float64, got {t.dtype}")


def _require_cuda(*tensors):
    dev = None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            raise RuntimeError(f"expected a torch.Tensor, got {type(t)}")
        if not t.is_cuda:
            raise RuntimeError("numml_b200 operators run on CUDA tensors only (there is no CPU path); "
                               "move the operands to a CUDA device")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"all operands must be on the same device, got {dev} and {t.device}")
    return dev


def _index_tensor(t):
    if t.dtype != torch.int64:
        raise RuntimeError(f"CSR index arrays must be int64 (as the reference stores them), got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _values(t, like=None):
    if like is not None and t.dtype != like.dtype:
        raise RuntimeError(f"operands must share one floating type, got {like.dtype} and {t.dtype}")
    t = t if t.is_contiguous() else t.contiguous()
    if t.data_ptr() % 16 != 0:
        t = t.clone()  # a view at an odd offset: the kernels need 16-byte aligned arrays
    return t


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() > 0 else 0)


def _stream():
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on(dev):
    """Device guard that costs nothing when `dev` is already the current device."""
    if dev.index is None or dev.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(dev)


_status_words = {}


def _status_word(dev):
    """One int32 device word per GPU into which kernels with bounded waits report a failure."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[key]


# -------------------------------------------------------------------------------------------------
# Compiled per-call path
# -------------------------------------------------------------------------------------------------
_ext = None
_ext_tried = False


def _planner(rows, cols, indices, indptr, transpose):
    """What the compiled shim caches per sparsity pattern (called by it on a cache miss)."""
    plan = _plan.get_plan(rows, cols, indices, indptr)
    idx, ptr, itype = plan.csr()
    dev = indices.device
    with _on(dev):
        out = {"idx": idx, "ptr": ptr, "itype": itype, "block_rows": plan.spmv_block_rows(), "status": _status_word(dev),
               "row_order": plan.spmm_row_order(), "t_indptr": None}
        if transpose:
            t_indptr, t_indices, t_perm, _ = plan.transpose()
            out.update(t_indptr=t_indptr, t_indices=t_indices, t_perm=t_perm,
                       t_block_rows=plan.spmv_block_rows(transposed=True), pattern_symmetric=plan.pattern_symmetric(),
                       t_row_order=plan.spmm_row_order(transposed=True))
    return out


def compiled_shim():
    """The extension module, or None when it has not been built (or has been switched off)."""
    global _ext, _ext_tried
    if not use_compiled_shim:
        return None
    if not _ext_tried:
        _ext_tried = True
        import importlib.util
        import os
        from . import build as _build
        path = _build.extension_path()
        if os.path.exists(path):
            _cabi.lib()                                  # the CUDA library first: the extension links against it
            spec = importlib.util.spec_from_file_location(_build.EXT_NAME, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.set_planner(_planner)
            _ext = mod
    return _ext


def _flags():
    if spmv_backward_mode not in ("transpose", "atomic"):
        raise RuntimeError(f"unknown spmv_backward_mode {spmv_backward_mode!r}")
    return (1 if spmv_kernel == "auto" else 0) | (2 if spmv_backward_mode == "transpose" else 0) | (4 if spmv_value_symmetry else 0)


def values_symmetric_state(rows, cols, indices, indptr):
    """What is known about the value symmetry of the last values used with this pattern in spgemv_backward:
    None (nothing tested yet), True or False."""
    ext = compiled_shim()
    if ext is not None:
        return {1: True, 2: False}.get(ext.values_state(indices, indptr))
    state = _plan.get_plan(rows, cols, indices, indptr).extra.get("values_symmetric")
    return None if state is None else state[1]


# -------------------------------------------------------------------------------------------------
# SpMV                                               reference cpp/sparse_csr.hpp:32-42
# -------------------------------------------------------------------------------------------------
def spgemv_forward(A_rows, A_cols, A_data, A_col_ind, A_rowptr, x):
    ext = compiled_shim()
    if ext is not None:
        return ext.spgemv_forward(A_rows, A_cols, A_data, A_col_ind, A_rowptr, x, _flags())
    dev = _require_cuda(A_data, A_col_ind, A_rowptr, x)
    A_data = _values(A_data)
    x = _values(x, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_col_ind), _index_tensor(A_rowptr))
    idx, ptr, itype = plan.csr()
    with _on(dev):
        block_rows = plan.spmv_block_rows() if spmv_kernel == "auto" else 0
        y = torch.empty(A_rows, dtype=A_data.dtype, device=dev)
        _cabi.call("nb200_spgemv_forward", A_rows, A_cols, plan.nnz, _ptr(A_data), _ptr(idx), _ptr(ptr),
                   None, _ptr(x), _ptr(y), block_rows, _ptr(_status_word(dev)), _dtype_code(A_data), itype, _stream())
    return y


def spgemv_backward(grad_z, A_rows, A_cols, A_data, A_col_ind, A_rowptr, x):
    ext = compiled_shim()
    if ext is not None:
        return ext.spgemv_backward(grad_z, A_rows, A_cols, A_data, A_col_ind, A_rowptr, x, _flags())
    dev = _require_cuda(grad_z, A_data, A_col_ind, A_rowptr, x)
    A_data = _values(A_data)
    x = _values(x, A_data)
    g = _values(grad_z, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_col_ind), _index_tensor(A_rowptr))
    idx, ptr, itype = plan.csr()
    if spmv_backward_mode == "transpose":
        t_indptr, t_indices, t_perm, _ = plan.transpose()
    elif spmv_backward_mode == "atomic":
        t_indptr = t_indices = t_perm = None
    else:
        raise RuntimeError(f"unknown spmv_backward_mode {spmv_backward_mode!r}")
    with _on(dev):
        auto = spmv_kernel == "auto"
        block_rows = plan.spmv_block_rows() if auto else 0
        t_block_rows = plan.spmv_block_rows(transposed=True) if (auto and t_indptr is not None) else 0
        symmetric = int(auto and t_indptr is not None and block_rows > 0 and plan.pattern_symmetric())
        if symmetric and spmv_value_symmetry and plan.values_symmetric(A_data):
            symmetric |= 2          # NB200_SYMMETRIC_VALUES
        grad_A = torch.empty_like(A_data)
        grad_x = torch.empty(A_cols, dtype=A_data.dtype, device=dev)
        _cabi.call("nb200_spgemv_backward", A_rows, A_cols, plan.nnz, _ptr(A_data), _ptr(idx), _ptr(ptr),
                   _ptr(x), _ptr(g),
                   _ptr(t_indptr) if t_indptr is not None else None,
                   _ptr(t_indices) if t_indptr is not None else None,
                   _ptr(t_perm) if t_indptr is not None else None,
                   _ptr(grad_A), _ptr(grad_x), block_rows, t_block_rows, symmetric, _ptr(_status_word(dev)),
                   _dtype_code(A_data), itype, _stream())
    return [grad_A, grad_x]


# -------------------------------------------------------------------------------------------------
# Transpose                                          reference cpp/sparse_csr.hpp:57-64
# -------------------------------------------------------------------------------------------------
def csr_transpose_forward(A_rows, A_columns, A_data, A_indices, A_indptr):
    dev = _require_cuda(A_data, A_indices, A_indptr)
    A_data = _values(A_data)
    A_indices, A_indptr = _index_tensor(A_indices), _index_tensor(A_indptr)
    nnz = int(A_indices.numel())
    # the returned arrays are int64 like the reference's, produced directly at that width
    t_indptr, t_indices, t_perm = _plan.transpose_structure(A_rows, A_columns, A_indices, A_indptr,
                                                            _cabi.I64, _cabi.I64)
    with _on(dev):
        At_data = torch.empty_like(A_data)
        _cabi.call("nb200_gather", nnz, _ptr(A_data), _ptr(t_perm), _ptr(At_data),
                   _dtype_code(A_data), _cabi.I64, _stream())
    return [At_data, t_indices, t_indptr, t_perm]


def csr_transpose_backward(grad_At, At_to_A_idx):
    dev = _require_cuda(grad_At, At_to_A_idx)
    grad_At = _values(grad_At)
    idx = _index_tensor(At_to_A_idx)
    with _on(dev):
        grad_A = torch.empty_like(grad_At)
        _cabi.call("nb200_scatter", int(grad_At.numel()), _ptr(grad_At), _ptr(idx), _ptr(grad_A),
                   _dtype_code(grad_At), _cabi.I64, _stream())
    return grad_A


# -------------------------------------------------------------------------------------------------
# SpMM                                               reference cpp/sparse_csr.hpp:81-91
# -------------------------------------------------------------------------------------------------
def _dense(t, like):
    if t.ndim != 2:
        raise RuntimeError(f"expected a 2-D dense matrix, got {t.ndim} dimensions")
    return _values(t, like)


def spdmm_forward(A_rows, A_cols, A_data, A_indices, A_indptr, B):
    ext = compiled_shim()
    if ext is not None:
        return ext.spdmm_forward(A_rows, A_cols, A_data, A_indices, A_indptr, B)
    dev = _require_cuda(A_data, A_indices, A_indptr, B)
    A_data = _values(A_data)
    B = _dense(B, A_data)
    if B.shape[0] != A_cols:
        raise RuntimeError(f"dense operand has {B.shape[0]} rows, expected {A_cols}")
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    idx, ptr, itype = plan.csr()
    K = int(B.shape[1])
    with _on(dev):
        C = torch.empty((A_rows, K), dtype=A_data.dtype, device=dev)
        order = plan.spmm_row_order()
        _cabi.call("nb200_spdmm_forward", A_rows, A_cols, K, plan.nnz, _ptr(A_data), _ptr(idx), _ptr(ptr), None,
                   _ptr(order) if order is not None else None, _ptr(B), _ptr(C), _dtype_code(A_data), itype, _stream())
    return C


def spdmm_backward(A_rows, A_cols, A_data, A_indices, A_indptr, B, grad_C):
    ext = compiled_shim()
    if ext is not None:
        return ext.spdmm_backward(A_rows, A_cols, A_data, A_indices, A_indptr, B, grad_C)
    dev = _require_cuda(A_data, A_indices, A_indptr, B, grad_C)
    A_data = _values(A_data)
    B = _dense(B, A_data)
    G = _dense(grad_C, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    idx, ptr, itype = plan.csr()
    t_indptr, t_indices, t_perm, _ = plan.transpose()
    K = int(B.shape[1])
    code = _dtype_code(A_data)
    with _on(dev):
        grad_A = torch.empty_like(A_data)
        grad_B = torch.empty((A_cols, K), dtype=A_data.dtype, device=dev)
        order, t_order = plan.spmm_row_order(), plan.spmm_row_order(transposed=True)
        _cabi.call("nb200_spdmm_backward_grad_A", A_rows, A_cols, K, plan.nnz, _ptr(idx), _ptr(ptr),
                   _ptr(order) if order is not None else None, _ptr(B), _ptr(G), _ptr(grad_A), code, itype, _stream())
        # grad_B = A^T grad_C: the forward kernel over the transposed structure, values via the permutation
        _cabi.call("nb200_spdmm_forward", A_cols, A_rows, K, plan.nnz, _ptr(A_data), _ptr(t_indices), _ptr(t_indptr),
                   _ptr(t_perm), _ptr(t_order) if t_order is not None else None, _ptr(G), _ptr(grad_B), code, itype, _stream())
    return [grad_A, grad_B]


# -------------------------------------------------------------------------------------------------
# SpGEMM                                             reference cpp/sparse_csr.hpp:45-54
# -------------------------------------------------------------------------------------------------
def _common_width(plan_a, plan_b):
    """CSR arrays of both operands in one index width (int32 only if both patterns fit)."""
    if plan_a.fits_int32() and plan_b.fits_int32():
        ai, ap, itype = plan_a.csr()
        bi, bp, _ = plan_b.csr()
        return ai, ap, bi, bp, itype
    return plan_a.indices, plan_a.indptr, plan_b.indices, plan_b.indptr, _cabi.I64


# positions in the 24-word header of an SpGEMM workspace (see nb200_spgemm_plan in the C header)
_HDR_SYM_SPILL, _HDR_NUM_SPILL, _HDR_NNZ, _HDR_ERROR = 6, 14, 15, 16


def _header(work):
    """The 24-word int64 header at the start of an SpGEMM workspace (device-to-host copy, syncs)."""
    return work[:192].view(torch.int64).cpu()


# Whether the results of the symbolic phase of the most recent product are kept with the plan of its left factor
# (about 40 bytes per row of A): a product of the same two patterns then runs its numeric phase only.
spgemm_keep_symbolic = True


def spgemm_forward(A_rows, A_cols, A_data, A_indices, A_indptr, B_rows, B_cols, B_data, B_indices, B_indptr):
    dev = _require_cuda(A_data, A_indices, A_indptr, B_data, B_indices, B_indptr)
    A_data = _values(A_data)
    B_data = _values(B_data, A_data)
    plan_a = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    plan_b = _plan.get_plan(B_rows, B_cols, _index_tensor(B_indices), _index_tensor(B_indptr))
    ai, ap, bi, bp, itype = _common_width(plan_a, plan_b)
    code = _dtype_code(A_data)
    vbytes = A_data.element_size()
    with _on(dev):
        wbytes = _cabi.lib().nb200_spgemm_workspace_bytes(A_rows)
        # The symbolic phase depends on the two patterns only.  Its results (row pointers of C, the binned row
        # lists the numeric phase walks, the size of its spill area) are kept with the plan of the left factor for
        # the most recent right factor (from the second product of the pair on), so that a product of the same
        # patterns with new values -- every step of a training loop -- runs the numeric phase alone, with no host
        # read in between.
        key = ("spgemm_symbolic", itype)
        kept = plan_a.extra.get(key) if spgemm_keep_symbolic else None
        if kept is not None and kept["plan_b"] is plan_b:
            C_indptr = kept["C_indptr"].clone()
            nnz_c, slots = kept["nnz"], kept["spill_slots"]
            spill = torch.empty(slots * (vbytes + 4), dtype=torch.uint8, device=dev) if slots else None
            C_indices = torch.empty(nnz_c, dtype=torch.int64, device=dev)
            C_data = torch.empty(nnz_c, dtype=A_data.dtype, device=dev)
            _cabi.call("nb200_spgemm_numeric", A_rows, A_cols, B_cols, _ptr(A_data), _ptr(ai), _ptr(ap),
                       _ptr(B_data), _ptr(bi), _ptr(bp), code, itype, _ptr(kept["work"]), wbytes, _ptr(spill), slots,
                       _ptr(C_indptr), _ptr(C_indices), _ptr(C_data), _stream())
            return [C_data, C_indices, C_indptr]
        work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        C_indptr = torch.empty(A_rows + 1, dtype=torch.int64, device=dev)

        b_sorted = int(not (plan_b.check_flags() & _plan.CHECK_UNSORTED))

        def count(spill, slots):
            _cabi.call("nb200_spgemm_plan", A_rows, A_cols, plan_a.nnz, _ptr(ai), _ptr(ap), _ptr(bp), b_sorted, itype,
                       _ptr(work), wbytes, _stream())
            _cabi.call("nb200_spgemm_symbolic", A_rows, A_cols, B_cols, _ptr(ai), _ptr(ap), _ptr(bi), _ptr(bp), itype,
                       _ptr(work), wbytes, _ptr(spill), slots, _ptr(C_indptr), _stream())
            return _header(work)

        # One host read per product: planning and the symbolic phase are enqueued together, without a
        # spill area.  Only a matrix with rows of more than 4096 products needs one; the header then says
        # how large, and the two steps run once more with it.
        head = count(None, 0)
        slots = int(head[_HDR_SYM_SPILL])
        if slots > 0:
            spill = torch.empty(slots * 4, dtype=torch.uint8, device=dev)
            head = count(spill, slots)
        if int(head[_HDR_ERROR]) != 0:
            raise RuntimeError("nb200_spgemm_symbolic: spill area too small")
        nnz_c, slots = int(head[_HDR_NNZ]), int(head[_HDR_NUM_SPILL])
        spill = torch.empty(slots * (vbytes + 4), dtype=torch.uint8, device=dev) if slots else None
        C_indices = torch.empty(nnz_c, dtype=torch.int64, device=dev)
        C_data = torch.empty(nnz_c, dtype=A_data.dtype, device=dev)
        _cabi.call("nb200_spgemm_numeric", A_rows, A_cols, B_cols, _ptr(A_data), _ptr(ai), _ptr(ap),
                   _ptr(B_data), _ptr(bi), _ptr(bp), code, itype, _ptr(work), wbytes, _ptr(spill), slots,
                   _ptr(C_indptr), _ptr(C_indices), _ptr(C_data), _stream())
        if spgemm_keep_symbolic:
            # kept from the second product of a pair of patterns on: a product that is formed once (an intermediate
            # of a chain with fresh operands) must not pin 40 bytes per row for the life of its plan
            seen = ("spgemm_seen", itype)
            if plan_a.extra.get(seen) is plan_b:
                plan_a.extra[key] = {"plan_b": plan_b, "work": work, "C_indptr": C_indptr.clone(), "nnz": nnz_c,
                                     "spill_slots": slots}
            else:
                plan_a.extra[seen] = plan_b
                plan_a.extra.pop(key, None)
    return [C_data, C_indices, C_indptr]


def spgemm_backward(grad_C, C_indices, C_indptr, A_rows, A_cols, A_data, A_indices, A_indptr,
                    B_rows, B_cols, B_data, B_indices, B_indptr):
    dev = _require_cuda(grad_C, C_indices, C_indptr, A_data, A_indices, A_indptr, B_data, B_indices, B_indptr)
    A_data = _values(A_data)
    B_data = _values(B_data, A_data)
    grad_C = _values(grad_C, A_data)
    C_indices, C_indptr = _index_tensor(C_indices), _index_tensor(C_indptr)
    plan_a = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    plan_b = _plan.get_plan(B_rows, B_cols, _index_tensor(B_indices), _index_tensor(B_indptr))
    # the gradients are found by merging / searching the sorted rows of B and C (the reference,
    # cpp/sparse_csr_cpu.cpp:218-307, assumes the same); the order of the entries within a row of A is free
    plan_b.require(sorted_columns=True, what="the SpGEMM backward")
    ai, ap, bi, bp, itype = _common_width(plan_a, plan_b)
    if itype == _cabi.I32:
        t_indptr, t_indices, t_perm, _ = plan_a.transpose()
    else:
        t_indptr, t_indices, t_perm = _plan.transpose_structure(A_rows, A_cols, ai, ap, _cabi.I64, _cabi.I64)
    with _on(dev):
        grad_A = torch.empty_like(A_data)
        grad_B = torch.empty_like(B_data)
        _cabi.call("nb200_spgemm_backward", A_rows, A_cols, plan_a.nnz, _ptr(A_data), _ptr(ai), _ptr(ap),
                   _ptr(t_indptr), _ptr(t_indices), _ptr(t_perm), B_rows, B_cols, plan_b.nnz,
                   _ptr(B_data), _ptr(bi), _ptr(bp), _ptr(grad_C), _ptr(C_indices), _ptr(C_indptr),
                   _ptr(grad_A), _ptr(grad_B), _dtype_code(A_data), itype, _stream())
    return [grad_A, grad_B]


# -------------------------------------------------------------------------------------------------
# Triangular solve                                   reference cpp/sparse_csr.hpp:94-105
# -------------------------------------------------------------------------------------------------
# Poll budget of the solve kernel in SM cycles (about a second) and whether every solve reads the
# device status word back (one small synchronising copy) so that an expired wait raises at once.
sptrsv_wait_budget_cycles = 2_000_000_000
_RESIDENT_THREADS = 148 * 2048               # threads a B200 keeps resident at once
sptrsv_check_status = True
# Which solve kernel runs: "auto" and "syncfree" take the grid-wide sync-free kernel; "cluster" takes the
# cluster kernel (levels one after the other inside one thread-block cluster, unknowns exchanged through
# distributed shared memory) whenever its ring of recent rows fits.  Results are identical; on B200 the
# cluster barrier costs more per level than a store and a poll through L2, so "auto" never picks it.
sptrsv_kernel = "auto"
sptrsv_cluster_ctas = 8


def check_status(device=None):
    """Read (and clear) the device status word written by kernels with bounded waits; raises
    RuntimeError if one of them gave up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(dev)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"numml_b200 device status {code}: "
                           f"{_cabi.lib().nb200_status_string(code).decode()} (results of the affected call hold NaN)")


def _team_lanes(n, nlevels):
    """Lanes per row for the triangular solve.  With narrow levels the solve is bound by the chain of
    poll round trips, and a warp that holds one row is not held up by the slowest of several; with
    wide levels the rows of a level fill the GPU and the lanes are better spent on more rows."""
    width = n / max(int(nlevels), 1)                     # average rows per level
    lanes = 32
    while lanes > 1 and width * lanes > _RESIDENT_THREADS:
        lanes //= 2
    return lanes


def _cluster_solve_fits(levels, n, nrhs):
    """Whether the cluster solve can run for this pattern and number of right-hand sides: its ring must
    hold `reach` rows of nrhs doubles within 200 KiB per CTA."""
    if levels is None or nrhs < 1:
        return False
    cap = 1
    while sptrsv_cluster_ctas * cap < levels["reach"]:
        cap *= 2
    return cap * nrhs * 8 <= 200 * 1024


def _solve(plan, data, idx, ptr, perm, itype, lower, unit, b, transposed=False):
    """x = A^{-1} b with the kernel named by ``sptrsv_kernel``."""
    n = plan.rows
    nrhs = 1 if b.ndim == 1 else int(b.shape[1])
    dev = b.device
    x = torch.empty_like(b)
    order, nlevels = plan.sptrsv_order(lower, transposed)
    if sptrsv_kernel == "cluster" and n > 0 and nrhs > 0:
        levels = plan.sptrsv_level_plan(lower, transposed)
        if _cluster_solve_fits(levels, n, nrhs):
            wbytes = _cabi.lib().nb200_sptrsv_solve_levels_workspace_bytes(n, nrhs, levels["entries"])
            work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
            _cabi.call("nb200_sptrsv_solve_levels", n, nrhs, levels["entries"], _ptr(data), _ptr(levels["src"]),
                       _ptr(levels["pos_ptr"]), _ptr(levels["dep"]), _ptr(order), _ptr(levels["level_ptr"]), nlevels,
                       levels["reach"], int(bool(unit)), _ptr(b), _ptr(x), _ptr(work), wbytes, int(sptrsv_cluster_ctas),
                       _dtype_code(data), _stream())
            return x
    xd = torch.empty(n * nrhs, dtype=torch.float64, device=dev) if b.dtype == torch.float32 else None
    status = _status_word(dev)
    _cabi.call("nb200_sptrsv_solve", n, plan.nnz, nrhs, _ptr(data), _ptr(idx), _ptr(ptr),
               _ptr(perm) if perm is not None else None, _ptr(order), int(bool(lower)), int(bool(unit)),
               _ptr(b), _ptr(x), _ptr(xd) if xd is not None else None, _ptr(status),
               int(sptrsv_wait_budget_cycles), _team_lanes(n, nlevels), _dtype_code(data), itype, _stream())
    if sptrsv_check_status:
        check_status(dev)
    return x


def _rhs(b, n, like):
    if b.ndim not in (1, 2) or b.shape[0] != n:
        raise RuntimeError(f"right-hand side must have shape ({n},) or ({n}, k), got {tuple(b.shape)}")
    return _values(b, like)


def sptrsv_forward(A_rows, A_cols, A_data, A_indices, A_indptr, lower, unit, b):
    dev = _require_cuda(A_data, A_indices, A_indptr, b)
    if A_rows != A_cols:
        raise RuntimeError(f"triangular solve needs a square matrix, got {A_rows} x {A_cols}")
    A_data = _values(A_data)
    b = _rhs(b, A_rows, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    plan.require(sorted_columns=True, diagonal=not unit, what="the triangular solve")
    idx, ptr, itype = plan.csr()
    with _on(dev):
        return _solve(plan, A_data, idx, ptr, None, itype, lower, unit, b)


def sptrsv_backward(grad_x, x, A_rows, A_cols, A_data, A_indices, A_indptr, lower, unit, b):
    dev = _require_cuda(grad_x, x, A_data, A_indices, A_indptr)
    A_data = _values(A_data)
    grad_x = _rhs(grad_x, A_rows, A_data)
    x = _rhs(x, A_rows, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    plan.require(sorted_columns=True, diagonal=not unit, what="the triangular solve")
    idx, ptr, itype = plan.csr()
    nrhs = 1 if x.ndim == 1 else int(x.shape[1])
    with _on(dev):
        t_indptr, t_indices, t_perm, _ = plan.transpose()
        # grad_b = A^{-T} grad_x: the opposite-triangle solve on the transposed structure
        grad_b = _solve(plan, A_data, t_indices, t_indptr, t_perm, itype, not lower, unit, grad_x, transposed=True)
        grad_A = torch.empty_like(A_data)
        _cabi.call("nb200_masked_outer", A_rows, plan.nnz, nrhs, _ptr(idx), _ptr(ptr), _ptr(grad_b), _ptr(x), -1.0,
                   _ptr(grad_A), _dtype_code(A_data), itype, _stream())
    return [grad_A, grad_b]


# -------------------------------------------------------------------------------------------------
# Conjugate gradients, fixed iteration count          reference numml/krylov.py:83-155
# -------------------------------------------------------------------------------------------------
def cg_fixed_iterations(A_rows, A_data, A_indices, A_indptr, b, x0, iterations):
    """``iterations`` unpreconditioned CG steps for the square matrix A, enqueued without any host
    synchronisation.  Returns ``(x, residual_history)``, the history having iterations + 1 entries."""
    dev = _require_cuda(A_data, A_indices, A_indptr, b)
    A_data = _values(A_data)
    b = _values(b, A_data)
    if b.ndim != 1 or b.shape[0] != A_rows:
        raise RuntimeError(f"right-hand side must have shape ({A_rows},), got {tuple(b.shape)}")
    plan = _plan.get_plan(A_rows, A_rows, _index_tensor(A_indices), _index_tensor(A_indptr))
    idx, ptr, itype = plan.csr()
    code = _dtype_code(A_data)
    with _on(dev):
        block_rows = plan.spmv_block_rows() if spmv_kernel == "auto" else 0
        x = _values(x0, A_data).clone() if x0 is not None else torch.empty_like(b)
        hist = torch.empty(iterations + 1, dtype=b.dtype, device=dev)
        wbytes = _cabi.lib().nb200_cg_workspace_bytes(A_rows, code)
        work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        _cabi.call("nb200_cg_fixed_iterations", A_rows, plan.nnz, _ptr(A_data), _ptr(idx), _ptr(ptr), block_rows,
                   _ptr(b), _ptr(x), int(x0 is not None), _ptr(hist), int(iterations), _ptr(work), wbytes,
                   _ptr(_status_word(dev)), code, itype, _stream())
    return x, hist


# -------------------------------------------------------------------------------------------------
# Pattern-building operators     reference cpp/sparse_csr.hpp:66-78, numml/sparse/_csr.py:78-99, 234-330
# -------------------------------------------------------------------------------------------------
def _pattern_workspace(rows, dev):
    wbytes = _cabi.lib().nb200_pattern_workspace_bytes(rows)
    return torch.empty(wbytes, dtype=torch.uint8, device=dev), wbytes


def splincomb_forward(rows, cols, alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr):
    """C = alpha A + beta B on the union pattern (both operands with ascending columns per row).
    ``alpha`` / ``beta`` are Python numbers or 0-d tensors, as in the reference."""
    dev = _require_cuda(A_data, A_indices, A_indptr, B_data, B_indices, B_indptr)
    A_data = _values(A_data)
    B_data = _values(B_data, A_data)
    A_indices, A_indptr = _index_tensor(A_indices), _index_tensor(A_indptr)
    B_indices, B_indptr = _index_tensor(B_indices), _index_tensor(B_indptr)
    _plan.get_plan(rows, cols, A_indices, A_indptr).require(sorted_columns=True, what="the linear combination")
    _plan.get_plan(rows, cols, B_indices, B_indptr).require(sorted_columns=True, what="the linear combination")
    alpha, beta = float(alpha), float(beta)
    with _on(dev):
        work, wbytes = _pattern_workspace(rows, dev)
        C_indptr = torch.empty(rows + 1, dtype=torch.int64, device=dev)
        _cabi.call("nb200_csr_lincomb_count", rows, _ptr(A_indices), _ptr(A_indptr), _ptr(B_indices), _ptr(B_indptr),
                   _ptr(C_indptr), _ptr(work), wbytes, _stream())
        nnz_c = int(C_indptr[-1].item())
        C_data = torch.empty(nnz_c, dtype=A_data.dtype, device=dev)
        C_indices = torch.empty(nnz_c, dtype=torch.int64, device=dev)
        _cabi.call("nb200_csr_lincomb_fill", rows, alpha, _ptr(A_data), _ptr(A_indices), _ptr(A_indptr), beta, _ptr(B_data),
                   _ptr(B_indices), _ptr(B_indptr), _ptr(C_indptr), _ptr(C_data), _ptr(C_indices), _dtype_code(A_data), _stream())
    return [C_data, C_indices, C_indptr]


def splincomb_backward(rows, cols, alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr,
                       grad_C_data, C_indices, C_indptr):
    dev = _require_cuda(A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, grad_C_data, C_indices, C_indptr)
    grad_C = _values(grad_C_data, A_data)
    with _on(dev):
        # every entry of A and of B lies in the union pattern, so both gradients are written in full
        grad_A = torch.empty_like(A_data)
        grad_B = torch.empty_like(B_data)
        _cabi.call("nb200_csr_lincomb_backward", rows, float(alpha), _ptr(_index_tensor(A_indices)), _ptr(_index_tensor(A_indptr)),
                   float(beta), _ptr(_index_tensor(B_indices)), _ptr(_index_tensor(B_indptr)), _ptr(grad_C),
                   _ptr(_index_tensor(C_indices)), _ptr(_index_tensor(C_indptr)), _ptr(grad_A), _ptr(grad_B),
                   _dtype_code(A_data), _stream())
    return [grad_A, grad_B]


def csr_triangle(rows, cols, A_data, A_indices, A_indptr, k, lower):
    """Entries on or below (``lower``) / on or above diagonal ``k``.  Returns ``[data, indices, indptr,
    positions]``, the last being the position in A of every entry kept."""
    dev = _require_cuda(A_data, A_indices, A_indptr)
    A_data = _values(A_data)
    A_indices, A_indptr = _index_tensor(A_indices), _index_tensor(A_indptr)
    _plan.get_plan(rows, cols, A_indices, A_indptr)             # structure check: nothing may index out of bounds
    with _on(dev):
        work, wbytes = _pattern_workspace(rows, dev)
        out_indptr = torch.empty(rows + 1, dtype=torch.int64, device=dev)
        _cabi.call("nb200_csr_triangle_count", rows, _ptr(A_indices), _ptr(A_indptr), int(k), int(bool(lower)),
                   _ptr(out_indptr), _ptr(work), wbytes, _stream())
        n = int(out_indptr[-1].item())
        out_data = torch.empty(n, dtype=A_data.dtype, device=dev)
        out_indices = torch.empty(n, dtype=torch.int64, device=dev)
        out_pos = torch.empty(n, dtype=torch.int64, device=dev)
        _cabi.call("nb200_csr_triangle_fill", rows, _ptr(A_data), _ptr(A_indices), _ptr(A_indptr), int(k), int(bool(lower)),
                   _ptr(out_indptr), _ptr(out_data), _ptr(out_indices), _ptr(out_pos), _dtype_code(A_data), _stream())
    return [out_data, out_indices, out_indptr, out_pos]


def scatter_into(dst, src, idx):
    """dst[idx[k]] = src[k] for every k, in place (``idx`` int64 without repeats); returns ``dst``."""
    dev = _require_cuda(dst, src, idx)
    with _on(dev):
        _cabi.call("nb200_scatter", int(src.numel()), _ptr(_values(src, dst)), _ptr(_index_tensor(idx)), _ptr(dst),
                   _dtype_code(dst), _cabi.I64, _stream())
    return dst


def coo_to_csr_order(row_ind, col_ind, nrows, ncols, sort_columns=True):
    """``(perm, indptr)`` of the COO entries sorted stably by (row, column) -- by row only when
    ``sort_columns`` is false: entry ``perm[q]`` comes q-th."""
    dev = _require_cuda(row_ind, col_ind)
    row_ind, col_ind = _index_tensor(row_ind), _index_tensor(col_ind)
    n = int(row_ind.numel())
    if n > 0 and (int(row_ind.min()) < 0 or int(row_ind.max()) >= nrows or int(col_ind.min()) < 0 or int(col_ind.max()) >= ncols):
        raise RuntimeError(f"COO indices outside the matrix shape ({nrows}, {ncols})")
    with _on(dev):
        wbytes = _cabi.lib().nb200_coo_workspace_bytes(n)
        work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        perm = torch.empty(n, dtype=torch.int64, device=dev)
        indptr = torch.empty(nrows + 1, dtype=torch.int64, device=dev)
        _cabi.call("nb200_coo_to_csr", n, _ptr(row_ind), _ptr(col_ind), nrows, ncols, int(bool(sort_columns)), _ptr(perm),
                   _ptr(indptr), _ptr(work), wbytes, _stream())
    return perm, indptr


# -------------------------------------------------------------------------------------------------
# Sparse LU and the direct solve                      reference cpp/sparse_csr.hpp:107-118
# -------------------------------------------------------------------------------------------------
def splu(A_rows, A_cols, A_data, A_indices, A_indptr):
    """LU without pivoting on the filled pattern.  Returns ``[M_data, M_indices, M_indptr, Mt_data,
    Mt_indices, Mt_indptr]`` like the reference: M = L + U (unit lower L, ones not stored) and its transpose."""
    dev = _require_cuda(A_data, A_indices, A_indptr)
    if A_rows != A_cols:
        raise RuntimeError(f"LU factorisation needs a square matrix, got {A_rows} x {A_cols}")
    A_data = _values(A_data)
    A_indices, A_indptr = _index_tensor(A_indices), _index_tensor(A_indptr)
    plan = _plan.get_plan(A_rows, A_cols, A_indices, A_indptr)
    plan.require(sorted_columns=True, diagonal=True, what="the LU factorisation")
    n = A_rows
    code = _dtype_code(A_data)
    with _on(dev):
        wbytes = _cabi.lib().nb200_splu_workspace_bytes(n)
        work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        M_indptr = torch.empty(n + 1, dtype=torch.int64, device=dev)
        _cabi.call("nb200_splu_symbolic_count", n, _ptr(A_indices), _ptr(A_indptr), _ptr(M_indptr), _ptr(work), wbytes, _stream())
        nnz_m = int(M_indptr[-1].item())
        M_indices = torch.empty(nnz_m, dtype=torch.int64, device=dev)
        M_data = torch.empty(nnz_m, dtype=A_data.dtype, device=dev)
        _cabi.call("nb200_splu_symbolic_fill", n, _ptr(A_data), _ptr(A_indices), _ptr(A_indptr), _ptr(M_indptr),
                   _ptr(M_indices), _ptr(M_data), _ptr(work), wbytes, code, _stream())
        del work
        Mt_data, Mt_indices, Mt_indptr, perm = csr_transpose_forward(n, n, M_data, M_indices, M_indptr)
        done = torch.empty(n, dtype=torch.int32, device=dev)
        status = _status_word(dev)
        _cabi.call("nb200_splu_numeric", n, _ptr(Mt_data), _ptr(Mt_indices), _ptr(Mt_indptr), _ptr(done), _ptr(status),
                   int(sptrsv_wait_budget_cycles), code, _stream())
        check_status(dev)
        # back to rows: entry q of the transpose is entry perm[q] of M
        _cabi.call("nb200_scatter", nnz_m, _ptr(Mt_data), _ptr(perm), _ptr(M_data), code, _cabi.I64, _stream())
    return [M_data, M_indices, M_indptr, Mt_data, Mt_indices, Mt_indptr]


def spsolve_backward(grad_x, x, A_rows, A_cols, Mt_data, Mt_indices, Mt_indptr, A_data, A_indices, A_indptr):
    """grad_b = A^{-T} grad_x by two triangular solves with the transposed factors (U^T is lower with the
    pivots on its diagonal, L^T is unit upper); grad_A = -(grad_b x^T) on the pattern of A."""
    y = sptrsv_forward(A_rows, A_cols, Mt_data, Mt_indices, Mt_indptr, True, False, grad_x)
    grad_b = sptrsv_forward(A_rows, A_cols, Mt_data, Mt_indices, Mt_indptr, False, True, y)
    dev = _require_cuda(A_data, A_indices, A_indptr, x)
    A_data = _values(A_data)
    x = _rhs(x, A_rows, A_data)
    plan = _plan.get_plan(A_rows, A_cols, _index_tensor(A_indices), _index_tensor(A_indptr))
    idx, ptr, itype = plan.csr()
    nrhs = 1 if x.ndim == 1 else int(x.shape[1])
    with _on(dev):
        grad_A = torch.empty_like(A_data)
        _cabi.call("nb200_masked_outer", A_rows, plan.nnz, nrhs, _ptr(idx), _ptr(ptr), _ptr(grad_b), _ptr(x), -1.0,
                   _ptr(grad_A), _dtype_code(A_data), itype, _stream())
    return [grad_A, grad_b]

