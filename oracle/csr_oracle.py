"""ctypes front-end of ``csr_oracle.c``, the plain-C restatement of the reference CPU algorithms.

TEST INFRASTRUCTURE ONLY.  The product never imports this; it exists so that the CUDA path
can be checked on machines where the reference sources are not present.  Function names and
argument order follow the reference operator module (``cpp/sparse_csr.hpp:32-105``), operating
on CPU torch tensors, so a test can run the same call against this port, against the compiled
reference (``oracle/_ref``) and against the CUDA path.
"""
import ctypes
import os
import subprocess

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csr_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libcsr_oracle.so")

_lib = None


def build(force=False):
    """Compile csr_oracle.c with gcc.  -ffp-contract=off keeps multiply and add separate, as in
    the reference's plain x86-64 -O2 build, so results are bit-identical to it."""
    if os.path.exists(LIB) and not force and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c99",
                           SRC, "-o", LIB])
    return LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_spgemm_symbolic.restype = ctypes.c_int64
    return _lib


def _sfx(t):
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise TypeError(f"oracle supports float32/float64, got {t.dtype}")


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _c(t, dtype=None):
    t = t.detach().cpu().contiguous()
    if dtype is not None:
        t = t.to(dtype)
    return t


def _i(v):
    return ctypes.c_int64(int(v))


def spgemv_forward(rows, cols, data, indices, indptr, x):
    data, indices, indptr, x = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64), _c(x)
    y = torch.empty(rows, dtype=data.dtype)
    getattr(lib(), "oracle_spgemv_forward_" + _sfx(data))(_i(rows), _p(data), _p(indices), _p(indptr), _p(x), _p(y))
    return y


def spgemv_backward(grad_z, rows, cols, data, indices, indptr, x):
    data, indices, indptr, x, g = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64), _c(x), _c(grad_z)
    grad_A = torch.empty_like(data)
    grad_x = torch.empty(cols, dtype=data.dtype)
    getattr(lib(), "oracle_spgemv_backward_" + _sfx(data))(
        _i(rows), _i(cols), _p(data), _p(indices), _p(indptr), _p(x), _p(g), _p(grad_A), _p(grad_x))
    return [grad_A, grad_x]


def spgemm_forward(A_rows, A_cols, A_data, A_indices, A_indptr, B_rows, B_cols, B_data, B_indices, B_indptr):
    A_data, A_indices, A_indptr = _c(A_data), _c(A_indices, torch.int64), _c(A_indptr, torch.int64)
    B_data, B_indices, B_indptr = _c(B_data), _c(B_indices, torch.int64), _c(B_indptr, torch.int64)
    C_indptr = torch.empty(A_rows + 1, dtype=torch.int64)
    nnz = lib().oracle_spgemm_symbolic(_i(A_rows), _i(A_cols), _i(B_cols), _p(A_indices), _p(A_indptr),
                                       _p(B_indices), _p(B_indptr), _p(C_indptr))
    C_data = torch.empty(nnz, dtype=A_data.dtype)
    C_indices = torch.empty(nnz, dtype=torch.int64)
    getattr(lib(), "oracle_spgemm_numeric_" + _sfx(A_data))(
        _i(A_rows), _i(A_cols), _i(B_cols), _p(A_data), _p(A_indices), _p(A_indptr),
        _p(B_data), _p(B_indices), _p(B_indptr), _p(C_indptr), _p(C_data), _p(C_indices))
    return [C_data, C_indices, C_indptr]


def spgemm_backward(grad_C, C_indices, C_indptr, A_rows, A_cols, A_data, A_indices, A_indptr,
                    B_rows, B_cols, B_data, B_indices, B_indptr):
    grad_C, C_indices, C_indptr = _c(grad_C), _c(C_indices, torch.int64), _c(C_indptr, torch.int64)
    A_data, A_indices, A_indptr = _c(A_data), _c(A_indices, torch.int64), _c(A_indptr, torch.int64)
    B_data, B_indices, B_indptr = _c(B_data), _c(B_indices, torch.int64), _c(B_indptr, torch.int64)
    grad_A = torch.empty_like(A_data)
    grad_B = torch.empty_like(B_data)
    getattr(lib(), "oracle_spgemm_backward_" + _sfx(A_data))(
        _p(grad_C), _p(C_indices), _p(C_indptr), _i(A_rows), _p(A_data), _p(A_indices), _p(A_indptr),
        _i(B_rows), _p(B_data), _p(B_indices), _p(B_indptr), _p(grad_A), _p(grad_B))
    return [grad_A, grad_B]


def csr_transpose_forward(rows, cols, data, indices, indptr):
    data, indices, indptr = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64)
    nnz = data.numel()
    t_data = torch.empty_like(data)
    t_indices = torch.empty(nnz, dtype=torch.int64)
    t_indptr = torch.empty(cols + 1, dtype=torch.int64)
    to_A = torch.empty(nnz, dtype=torch.int64)
    getattr(lib(), "oracle_csr_transpose_forward_" + _sfx(data))(
        _i(rows), _i(cols), _p(data), _p(indices), _p(indptr), _p(t_data), _p(t_indices), _p(t_indptr), _p(to_A))
    return [t_data, t_indices, t_indptr, to_A]


def csr_transpose_backward(grad_At, At_to_A_idx):
    grad_At, to_A = _c(grad_At), _c(At_to_A_idx, torch.int64)
    grad_A = torch.empty_like(grad_At)
    getattr(lib(), "oracle_csr_transpose_backward_" + _sfx(grad_At))(_i(grad_At.numel()), _p(grad_At), _p(to_A), _p(grad_A))
    return grad_A


def spdmm_forward(rows, cols, data, indices, indptr, B):
    data, indices, indptr, B = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64), _c(B)
    C = torch.empty((rows, B.shape[1]), dtype=data.dtype)
    getattr(lib(), "oracle_spdmm_forward_" + _sfx(data))(
        _i(rows), _p(data), _p(indices), _p(indptr), _p(B), _i(B.shape[1]), _p(C))
    return C


def spdmm_backward(rows, cols, data, indices, indptr, B, grad_C):
    data, indices, indptr = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64)
    B, grad_C = _c(B), _c(grad_C)
    grad_A = torch.empty_like(data)
    grad_B = torch.empty_like(B)
    getattr(lib(), "oracle_spdmm_backward_" + _sfx(data))(
        _i(rows), _i(cols), _p(data), _p(indices), _p(indptr), _p(B), _p(grad_C), _i(B.shape[1]),
        _p(grad_A), _p(grad_B))
    return [grad_A, grad_B]


def sptrsv_forward(rows, cols, data, indices, indptr, lower, unit, b):
    data, indices, indptr, b = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64), _c(b)
    x = torch.empty(rows, dtype=data.dtype)
    getattr(lib(), "oracle_sptrsv_forward_" + _sfx(data))(
        _i(rows), _p(data), _p(indices), _p(indptr), ctypes.c_int(bool(lower)), ctypes.c_int(bool(unit)), _p(b), _p(x))
    return x


def sptrsv_backward(grad_x, x, rows, cols, data, indices, indptr, lower, unit, b):
    data, indices, indptr = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64)
    grad_x, x = _c(grad_x), _c(x)
    grad_A = torch.empty_like(data)
    grad_b = torch.empty(rows, dtype=data.dtype)
    getattr(lib(), "oracle_sptrsv_backward_" + _sfx(data))(
        _i(rows), _p(data), _p(indices), _p(indptr), ctypes.c_int(bool(lower)), ctypes.c_int(bool(unit)),
        _p(grad_x), _p(x), _p(grad_A), _p(grad_b))
    return [grad_A, grad_b]


def splincomb_forward(rows, cols, alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr):
    A_data, A_indices, A_indptr = _c(A_data), _c(A_indices, torch.int64), _c(A_indptr, torch.int64)
    B_data, B_indices, B_indptr = _c(B_data), _c(B_indices, torch.int64), _c(B_indptr, torch.int64)
    lib().oracle_splincomb_count.restype = ctypes.c_int64
    C_indptr = torch.empty(rows + 1, dtype=torch.int64)
    nnz = lib().oracle_splincomb_count(_i(rows), _p(A_indices), _p(A_indptr), _p(B_indices), _p(B_indptr), _p(C_indptr))
    C_data = torch.empty(nnz, dtype=A_data.dtype)
    C_indices = torch.empty(nnz, dtype=torch.int64)
    scalar = ctypes.c_double if A_data.dtype == torch.float64 else ctypes.c_float
    getattr(lib(), "oracle_splincomb_forward_" + _sfx(A_data))(
        _i(rows), scalar(float(alpha)), _p(A_data), _p(A_indices), _p(A_indptr), scalar(float(beta)), _p(B_data),
        _p(B_indices), _p(B_indptr), _p(C_data), _p(C_indices))
    return [C_data, C_indices, C_indptr]


def splincomb_backward(rows, cols, alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr,
                       grad_C, C_indices, C_indptr):
    A_data, A_indices, A_indptr = _c(A_data), _c(A_indices, torch.int64), _c(A_indptr, torch.int64)
    B_data, B_indices, B_indptr = _c(B_data), _c(B_indices, torch.int64), _c(B_indptr, torch.int64)
    grad_C, C_indices, C_indptr = _c(grad_C), _c(C_indices, torch.int64), _c(C_indptr, torch.int64)
    scalar = ctypes.c_double if A_data.dtype == torch.float64 else ctypes.c_float
    fn = getattr(lib(), "oracle_splincomb_backward_" + _sfx(A_data))
    grad_A, grad_B = torch.empty_like(A_data), torch.empty_like(B_data)
    fn(_i(rows), scalar(float(alpha)), _p(A_indices), _p(A_indptr), _p(grad_C), _p(C_indices), _p(C_indptr), _p(grad_A))
    fn(_i(rows), scalar(float(beta)), _p(B_indices), _p(B_indptr), _p(grad_C), _p(C_indices), _p(C_indptr), _p(grad_B))
    return [grad_A, grad_B]


def splu(rows, cols, data, indices, indptr):
    """Sparse LU without pivoting, as the reference's splu (cpp/sparse_csr_cpu.cpp:778-1017): returns
    ``[M_data, M_indices, M_indptr, Mt_data, Mt_indices, Mt_indptr]`` with M = L + U (unit lower L, its
    ones not stored) on the filled pattern and Mt its transpose."""
    data, indices, indptr = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64)
    n = rows
    lib().oracle_splu_symbolic.restype = ctypes.c_int64
    M_indptr = torch.empty(n + 1, dtype=torch.int64)
    nnz = lib().oracle_splu_symbolic(_i(n), _p(indices), _p(indptr), _p(M_indptr), None, None)
    M_indices = torch.empty(nnz, dtype=torch.int64)
    is_fill = torch.empty(nnz, dtype=torch.int32)
    lib().oracle_splu_symbolic(_i(n), _p(indices), _p(indptr), _p(M_indptr), _p(M_indices), _p(is_fill))
    # values of A on the filled pattern, explicit zeros where fill is introduced
    M_data = torch.zeros(nnz, dtype=data.dtype)
    M_data[is_fill == 0] = data
    Mt_data, Mt_indices, Mt_indptr, _ = csr_transpose_forward(n, n, M_data, M_indices, M_indptr)
    getattr(lib(), "oracle_splu_numeric_" + _sfx(data))(_i(n), _p(Mt_data), _p(Mt_indices), _p(Mt_indptr))
    M_data, M_indices, M_indptr, _ = csr_transpose_forward(n, n, Mt_data, Mt_indices, Mt_indptr)
    return [M_data, M_indices, M_indptr, Mt_data, Mt_indices, Mt_indptr]


def spsolve_backward(grad_x, x, rows, cols, Mt_data, Mt_indices, Mt_indptr, A_data, A_indices, A_indptr):
    """grad_b = A^{-T} grad_x by two triangular solves with the transposed factors, grad_A = -(grad_b x^T)
    on the pattern of A (reference cpp/sparse_csr_cpu.cpp:1019-1052)."""
    y = sptrsv_forward(rows, cols, Mt_data, Mt_indices, Mt_indptr, True, False, grad_x)
    grad_b = sptrsv_forward(rows, cols, Mt_data, Mt_indices, Mt_indptr, False, True, y)
    A_indices, A_indptr, x = _c(A_indices, torch.int64), _c(A_indptr, torch.int64), _c(x)
    row_of = torch.repeat_interleave(torch.arange(rows), A_indptr[1:] - A_indptr[:-1])
    grad_A = -(grad_b[row_of] * x[A_indices])
    return [grad_A, grad_b]


def triangle(rows, data, indices, indptr, k, lower):
    """tril (``lower``) / triu of a CSR matrix with ascending columns per row, as the reference's Python
    loops compute it (numml/sparse/_csr.py:234-330): entries with column <= row + k (>= row + k), in
    storage order.  Returns (data, indices, indptr, position in A of every entry kept)."""
    data, indices, indptr = _c(data), _c(indices, torch.int64), _c(indptr, torch.int64)
    row_of = torch.repeat_interleave(torch.arange(rows), indptr[1:] - indptr[:-1])
    keep = (indices <= row_of + k) if lower else (indices >= row_of + k)
    out_ptr = torch.zeros(rows + 1, dtype=torch.int64)
    out_ptr[1:] = torch.cumsum(torch.bincount(row_of[keep], minlength=rows), 0)
    return data[keep], indices[keep], out_ptr, torch.nonzero(keep).flatten()


if __name__ == "__main__":
    print(build(force=True))
