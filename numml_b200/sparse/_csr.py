"""``SparseCSRTensor`` and its differentiable operators: the host-side mirror of the reference's
``numml.sparse`` (reference ``numml/sparse/_csr.py``).  Class, method and autograd ``Function``
names, argument meaning and error behaviour follow the reference so that code written against it
runs unchanged; the hot operators (matrix-vector, matrix-dense, matrix-matrix products and the
transpose) call the CUDA kernels through ``numml_b200.numml_torch_cpp``.

Operators that are not part of the accelerated path (element-wise combination, dense
conversion, row sums, diagonal, triangular parts) are written with ordinary differentiable torch
tensor operations, so they run wherever the tensors live and build patterns without host loops.
"""
import importlib

import numpy as np
import torch

from .. import numml_torch_cpp
from .. import profiler as _profiler
from .. import utils


def _scipy_sparse():
    try:
        return importlib.import_module("scipy.sparse")
    except ImportError:
        return None


sci_sp = _scipy_sparse()


class _NullProfiler:
    def __init__(self, *a, **k):
        pass

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        return False


Profiler = _NullProfiler


def _debug_set_profiler_enabled(val):
    """Wrap every operator call in a nested wall-clock ``Profiler`` section (reference
    ``numml/sparse/_csr.py:57-62``)."""
    global Profiler
    Profiler = _profiler.Profiler if val else _NullProfiler


_NP_TO_TORCH = {np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
                np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64}


def numpy_to_torch_dtype(np_type):
    try:
        return _NP_TO_TORCH[np.dtype(np_type)]
    except (KeyError, TypeError):
        raise RuntimeError(f'Unknown numpy type for conversion: {np_type}.')


def _row_ids(indptr, nnz):
    """Row number of every stored entry."""
    rows = indptr.numel() - 1
    counts = indptr[1:] - indptr[:-1]
    return torch.repeat_interleave(torch.arange(rows, device=indptr.device), counts, output_size=nnz)


def coo_to_csr(values, row_ind, col_ind, shape, sort=True):
    """COO triplets to CSR arrays; with ``sort`` entries are ordered by (row, column) first
    (reference ``numml/sparse/_csr.py:78-99``)."""
    row_ind = row_ind.long()
    col_ind = col_ind.long()
    if values.is_cuda and values.numel() > 0:
        # one stable two-key radix sort on the device (order and row pointers together)
        perm, indptr = numml_torch_cpp.coo_to_csr_order(row_ind, col_ind, int(shape[0]), int(shape[1]), sort_columns=sort)
        return values[perm], col_ind[perm], indptr
    if sort and values.numel() > 0:
        order = torch.argsort(row_ind * int(shape[1]) + col_ind, stable=True)
        values, row_ind, col_ind = values[order], row_ind[order], col_ind[order]
    counts = torch.bincount(row_ind, minlength=int(shape[0]))
    indptr = torch.zeros(int(shape[0]) + 1, dtype=torch.long, device=values.device)
    indptr[1:] = torch.cumsum(counts, 0)
    return values, col_ind, indptr


# ---------------------------------------------------------------------------------------------
# Autograd Functions on the accelerated path
# ---------------------------------------------------------------------------------------------
class spgemv(torch.autograd.Function):
    """Sparse matrix times dense vector (reference ``numml/sparse/_csr.py:102-133``)."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_col_ind, A_rowptr, x):
        if A_data.type() != x.type():
            raise RuntimeError(f'Matrix and vector should be same data type, got {A_data.type()} and {x.type()}, respectively.')
        with Profiler('spgemv forward'):
            Ax = numml_torch_cpp.spgemv_forward(A_shape[0], A_shape[1], A_data, A_col_ind, A_rowptr, x)
        ctx.save_for_backward(x, A_data, A_col_ind, A_rowptr)
        ctx.shape = A_shape
        return Ax

    @staticmethod
    def backward(ctx, df_dz):
        x, A_data, A_col_ind, A_rowptr = ctx.saved_tensors
        with Profiler('spgemv backward'):
            grad_A, grad_x = numml_torch_cpp.spgemv_backward(df_dz, ctx.shape[0], ctx.shape[1],
                                                             A_data, A_col_ind, A_rowptr, x)
        return None, grad_A, None, None, grad_x


class spgemm(torch.autograd.Function):
    """Sparse matrix times sparse matrix (reference ``numml/sparse/_csr.py:136-184``)."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_indices, A_indptr, B_shape, B_data, B_indices, B_indptr):
        if A_data.type() != B_data.type():
            raise RuntimeError(f'Matrices should be same data type, got {A_data.type()} and {B_data.type()}, respectively.')
        if A_shape[1] != B_shape[0]:
            raise RuntimeError(f'Incompatible matrix shapes for multiplication.  Got {A_shape} and {B_shape}.')
        C_shape = (A_shape[0], B_shape[1])
        with Profiler('spgemm forward'):
            C_data, C_indices, C_indptr = numml_torch_cpp.spgemm_forward(
                A_shape[0], A_shape[1], A_data, A_indices, A_indptr,
                B_shape[0], B_shape[1], B_data, B_indices, B_indptr)
        ctx.save_for_backward(A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, C_indices, C_indptr)
        ctx.A_shape, ctx.B_shape = A_shape, B_shape
        ctx.mark_non_differentiable(C_indices, C_indptr)
        return C_shape, C_data, C_indices, C_indptr

    @staticmethod
    def backward(ctx, _gs, grad_C_data, _gi, _gp):
        A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, C_indices, C_indptr = ctx.saved_tensors
        with Profiler('spgemm backward'):
            grad_A, grad_B = numml_torch_cpp.spgemm_backward(
                grad_C_data, C_indices, C_indptr,
                ctx.A_shape[0], ctx.A_shape[1], A_data, A_indices, A_indptr,
                ctx.B_shape[0], ctx.B_shape[1], B_data, B_indices, B_indptr)
        return None, grad_A, None, None, None, grad_B, None, None


class sptranspose(torch.autograd.Function):
    """Eager CSR transpose (reference ``numml/sparse/_csr.py:333-354``)."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_indices, A_indptr):
        with Profiler('sptranspose forward'):
            At_data, At_indices, At_indptr, At_to_A_idx = \
                numml_torch_cpp.csr_transpose_forward(A_shape[0], A_shape[1], A_data, A_indices, A_indptr)
        ctx.save_for_backward(At_to_A_idx)
        ctx.mark_non_differentiable(At_indices, At_indptr)
        return tuple(A_shape[::-1]), At_data, At_indices, At_indptr

    @staticmethod
    def backward(ctx, _gs, grad_At_data, _gi, _gp):
        (At_to_A_idx,) = ctx.saved_tensors
        with Profiler('sptranspose backward'):
            grad_A = numml_torch_cpp.csr_transpose_backward(grad_At_data, At_to_A_idx)
        return None, grad_A, None, None


class spdmm(torch.autograd.Function):
    """Sparse matrix times dense matrix (reference ``numml/sparse/_csr.py:357-387``)."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_indices, A_indptr, B):
        if A_data.type() != B.type():
            raise RuntimeError(f'Matrices should be same data type, got {A_data.type()} and {B.type()}, respectively.')
        if A_shape[1] != B.shape[0]:
            raise RuntimeError(f'Incompatible matrix shapes for multiplication.  Got {A_shape} and {B.shape}.')
        ctx.save_for_backward(A_data, A_indices, A_indptr, B)
        ctx.A_shape = A_shape
        with Profiler('spdmm forward'):
            C = numml_torch_cpp.spdmm_forward(A_shape[0], A_shape[1], A_data, A_indices, A_indptr, B)
        return C

    @staticmethod
    def backward(ctx, grad_C):
        A_data, A_indices, A_indptr, B = ctx.saved_tensors
        with Profiler('spdmm backward'):
            grad_A, grad_B = numml_torch_cpp.spdmm_backward(ctx.A_shape[0], ctx.A_shape[1],
                                                            A_data, A_indices, A_indptr, B, grad_C)
        return None, grad_A, None, None, grad_B


class sprowsum(torch.autograd.Function):
    """Row sums of a CSR matrix (reference ``numml/sparse/_csr.py:416-439``).  On the device this is
    the SpMV kernel applied to the all-ones vector: multiplying by one is exact and the kernel adds
    in storage order, so the sums are those of the reference's sequential loop, bit for bit, and
    do not depend on scheduling (an ``index_add`` would use atomics).  The gradient of a row sum
    with respect to an entry is the upstream value of its row."""

    @staticmethod
    def forward(ctx, A_shape, A_data, A_indices, A_indptr):
        ones = torch.ones(A_shape[1], dtype=A_data.dtype, device=A_data.device)
        with Profiler('sprowsum forward'):
            out = numml_torch_cpp.spgemv_forward(A_shape[0], A_shape[1], A_data, A_indices, A_indptr, ones)
        ctx.save_for_backward(A_indptr)
        ctx.nnz = A_data.numel()
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (A_indptr,) = ctx.saved_tensors
        with Profiler('sprowsum backward'):
            grad_A = grad_out.contiguous()[_row_ids(A_indptr, ctx.nnz)]
        return None, grad_A, None, None


# ---------------------------------------------------------------------------------------------
# Pattern helpers written with torch tensor ops (differentiable through `data`)
# ---------------------------------------------------------------------------------------------
class splincomb(torch.autograd.Function):
    """alpha*A + beta*B on the union pattern (reference ``numml/sparse/_csr.py:187-232``), CUDA tensors."""

    @staticmethod
    def forward(ctx, shape, alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr):
        with Profiler('splincomb forward'):
            C_data, C_indices, C_indptr = numml_torch_cpp.splincomb_forward(
                shape[0], shape[1], alpha, A_data, A_indices, A_indptr, beta, B_data, B_indices, B_indptr)
        ctx.save_for_backward(A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, C_indices, C_indptr)
        ctx.shape, ctx.alpha, ctx.beta = shape, alpha, beta
        ctx.mark_non_differentiable(C_indices, C_indptr)
        return C_data, C_indices, C_indptr

    @staticmethod
    def backward(ctx, grad_C_data, _gi, _gp):
        A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, C_indices, C_indptr = ctx.saved_tensors
        with Profiler('splincomb backward'):
            grad_A, grad_B = numml_torch_cpp.splincomb_backward(
                ctx.shape[0], ctx.shape[1], ctx.alpha, A_data, A_indices, A_indptr, ctx.beta, B_data, B_indices, B_indptr,
                grad_C_data.contiguous(), C_indices, C_indptr)
        return None, None, grad_A, None, None, None, grad_B, None, None


class sptriangle(torch.autograd.Function):
    """tril / triu (reference ``numml/sparse/_csr.py:234-330``) on CUDA tensors; the backward scatters
    the gradient of the kept entries back to their positions in A and leaves zeros elsewhere."""

    @staticmethod
    def forward(ctx, shape, A_data, A_indices, A_indptr, k, lower):
        with Profiler('tril forward' if lower else 'triu forward'):
            data, indices, indptr, pos = numml_torch_cpp.csr_triangle(shape[0], shape[1], A_data, A_indices, A_indptr, k, lower)
        ctx.save_for_backward(pos)
        ctx.nnz = A_data.numel()
        ctx.mark_non_differentiable(indices, indptr)
        return data, indices, indptr

    @staticmethod
    def backward(ctx, grad_data, _gi, _gp):
        (pos,) = ctx.saved_tensors
        grad_A = torch.zeros(ctx.nnz, dtype=grad_data.dtype, device=grad_data.device)
        if pos.numel() > 0:
            grad_A = numml_torch_cpp.scatter_into(grad_A, grad_data.contiguous(), pos)
        return None, grad_A, None, None, None, None


def _lincomb(shape, alpha, A, beta, B):
    """C = alpha*A + beta*B on the union pattern, columns ascending per row."""
    if A.data.is_cuda and not isinstance(alpha, torch.Tensor) and not isinstance(beta, torch.Tensor):
        return splincomb.apply(tuple(shape), alpha, A.data, A.indices, A.indptr, beta, B.data, B.indices, B.indptr)
    rows, cols = int(shape[0]), int(shape[1])
    ra, rb = _row_ids(A.indptr, A.nnz), _row_ids(B.indptr, B.nnz)
    keys = torch.cat((ra * cols + A.indices, rb * cols + B.indices))
    uniq, inverse = torch.unique(keys, sorted=True, return_inverse=True)
    vals = torch.cat((alpha * A.data, beta * B.data))
    data = torch.zeros(uniq.numel(), dtype=vals.dtype, device=vals.device).index_add(0, inverse, vals)
    r = torch.div(uniq, cols, rounding_mode='floor')
    indptr = torch.zeros(rows + 1, dtype=torch.long, device=vals.device)
    indptr[1:] = torch.cumsum(torch.bincount(r, minlength=rows), 0)
    return data, uniq - r * cols, indptr


def _triangle(A, k, lower):
    if A.data.is_cuda:
        return SparseCSRTensor(sptriangle.apply(tuple(A.shape), A.data, A.indices, A.indptr, int(k), bool(lower)), A.shape, clone=False)
    r = _row_ids(A.indptr, A.nnz)
    keep = (A.indices <= r + k) if lower else (A.indices >= r + k)
    indptr = torch.zeros(A.shape[0] + 1, dtype=torch.long, device=A.indptr.device)
    indptr[1:] = torch.cumsum(torch.bincount(r[keep], minlength=A.shape[0]), 0)
    return SparseCSRTensor((A.data[keep], A.indices[keep], indptr), A.shape, clone=False)


def _band(N, k, vals, device):
    n_k = vals.numel()
    if k >= 0:
        rows, cols = torch.arange(n_k, device=device), torch.arange(k, N, device=device)
    else:
        rows, cols = torch.arange(-k, N, device=device), torch.arange(n_k, device=device)
    return SparseCSRTensor((vals, (rows, cols)), shape=(N, N))


def eye(N, k=0, dtype=torch.float32, device='cpu'):
    """Identity (or a shifted diagonal of ones) as a sparse tensor (reference ``_csr.py:467-486``)."""
    if abs(k) >= N:
        raise RuntimeError(f'Specified bandwidth for eye() is larger than matrix size.  Got k={abs(k)}, N={N}.')
    return _band(N, k, torch.ones(N - abs(k), dtype=dtype, device=device), device)


def diag(x, k=0):
    """Sparse matrix with ``x`` on diagonal ``k`` (reference ``_csr.py:489-508``)."""
    return _band(len(x) + abs(k), k, x, x.device)


def spouter(x, y):
    """Outer product x y^T restricted to the nonzeros of x and y (reference ``_csr.py:511-538``)."""
    x_nz = torch.nonzero(x).flatten()
    y_nz = torch.nonzero(y).flatten()
    row, col = torch.meshgrid(x_nz, y_nz, indexing='ij')
    row, col = row.flatten(), col.flatten()
    return SparseCSRTensor((x[row] * y[col], (row, col)), shape=(len(x), len(y)))


def unpack_csr(A):
    return A.data, A.indices, A.indptr, A.shape


def repack_csr(A_data, A_indices, A_indptr, A_shape):
    return SparseCSRTensor((A_data, A_indices, A_indptr), A_shape, clone=False)


def _as_tensor(a, dtype, device):
    if isinstance(a, torch.Tensor):
        t = a
    else:
        t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    if device is not None:
        t = t.to(device)
    return t


class SparseCSRTensor(object):
    """Compressed-sparse-row matrix whose stored values carry gradients.

    Construction follows the reference class (``numml/sparse/_csr.py:549-650``):
    ``SparseCSRTensor(dense)``, ``SparseCSRTensor(torch_sparse_coo)``, ``SparseCSRTensor(scipy_matrix)``,
    ``SparseCSRTensor((data, (row, col)), shape=...)`` and ``SparseCSRTensor((data, indices, indptr), shape=...)``.
    ``indices`` and ``indptr`` are int64 tensors.  Array inputs are converted without passing
    through float32, so float64 values and large offsets are kept exactly.
    """

    def __init__(self, arg1, shape=None, clone=True, dtype=None, device=None):
        if isinstance(arg1, torch.Tensor):
            if arg1.layout == torch.sparse_coo:
                arg1 = arg1.coalesce()
                rows, cols = arg1.indices()
                self.data, self.indices, self.indptr = coo_to_csr(arg1.values(), rows, cols, arg1.shape, sort=True)
            else:
                rows, cols = torch.nonzero(arg1).T
                self.data, self.indices, self.indptr = coo_to_csr(arg1[rows, cols], rows, cols, arg1.shape, sort=True)
            self.shape = tuple(shape) if shape is not None else tuple(arg1.shape)
        elif sci_sp is not None and isinstance(arg1, sci_sp.spmatrix) or (sci_sp is not None and hasattr(sci_sp, 'sparray') and isinstance(arg1, sci_sp.sparray)):
            csr = arg1.tocsr()
            csr.sort_indices()
            if dtype is None:
                dtype = numpy_to_torch_dtype(csr.data.dtype)
            if device is None:
                device = torch.device('cpu')
            self.data = _as_tensor(csr.data.copy(), dtype, device)
            self.indices = _as_tensor(csr.indices.copy(), torch.int64, device)
            self.indptr = _as_tensor(csr.indptr.copy(), torch.int64, device)
            self.shape = tuple(int(s) for s in csr.shape)
        elif isinstance(arg1, tuple):
            assert shape is not None
            if len(arg1) == 3:
                data, indices, indptr = arg1
                if isinstance(data, torch.Tensor) and not clone and dtype is None and device is None:
                    self.data, self.indices, self.indptr = data, indices, indptr
                else:
                    if dtype is None:
                        dtype = data.dtype if isinstance(data, torch.Tensor) else numpy_to_torch_dtype(data.dtype)
                    if device is None:
                        device = data.device if isinstance(data, torch.Tensor) else torch.device('cpu')
                    self.data = _as_tensor(data, dtype, device)
                    self.indices = _as_tensor(indices, torch.int64, device)
                    self.indptr = _as_tensor(indptr, torch.int64, device)
                    if clone:
                        if isinstance(data, torch.Tensor) and self.data.data_ptr() == data.data_ptr():
                            self.data = torch.clone(self.data)
                        if isinstance(indices, torch.Tensor) and self.indices.data_ptr() == indices.data_ptr():
                            self.indices = torch.clone(self.indices)
                        if isinstance(indptr, torch.Tensor) and self.indptr.data_ptr() == indptr.data_ptr():
                            self.indptr = torch.clone(self.indptr)
            elif len(arg1) == 2:
                data, (rows, cols) = arg1
                self.data, self.indices, self.indptr = coo_to_csr(data, rows, cols, shape)
            else:
                raise RuntimeError(f'Unknown tuple given as argument of SparseCSRTensor: length {len(arg1)}')
            self.shape = tuple(int(s) for s in shape)
        else:
            raise RuntimeError(f'Unknown type given as argument of SparseCSRTensor: {type(arg1)}')

    # -- products ----------------------------------------------------------------------------
    def spmv(self, x):
        if self.shape[1] != torch.numel(x):
            raise RuntimeError(f'Number of columns of tensor must equal number of rows of vector.  Got shapes: {self.shape} and {x.shape}')
        y = spgemv.apply(self.shape, self.data, self.indices, self.indptr, x.reshape(-1))
        return utils.unsqueeze_like(y, x)

    def solve_triangular(self, upper, unit, b):
        """Solve this triangular system for ``b`` (1-D, or [n, k] for k right-hand sides).
        ``upper``: the matrix is upper triangular; ``unit``: assume a unit diagonal and ignore
        stored diagonal entries (reference ``numml/sparse/_csr.py:661-680``)."""
        from . import linalg as spla
        return spla.sptrsv.apply(self.shape, self.data, self.indices, self.indptr, not upper, unit, b)

    def spspmm(self, othr):
        C_shape, C_data, C_indices, C_indptr = spgemm.apply(self.shape, self.data, self.indices, self.indptr,
                                                            othr.shape, othr.data, othr.indices, othr.indptr)
        # the kernel's outputs are fresh tensors: wrap them without the extra copy
        return SparseCSRTensor((C_data, C_indices, C_indptr), C_shape, clone=False)

    def spdmm(self, othr):
        return spdmm.apply(self.shape, self.data, self.indices, self.indptr, othr)

    def __matmul__(self, x):
        if isinstance(x, SparseCSRTensor):
            return self.spspmm(x)
        if not isinstance(x, torch.Tensor):
            raise RuntimeError(f'Unknown type for matmul: {type(x)}.')
        dims = x.ndim
        if dims == 0:
            if self.shape == (1, 1):
                return self.data * x.item()
            if self.shape[0] == 1 or self.shape[1] == 1:
                return self.to_dense() * x.item()
            return self * x.item()
        if dims == 1:
            return self.spmv(x)
        if dims == 2:
            return self.spdmm(x)
        if x.shape[-2] == self.shape[1]:
            # batched product: (a_1, ..., a_k, n, b) -> move n first, flatten the rest, multiply once
            x_tr = torch.transpose(x, 0, dims - 2)
            y_fl = self.spdmm(torch.flatten(x_tr, 1).contiguous())
            return torch.transpose(y_fl.reshape((self.shape[0],) + tuple(x_tr.shape[1:])), 0, dims - 2)
        if any(s == 1 for s in x.shape):
            return self.__matmul__(torch.squeeze(x))
        raise RuntimeError(f'invalid tensor found for sparse multiply: mode {dims} tensor found.  Trying to multiply {self.shape} sparse matrix by {x.shape} tensor.')

    # -- conversions ---------------------------------------------------------------------------
    def to_dense(self):
        """Dense copy; gradients flow back to the stored entries."""
        out = torch.zeros(self.shape, dtype=self.data.dtype, device=self.device)
        return out.index_put((_row_ids(self.indptr, self.nnz), self.indices), self.data)

    def to_coo(self):
        idx = torch.stack((_row_ids(self.indptr, self.nnz), self.indices))
        return torch.sparse_coo_tensor(idx, self.data, self.shape, device=self.device)

    def tocoo(self):
        rows = _row_ids(self.indptr, self.nnz).cpu().numpy()
        return sci_sp.coo_matrix((self.data.detach().cpu().numpy(), (rows, self.indices.cpu().numpy())), shape=self.shape)

    def to_scipy_csr(self):
        return sci_sp.csr_matrix((self.data.detach().cpu().numpy(), self.indices.cpu().numpy(),
                                  self.indptr.cpu().numpy()), self.shape)

    def tocsr(self):
        return self.to_scipy_csr()

    # -- reductions ----------------------------------------------------------------------------
    def sum(self):
        return self.data.sum()

    def row_sum(self):
        if self.data.is_cuda:
            return sprowsum.apply(self.shape, self.data, self.indices, self.indptr)
        out = torch.zeros(self.shape[0], dtype=self.data.dtype, device=self.device)
        return out.index_add(0, _row_ids(self.indptr, self.nnz), self.data)

    def diagonal(self):
        r = _row_ids(self.indptr, self.nnz)
        on = r == self.indices
        out = torch.zeros(min(self.shape), dtype=self.data.dtype, device=self.device)
        return out.index_put((r[on],), self.data[on])

    def trace(self):
        return self.diagonal().sum()

    # -- element-wise --------------------------------------------------------------------------
    @staticmethod
    def _isscalar(x):
        return isinstance(x, (float, int)) or (isinstance(x, torch.Tensor) and x.ndim == 0)

    def _with_data(self, data):
        return SparseCSRTensor((data, self.indices, self.indptr), self.shape, clone=False)

    def abs(self):
        return self._with_data(torch.abs(self.data))

    def __abs__(self):
        return self.abs()

    def __add__(self, othr):
        if SparseCSRTensor._isscalar(othr):
            return self._with_data(self.data + othr)
        if isinstance(othr, SparseCSRTensor):
            if tuple(self.shape) != tuple(othr.shape):
                raise RuntimeError(f'Incompatible shapes for entrywise addition, got {self.shape} and {othr.shape}, respectively.')
            return SparseCSRTensor(_lincomb(self.shape, 1., self, 1., othr), self.shape, clone=False)
        raise RuntimeError(f'Unknown type for sparse tensor addition: {type(othr)}.')

    def __sub__(self, othr):
        if SparseCSRTensor._isscalar(othr):
            return self._with_data(self.data - othr)
        if isinstance(othr, SparseCSRTensor):
            if tuple(self.shape) != tuple(othr.shape):
                raise RuntimeError(f'Incompatible shapes for entrywise subtraction, got {self.shape} and {othr.shape}, respectively.')
            return SparseCSRTensor(_lincomb(self.shape, 1., self, -1., othr), self.shape, clone=False)
        raise RuntimeError(f'Unknown type for sparse tensor addition: {type(othr)}.')

    def __mul__(self, other):
        if SparseCSRTensor._isscalar(other):
            return self._with_data(self.data * other)
        if isinstance(other, torch.Tensor) and len(torch.squeeze(other).shape) == 2:
            raise RuntimeError('Element-wise hadamard product not implemented')
        raise RuntimeError(f'Unknown type for multiplication: {type(other)}.')

    def __rmul__(self, other):
        return self.__mul__(other)

    def __rtruediv__(self, other):
        if SparseCSRTensor._isscalar(other):
            return self._with_data(other / self.data)
        raise RuntimeError(f'Unknown type for right-division: {type(other)}.')

    def __neg__(self):
        return self._with_data(-self.data)

    def __pow__(self, p):
        return self._with_data(self.data ** p)

    def conjugate(self):
        return self._with_data(self.data.conj())

    def conj(self):
        return self.conjugate()

    def __repr__(self):
        grad_str = ''
        if self.data.grad_fn is not None:
            grad_str = f', grad_fn=<{self.data.grad_fn.__class__.__name__}>'
        elif self.requires_grad:
            grad_str = ', requires_grad=True'
        dev_str = f", device='{self.device}'" if self.device.type != 'cpu' else ''
        return (f"<{self.shape[0]}x{self.shape[1]} sparse matrix tensor of type '{self.data.dtype}'\n"
                f"\twith {len(self.data)} stored elements in Compressed Sparse Row format{dev_str}{grad_str}>")

    # -- copies, gradients, properties -----------------------------------------------------
    def clone(self):
        return SparseCSRTensor((self.data, self.indices, self.indptr), shape=self.shape)

    def copy(self):
        return self.clone()

    def detach(self):
        return self._with_data(self.data.detach())

    @property
    def requires_grad(self):
        return self.data.requires_grad

    @requires_grad.setter
    def requires_grad(self, b):
        self.data.requires_grad = b

    @property
    def grad(self):
        return SparseCSRTensor((self.data.grad, self.indices, self.indptr), shape=self.shape, clone=False)

    @property
    def grad_fn(self):
        return self.data.grad_fn

    @property
    def nnz(self):
        """Number of stored values, explicit zeros included."""
        return len(self.data)

    @property
    def diagonal_idx(self):
        """idx[i] = position of the diagonal entry of row i in ``data``, or -1."""
        r = _row_ids(self.indptr, self.nnz)
        on = r == self.indices
        idx = torch.full((min(self.shape),), -1, dtype=torch.long, device=self.device)
        idx[r[on]] = torch.nonzero(on).flatten()
        return idx

    @property
    def row_indices(self):
        return _row_ids(self.indptr, self.nnz)

    def tril(self, k=0):
        return _triangle(self, k, lower=True)

    def triu(self, k=0):
        return _triangle(self, k, lower=False)

    def transpose(self):
        """Eager transpose (there is no lazy CSC view)."""
        At_shape, At_data, At_indices, At_indptr = sptranspose.apply(self.shape, self.data, self.indices, self.indptr)
        return SparseCSRTensor((At_data, At_indices, At_indptr), At_shape, clone=False)

    def hermitian(self):
        At_shape, At_data, At_indices, At_indptr = sptranspose.apply(self.shape, self.data.conj(), self.indices, self.indptr)
        return SparseCSRTensor((At_data, At_indices, At_indptr), At_shape, clone=False)

    @property
    def T(self):
        return self.transpose()

    @property
    def H(self):
        return self.hermitian()

    @property
    def device(self):
        assert self.data.device == self.indptr.device and self.indptr.device == self.indices.device
        return self.data.device

    @property
    def dtype(self):
        return self.data.dtype

    def to(self, device):
        return SparseCSRTensor((self.data.to(device), self.indices.to(device), self.indptr.to(device)), self.shape, clone=False)

    def cuda(self, device=None):
        return self.to(torch.device('cuda', torch.cuda.current_device() if device is None else device))

    def cpu(self):
        return self.to('cpu')

    def float(self):
        return self._with_data(self.data.float())

    def double(self):
        return self._with_data(self.data.double())
