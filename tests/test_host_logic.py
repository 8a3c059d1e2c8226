"""CPU tests of the host-side mirror of numml.sparse: constructors, pattern helpers written
with torch ops, error behaviour, and the refusal to run the accelerated operators on CPU."""
import numpy as np
import pytest
import scipy.sparse as sps
import torch

import numml_b200.sparse as sp
from numml_b200 import workloads as W


def test_constructors_agree():
    d = torch.tensor([[1., 0., 2.], [0., 0., 3.], [4., 5., 0.]])
    A = sp.SparseCSRTensor(d)
    assert A.indptr.tolist() == [0, 2, 3, 5] and A.indices.tolist() == [0, 2, 2, 0, 1]
    B = sp.SparseCSRTensor(d.to_sparse())
    C = sp.SparseCSRTensor(sps.csr_matrix(d.numpy()))
    r, c = torch.nonzero(d).T
    D = sp.SparseCSRTensor((d[r, c], (r, c)), shape=(3, 3))
    E = sp.SparseCSRTensor((A.data, A.indices, A.indptr), shape=(3, 3))
    for M in (B, C, D, E):
        assert torch.equal(M.to_dense(), d)
    assert E.data.data_ptr() != A.data.data_ptr()          # clone=True copies
    F = sp.SparseCSRTensor((A.data, A.indices, A.indptr), shape=(3, 3), clone=False)
    assert F.data.data_ptr() == A.data.data_ptr()


def test_array_constructor_keeps_float64_and_large_offsets():
    """The reference rounds numpy inputs through float32 (numml/sparse/_csr.py:598-600); here
    float64 values and offsets above 2**24 survive exactly."""
    data = np.array([1.0 + 2.0 ** -40, 2.0])
    A = sp.SparseCSRTensor((data, np.array([0, 1]), np.array([0, 1, 2])), shape=(2, 2))
    assert A.data.dtype == torch.float64 and A.data[0].item() == data[0]
    big = np.array([0, 2 ** 24 + 1], dtype=np.int64)
    B = sp.SparseCSRTensor((np.zeros(0), np.zeros(0, dtype=np.int64), big), shape=(1, 1))
    assert B.indptr[1].item() == 2 ** 24 + 1


def test_elementwise_and_patterns():
    n = 6
    A = sp.eye(n) * 2 - sp.eye(n, k=-1) - sp.eye(n, k=1)
    dense = 2 * torch.eye(n) - torch.diag(torch.ones(n - 1), -1) - torch.diag(torch.ones(n - 1), 1)
    assert torch.equal(A.to_dense(), dense)
    assert torch.equal(A.tril().to_dense(), torch.tril(dense))
    assert torch.equal(A.triu(1).to_dense(), torch.triu(dense, 1))
    assert torch.equal(A.row_sum(), dense.sum(1))
    assert torch.equal(A.diagonal(), torch.diag(dense))
    assert A.trace().item() == 12
    assert torch.equal((A + A).to_dense(), 2 * dense)
    assert torch.equal(abs(-A).to_dense(), dense.abs())
    assert torch.equal((A ** 2).to_dense(), dense ** 2)
    assert A.diagonal_idx.tolist() == [0, 3, 6, 9, 12, 15]
    assert torch.equal(sp.diag(torch.arange(1., 4.), k=1).to_dense(), torch.diag(torch.arange(1., 4.), 1))
    with pytest.raises(RuntimeError, match="bandwidth"):
        sp.eye(3, k=3)
    with pytest.raises(RuntimeError, match="Incompatible shapes"):
        A + sp.eye(n + 1)


def test_pattern_helpers_are_differentiable():
    A = sp.eye(4, dtype=torch.float64) * 3 - sp.eye(4, k=1, dtype=torch.float64)
    A.requires_grad = True
    (A.to_dense() * torch.arange(16.).reshape(4, 4)).sum().backward()
    assert A.data.grad is not None and A.data.grad.shape == A.data.shape
    B = A.detach()
    B.requires_grad = True
    B.tril().sum().backward()
    assert B.data.grad.sum().item() == 4    # only the diagonal survives tril


def test_scipy_round_trip():
    d, i, p, shape = W.random_csr(20, 30, 0.2, seed=1)
    A = sp.SparseCSRTensor((d, i, p), shape)
    S = A.to_scipy_csr()
    assert (S != sps.csr_matrix((d.numpy(), i.numpy(), p.numpy()), shape=shape)).nnz == 0
    assert A.tocoo().nnz == A.nnz


def test_accelerated_operators_refuse_cpu_tensors():
    A = sp.eye(4)
    with pytest.raises(RuntimeError, match="CUDA"):
        A @ torch.ones(4)
    with pytest.raises(RuntimeError, match="CUDA"):
        A @ A
    with pytest.raises(RuntimeError, match="CUDA"):
        A.T
    with pytest.raises(RuntimeError, match="CUDA"):
        A.solve_triangular(False, False, torch.ones(4))
    with pytest.raises(RuntimeError, match="Unknown type"):
        A @ "x"


def test_lu_has_no_cpu_path():
    import numml_b200.sparse.linalg as spla
    with pytest.raises(RuntimeError, match="CUDA"):
        spla.splu(sp.eye(3))
    with pytest.raises(RuntimeError, match="CUDA"):
        spla.spsolve(sp.eye(3), torch.ones(3))


def test_linear_operator_and_profiler(capsys):
    L = sp.LinearOperator((3, 3), rm=lambda v: 2 * v, lm=lambda v: 3 * v)
    assert torch.equal(L @ torch.ones(3), 2 * torch.ones(3))
    assert torch.equal(torch.ones(3) @ L, 3 * torch.ones(3))
    from numml_b200.profiler import Profiler
    with Profiler("outer"):
        with Profiler("inner"):
            pass
    out = capsys.readouterr().out
    assert "[outer]" in out and "  [inner]" in out


def test_triangular_solve_team_size_follows_level_width():
    """Lanes per row for the triangular solve: a whole warp when the dependency levels are narrow
    (latency-bound), fewer lanes as the average level gets wide enough to fill the GPU by itself."""
    from numml_b200 import numml_torch_cpp as ops
    assert ops._team_lanes(1 << 20, 3070) == 32            # 9-point factor on a 1024^2 grid: 341 rows per level
    assert ops._team_lanes(1000, 1000) == 32               # a chain
    assert ops._team_lanes(1 << 20, 1) == 1                # diagonal matrix: one level holds every row
    wide = ops._team_lanes(1 << 22, 100)                   # 42 k rows per level
    assert wide in (1, 2, 4, 8) and 42000 * wide <= 148 * 2048 < 42000 * wide * 2
    assert ops._team_lanes(5, 0) == 32                     # no levels recorded (empty matrix): harmless


def test_row_range_hint_names_the_streaming_kernel_for_sub_ranges():
    """A launch over a proper sub-range of rows must not let nnz / rows pick the kernel: it asks for the
    row-streaming kernel (-1) unless the pipelined kernel applies (plan allows it, range starts on a block)."""
    from numml_b200.distributed import DistSpMVEngine as E
    assert E._row_range_hint(0, 100, 100, 0) == 0          # the whole matrix: the library chooses
    assert E._row_range_hint(0, 50, 100, 0) == -1
    assert E._row_range_hint(256, 512, 1000, 128) == 128
    assert E._row_range_hint(100, 512, 1000, 128) == -1    # does not start on a row block
    assert E._row_range_hint(0, 100, 100, -1) == -1
