"""Seeded synthetic CSR workloads used by the benchmark and the parity tests.

Everything is built with numpy integer arithmetic and returned as CPU torch tensors
``(data, indices[int64], indptr[int64], shape)``.  Matrices are always handed to
``SparseCSRTensor`` as a 3-tuple of torch tensors: the reference's scipy / ndarray constructor
branches round through float32 (reference ``numml/sparse/_csr.py:598-600,613,626,634``).
"""
import numpy as np
import torch


def _pack(data, indices, indptr, shape, dtype):
    return (torch.from_numpy(np.ascontiguousarray(data)).to(dtype),
            torch.from_numpy(np.ascontiguousarray(indices).astype(np.int64)),
            torch.from_numpy(np.ascontiguousarray(indptr).astype(np.int64)),
            (int(shape[0]), int(shape[1])))


def _stencil(dims, offsets, diag_val, off_val, dtype, lower_only=False, row_range=None):
    """Dirichlet stencil on a regular grid in natural (row-major) ordering.

    dims      : grid extents, slowest index first
    offsets   : list of index-offset tuples, excluding the centre
    row_range : (lo, hi) builds only rows lo..hi-1 (columns stay global); the returned shape is
                (hi - lo, number of grid points)
    """
    dims = tuple(int(d) for d in dims)
    ntot = int(np.prod(dims))
    lo, hi = (0, ntot) if row_range is None else (int(row_range[0]), int(row_range[1]))
    ids = np.arange(lo, hi, dtype=np.int64)
    n = hi - lo
    coords = np.unravel_index(ids, dims)
    strides = [int(np.prod(dims[k + 1:])) for k in range(len(dims))]
    cols = [ids]
    vals = [np.full(n, diag_val, dtype=np.float64)]
    valid = [np.ones(n, dtype=bool)]
    for off in offsets:
        ok = np.ones(n, dtype=bool)
        delta = 0
        for k, o in enumerate(off):
            c = coords[k] + o
            ok &= (c >= 0) & (c < dims[k])
            delta += o * strides[k]
        if lower_only and delta > 0:
            continue
        cols.append(ids + delta)
        vals.append(np.full(n, off_val, dtype=np.float64))
        valid.append(ok)
    cols = np.stack(cols, axis=1)
    vals = np.stack(vals, axis=1)
    valid = np.stack(valid, axis=1)
    order = np.argsort(np.where(valid, cols, np.iinfo(np.int64).max), axis=1, kind="stable")
    cols = np.take_along_axis(cols, order, axis=1)
    vals = np.take_along_axis(vals, order, axis=1)
    valid = np.take_along_axis(valid, order, axis=1)
    counts = valid.sum(axis=1)
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=indptr[1:])
    return _pack(vals[valid], cols[valid], indptr, (n, ntot), dtype)


def poisson2d_5pt(n, dtype=torch.float32):
    """5-point Laplacian on an n x n grid: 4 on the diagonal, -1 off; nnz = 5n^2 - 4n."""
    return _stencil((n, n), [(-1, 0), (0, -1), (0, 1), (1, 0)], 4.0, -1.0, dtype)


def poisson3d_7pt(n, dtype=torch.float64, nz=None, row_range=None):
    """7-point Laplacian on an nz x n x n grid (nz = n by default): 6 on the diagonal, -1 off;
    nnz = 7n^3 - 6n^2 for the cube.  ``row_range`` builds a block of rows only (global columns)."""
    offs = [(-1, 0, 0), (0, -1, 0), (0, 0, -1), (0, 0, 1), (0, 1, 0), (1, 0, 0)]
    return _stencil((n if nz is None else nz, n, n), offs, 6.0, -1.0, dtype, row_range=row_range)


def poisson2d_9pt_lower(n, dtype=torch.float64):
    """Lower triangle (diagonal included) of the 9-point Laplacian on an n x n grid:
    8 on the diagonal, -1 off; nnz = 5n^2 - 6n + 2."""
    offs = [(a, b) for a in (-1, 0, 1) for b in (-1, 0, 1) if (a, b) != (0, 0)]
    return _stencil((n, n), offs, 8.0, -1.0, dtype, lower_only=True)


def aggregation_2x2(n, dtype=torch.float64):
    """Piecewise-constant aggregation of 2x2 blocks of an n x n grid: (n^2) x (n/2)^2, one 1.0
    per row, P[(r,c), (r//2)*(n/2) + c//2] = 1."""
    assert n % 2 == 0
    r, c = np.divmod(np.arange(n * n, dtype=np.int64), n)
    cols = (r // 2) * (n // 2) + (c // 2)
    return _pack(np.ones(n * n), cols, np.arange(n * n + 1, dtype=np.int64), (n * n, (n // 2) ** 2), dtype)


def powerlaw_graph(n, alpha=2.1, scale=4, max_deg=4096, seed=0, dtype=torch.float32):
    """Row-normalised adjacency of a synthetic power-law graph.

    Out-degree of node i is clip(scale * Zipf(alpha), 1, max_deg) (scale=4 gives a mean near 16,
    scale=1 is the literal clipped Zipf with mean near 4); targets are uniform over [0, n) from a
    second generator; duplicate targets within a row are merged and the row's columns sorted;
    every stored value is 1/deg_i after merging.
    """
    z = np.random.default_rng(seed).zipf(alpha, n)
    deg = np.clip(scale * z, 1, min(max_deg, n)).astype(np.int64)
    total = int(deg.sum())
    rows = np.repeat(np.arange(n, dtype=np.int64), deg)
    cols = np.random.default_rng(seed + 1).integers(0, n, size=total, dtype=np.int64)
    key = np.unique(rows * n + cols)            # sorts by (row, col) and merges duplicates
    rows, cols = np.divmod(key, n)
    counts = np.bincount(rows, minlength=n)
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=indptr[1:])
    vals = 1.0 / np.repeat(counts, counts).astype(np.float64)
    return _pack(vals, cols, indptr, (n, n), dtype)


def random_csr(rows, cols, density, seed=0, dtype=torch.float64, empty_rows=True):
    """Random sparse matrix with N(0,1) values, sorted unique columns per row; when
    ``empty_rows`` a tenth of the rows are emptied to exercise ragged structure."""
    rng = np.random.default_rng(seed)
    nnz_target = int(np.ceil(density * rows * cols))
    r = rng.integers(0, rows, size=nnz_target, dtype=np.int64)
    c = rng.integers(0, cols, size=nnz_target, dtype=np.int64)
    if empty_rows and rows > 4:
        dead = rng.choice(rows, size=max(1, rows // 10), replace=False)
        keep = ~np.isin(r, dead)
        r, c = r[keep], c[keep]
    key = np.unique(r * cols + c)
    r, c = np.divmod(key, cols)
    counts = np.bincount(r, minlength=rows)
    indptr = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(counts, out=indptr[1:])
    vals = rng.standard_normal(len(c))
    return _pack(vals, c, indptr, (rows, cols), dtype)


def random_triangular(n, density, lower=True, seed=0, dtype=torch.float64, diag=2.0, with_diag=True):
    """Random triangular matrix: strictly-triangular N(0,1) entries scaled by 1/sqrt(row length)
    (keeps the solve well conditioned) plus, when ``with_diag``, a constant diagonal."""
    rng = np.random.default_rng(seed)
    m = int(np.ceil(density * n * n))
    r = rng.integers(0, n, size=m, dtype=np.int64)
    c = rng.integers(0, n, size=m, dtype=np.int64)
    lo, hi = np.minimum(r, c), np.maximum(r, c)
    keep = lo != hi
    r, c = (hi[keep], lo[keep]) if lower else (lo[keep], hi[keep])
    if with_diag:
        r = np.concatenate([r, np.arange(n, dtype=np.int64)])
        c = np.concatenate([c, np.arange(n, dtype=np.int64)])
    key = np.unique(r * n + c)
    r, c = np.divmod(key, n)
    counts = np.bincount(r, minlength=n)
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=indptr[1:])
    vals = rng.standard_normal(len(c)) / np.sqrt(np.repeat(np.maximum(counts, 1), counts))
    vals[r == c] = diag
    return _pack(vals, c, indptr, (n, n), dtype)


def randn(shape, seed, dtype):
    """N(0,1) tensor from a seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=dtype)
