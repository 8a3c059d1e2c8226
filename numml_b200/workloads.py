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

    The entries of a row are laid out in ascending order of their column offset, so masking out
    the neighbours that fall off the grid leaves every row sorted without a sort.
    """
    dims = tuple(int(d) for d in dims)
    ntot = int(np.prod(dims))
    lo, hi = (0, ntot) if row_range is None else (int(row_range[0]), int(row_range[1]))
    n = hi - lo
    strides = [int(np.prod(dims[k + 1:])) for k in range(len(dims))]
    ids = torch.arange(lo, hi, dtype=torch.int64)
    coords = [((ids // strides[k]) % dims[k]).to(torch.int32) for k in range(len(dims))]
    entries = [(0, None, diag_val)]
    for off in offsets:
        delta = sum(o * s for o, s in zip(off, strides))
        if lower_only and delta > 0:
            continue
        entries.append((delta, off, off_val))
    entries.sort(key=lambda e: e[0])
    valid = torch.ones((n, len(entries)), dtype=torch.bool)
    for q, (_, off, _) in enumerate(entries):
        for k, o in enumerate(off or ()):
            if o > 0:
                valid[:, q] &= coords[k] < dims[k] - o
            elif o < 0:
                valid[:, q] &= coords[k] >= -o
    indptr = torch.zeros(n + 1, dtype=torch.int64)
    torch.cumsum(valid.sum(dim=1), 0, out=indptr[1:])
    deltas = torch.tensor([e[0] for e in entries], dtype=torch.int64)
    row_vals = torch.tensor([e[2] for e in entries], dtype=dtype)
    cols = (ids[:, None] + deltas[None, :])[valid]
    vals = row_vals.expand(n, len(entries))[valid]
    return vals.contiguous(), cols.contiguous(), indptr, (n, ntot)


def poisson2d_5pt(n, dtype=torch.float32, row_range=None):
    """5-point Laplacian on an n x n grid: 4 on the diagonal, -1 off; nnz = 5n^2 - 4n.
    ``row_range`` builds a block of rows only (global columns)."""
    return _stencil((n, n), [(-1, 0), (0, -1), (0, 1), (1, 0)], 4.0, -1.0, dtype, row_range=row_range)


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


def row_block(data, indices, indptr, lo, hi):
    """Rows lo..hi-1 of a CSR matrix as a CSR matrix of their own (columns unchanged)."""
    a, b = int(indptr[lo]), int(indptr[hi])
    return data[a:b].contiguous(), indices[a:b].contiguous(), (indptr[lo:hi + 1] - a).contiguous()


def rows_subset(data, indices, indptr, rows):
    """The given rows (a 1-D int64 tensor, any order) of a CSR matrix as a CSR matrix of their own,
    plus the storage position in the original arrays of every entry taken."""
    lens = (indptr[1:] - indptr[:-1])[rows]
    ptr = torch.zeros(rows.numel() + 1, dtype=torch.int64)
    torch.cumsum(lens, 0, out=ptr[1:])
    pos = torch.repeat_interleave(indptr[rows] - ptr[:-1], lens) + torch.arange(int(ptr[-1]))
    return data[pos].contiguous(), indices[pos].contiguous(), ptr, pos


def randn(shape, seed, dtype):
    """N(0,1) tensor from a seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=dtype)
