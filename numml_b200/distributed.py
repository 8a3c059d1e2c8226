"""Row-block partitioned sparse operators over ``torch.distributed`` (one process per GPU).

The reference has no multi-device path at all; this module adds the one the hot path shards
along: contiguous row blocks of A (and of every vector / dense operand / second sparse factor),
with one exchange step per operator:

  * SpMV / SpMM forward: the entries (rows) of x that a rank's columns refer to but another rank
    owns are packed by the owner and sent point to point; they land in the rank's own memory,
    behind its local part, before the local kernel runs.  Columns are renumbered to
    ``[local | halo]`` once, when the partition is built.
  * SpMV / SpMM backward: grad_A is local; grad_x gets contributions for halo columns, which are
    sent back to their owners and added in a fixed peer order (deterministic).
  * SpGEMM: the rows of B that a rank's columns refer to are fetched from their owners (row
    lengths, then indices and values); the local product's rows concatenate to the single-device
    result bit for bit, since output rows are independent.  Backward: grad_A is local; gradients
    of fetched rows of B are sent back to their owners and added there.

All exchanges are grouped ``isend`` / ``irecv`` calls (NCCL over NVLink on GPUs, gloo on CPU);
the local compute goes through an operator module with the reference's function names
(``numml_b200.numml_torch_cpp`` by default), which lets the host logic be exercised on CPU
ranks with a CPU implementation of the same functions injected by the tests.
The triangular solve does not shard (its dependency chain spans the matrix).
"""
import os
import sys

import torch
import torch.distributed as dist


def partition_rows(n, world, indptr=None):
    """Bounds of ``world`` contiguous row blocks: equal row counts, or equal nonzero counts when
    the global ``indptr`` is given (for skewed row lengths)."""
    if indptr is None:
        return [(n * r) // world for r in range(world + 1)]
    nnz = int(indptr[-1])
    targets = torch.tensor([(nnz * r) // world for r in range(1, world)], dtype=indptr.dtype)
    cuts = torch.searchsorted(indptr, targets, right=False).tolist()
    bounds = [0] + [min(max(int(c), 0), n) for c in cuts] + [n]
    for r in range(1, world + 1):
        bounds[r] = max(bounds[r], bounds[r - 1])
    return bounds


def _take(x, idx):
    """x[idx] along dim 0 (the pack step of an exchange)."""
    if x.is_cuda and x.ndim == 1 and x.dtype in (torch.float32, torch.float64):
        import ctypes
        from . import _cabi
        out = torch.empty(idx.numel(), dtype=x.dtype, device=x.device)
        _cabi.call("nb200_gather", idx.numel(), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(idx.data_ptr()),
                   ctypes.c_void_p(out.data_ptr()), _cabi.F64 if x.dtype == torch.float64 else _cabi.F32, _cabi.I64,
                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        return out
    return x.index_select(0, idx)


class HaloPlan:
    """Who needs which of my entries, and where the entries I need arrive.

    ``need[p]``  sorted global column ids this rank reads and rank p owns (p != rank)
    ``send[p]``  local indices (into this rank's block) that rank p reads
    Halo slot of a needed column = n_local + its rank among all needed columns in ascending
    global order; since blocks are contiguous and ordered, the slots of one owner are contiguous.
    """

    def __init__(self, needed_cols, col_bounds, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.col_bounds = list(col_bounds)
        self.lo, self.hi = self.col_bounds[self.rank], self.col_bounds[self.rank + 1]
        self.n_local = self.hi - self.lo
        dev = needed_cols.device
        bounds_t = torch.tensor(self.col_bounds, dtype=torch.int64, device=dev)
        owner = torch.searchsorted(bounds_t, needed_cols, right=True) - 1
        self.halo_cols = needed_cols
        self.n_halo = int(needed_cols.numel())
        self.need = [needed_cols[owner == p] for p in range(self.world)]
        counts = torch.tensor([int(t.numel()) for t in self.need], dtype=torch.int64, device=dev)
        self.recv_counts = counts.tolist()
        self.recv_offsets = [0]
        for c in self.recv_counts:
            self.recv_offsets.append(self.recv_offsets[-1] + c)
        # tell every owner how many / which of its entries this rank needs
        all_counts = [torch.empty_like(counts) for _ in range(self.world)]
        dist.all_gather(all_counts, counts, group=group)
        self.send_counts = [int(all_counts[p][self.rank]) for p in range(self.world)]
        self.send = [torch.empty(self.send_counts[p], dtype=torch.int64, device=dev) for p in range(self.world)]
        ops = []
        for p in range(self.world):
            if p == self.rank:
                continue
            if self.recv_counts[p] > 0:
                ops.append(dist.P2POp(dist.isend, self.need[p].contiguous(), self._peer(p), group=group))
            if self.send_counts[p] > 0:
                ops.append(dist.P2POp(dist.irecv, self.send[p], self._peer(p), group=group))
        self._run(ops)
        for p in range(self.world):
            self.send[p] = self.send[p] - self.lo
        self.peers_in = [p for p in range(self.world) if p != self.rank and self.recv_counts[p] > 0]
        self.peers_out = [p for p in range(self.world) if p != self.rank and self.send_counts[p] > 0]

    def _peer(self, p):
        return p if self.group is None else dist.get_global_rank(self.group, p)

    @staticmethod
    def _run(ops):
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def extend(self, x_local):
        """[x_local | halo entries fetched from their owners], rows along dim 0."""
        tail = tuple(x_local.shape[1:])
        x_ext = torch.empty((self.n_local + self.n_halo,) + tail, dtype=x_local.dtype, device=x_local.device)
        x_ext[:self.n_local] = x_local
        ops, keep = [], []
        for p in self.peers_out:
            buf = _take(x_local, self.send[p])
            keep.append(buf)
            ops.append(dist.P2POp(dist.isend, buf, self._peer(p), group=self.group))
        for p in self.peers_in:
            a = self.n_local + self.recv_offsets[p]
            ops.append(dist.P2POp(dist.irecv, x_ext[a:a + self.recv_counts[p]], self._peer(p), group=self.group))
        self._run(ops)
        return x_ext

    def reduce(self, g_ext):
        """Inverse of ``extend`` for gradients: the halo part of g_ext is sent back to the owners
        and added to their local part (peers in ascending order, so the sum is reproducible)."""
        g_local = g_ext[:self.n_local].clone()
        ops, bufs = [], {}
        for p in self.peers_in:
            a = self.n_local + self.recv_offsets[p]
            ops.append(dist.P2POp(dist.isend, g_ext[a:a + self.recv_counts[p]].contiguous(), self._peer(p), group=self.group))
        for p in self.peers_out:
            bufs[p] = torch.empty((self.send_counts[p],) + tuple(g_ext.shape[1:]), dtype=g_ext.dtype, device=g_ext.device)
            ops.append(dist.P2POp(dist.irecv, bufs[p], self._peer(p), group=self.group))
        self._run(ops)
        for p in self.peers_out:
            g_local.index_add_(0, self.send[p], bufs[p])
        return g_local


class _DistMatVec(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, data, x_local):
        rows = _row_exchange(A, x_local)
        x_ext = rows.extend(x_local.detach()) if rows is not None else A.halo.extend(x_local.detach())
        ctx.A, ctx.rows = A, rows
        ctx.save_for_backward(data, x_ext)
        n_ext = A.halo.n_local + A.halo.n_halo
        if x_local.ndim == 1:
            return A.ops.spgemv_forward(A.n_rows, n_ext, data, A.indices, A.indptr, x_ext)
        return A.ops.spdmm_forward(A.n_rows, n_ext, data, A.indices, A.indptr, x_ext)

    @staticmethod
    def backward(ctx, g):
        A = ctx.A
        data, x_ext = ctx.saved_tensors
        n_ext = A.halo.n_local + A.halo.n_halo
        g = g.contiguous()
        if x_ext.ndim == 1:
            grad_A, grad_x_ext = A.ops.spgemv_backward(g, A.n_rows, n_ext, data, A.indices, A.indptr, x_ext)
        else:
            grad_A, grad_x_ext = A.ops.spdmm_backward(A.n_rows, n_ext, data, A.indices, A.indptr, x_ext, g)
        if ctx.rows is not None:
            return None, grad_A, ctx.rows.reduce(grad_x_ext)
        return None, grad_A, A.halo.reduce(grad_x_ext)


class DistSparseCSR:
    """This rank's block of rows of a row-partitioned CSR matrix.

    ``data, indices, indptr`` hold the rows ``row_bounds[rank] .. row_bounds[rank+1]`` with GLOBAL
    column ids; ``col_bounds`` is the partition of the column space (the partition of x; equal to
    ``row_bounds`` for a square matrix).  Construction renumbers the columns to
    ``[local | halo]`` and builds the exchange plan (collective over ``group``).
    """

    def __init__(self, data, indices, indptr, global_shape, row_bounds, col_bounds=None, group=None, ops=None):
        if ops is None:
            from . import numml_torch_cpp as ops
        self.ops = ops
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.global_shape = tuple(global_shape)
        self.row_bounds = list(row_bounds)
        self.col_bounds = list(col_bounds) if col_bounds is not None else list(row_bounds)
        self.n_rows = self.row_bounds[self.rank + 1] - self.row_bounds[self.rank]
        lo, hi = self.col_bounds[self.rank], self.col_bounds[self.rank + 1]
        self.data = data
        self.global_indices = indices
        self.indptr = indptr
        remote = (indices < lo) | (indices >= hi)
        needed = torch.unique(indices[remote])                    # sorted ascending
        self.halo = HaloPlan(needed, self.col_bounds, group)
        local_ids = torch.where(remote, (hi - lo) + torch.searchsorted(needed, indices), indices - lo)
        self.indices = local_ids.contiguous()

    @property
    def requires_grad(self):
        return self.data.requires_grad

    @requires_grad.setter
    def requires_grad(self, b):
        self.data.requires_grad = b

    def __matmul__(self, x_local):
        """A @ x for this rank's rows; ``x_local`` is this rank's block of x (vector or [n, K])."""
        if isinstance(x_local, DistSparseCSR):
            return dist_spgemm(self, x_local)
        return _DistMatVec.apply(self, self.data, x_local)


def dist_dot(a, b, group=None):
    s = torch.dot(a, b)
    dist.all_reduce(s, group=group)
    return s


def dist_conjugate_gradient(A, b_local, iterations, x_local=None):
    """Unpreconditioned CG on a row-partitioned SPD matrix with a fixed iteration count (the
    recurrence of ``numml_b200.krylov.conjugate_gradient``; dot products are all-reduced).
    Returns this rank's block of the solution and the residual-norm history."""
    group = A.group
    x = torch.zeros_like(b_local) if x_local is None else x_local
    r = b_local.clone() if x_local is None else b_local - (A @ x)
    p = r.clone()
    rz = dist_dot(r, r, group)
    hist = [torch.sqrt(rz)]
    for _ in range(iterations):
        Ap = A @ p
        alpha = rz / dist_dot(Ap, p, group)
        x = x + alpha * p
        r = r - alpha * Ap
        rz_new = dist_dot(r, r, group)
        p = r + (rz_new / rz) * p
        rz = rz_new
        hist.append(torch.sqrt(rz))
    return x, torch.stack(hist)


class _FetchedRows:
    """Structure of the rows of B that A's halo columns refer to, fetched once per pair of patterns:
    the column indices and row pointers of the fetched rows, the extended structure ``[B_local ; fetched
    rows]``, for every peer served the positions in this rank's B arrays of the entries it reads, and
    for every peer read from the range of fetched entries that it owns.  Values travel per call."""

    def __init__(self, A, B):
        halo = A.halo
        dev = B.indptr.device
        lens_local = (B.indptr[1:] - B.indptr[:-1])
        lens_ext = halo.extend(lens_local)                       # row lengths of [local | halo] rows
        indptr = torch.zeros(halo.n_halo + 1, dtype=torch.int64, device=dev)
        indptr[1:] = torch.cumsum(lens_ext[halo.n_local:], 0)
        bounds = indptr.cpu()
        total = int(bounds[-1])
        indices = torch.empty(total, dtype=torch.int64, device=dev)
        ops, keep, self.sent_pos, self.ranges_in = [], [], {}, {}
        for p in halo.peers_out:                                 # rows of mine that rank p needs
            rows = halo.send[p]
            starts, cnts = B.indptr[rows], lens_local[rows]
            pos = torch.repeat_interleave(starts - torch.cumsum(cnts, 0) + cnts, cnts) + torch.arange(int(cnts.sum()), device=dev)
            self.sent_pos[p] = pos
            c = B.global_indices[pos].contiguous()
            keep.append(c)
            if c.numel() > 0:
                ops.append(dist.P2POp(dist.isend, c, halo._peer(p), group=halo.group))
        for p in halo.peers_in:
            a, b = int(bounds[halo.recv_offsets[p]]), int(bounds[halo.recv_offsets[p] + halo.recv_counts[p]])
            self.ranges_in[p] = (a, b)
            if b > a:
                ops.append(dist.P2POp(dist.irecv, indices[a:b], halo._peer(p), group=halo.group))
        HaloPlan._run(ops)
        self.halo = halo
        self.total = total
        self.h_indptr = indptr
        self.nb = int(B.indptr[-1])
        self.ext_indices = torch.cat((B.global_indices, indices))
        self.ext_indptr = torch.cat((B.indptr, indptr[1:] + B.indptr[-1]))

    def values(self, B_data):
        """``[B_local values ; values of the fetched rows]`` for the current values of B."""
        halo = self.halo
        ext = torch.empty(self.nb + self.total, dtype=B_data.dtype, device=B_data.device)
        ext[:self.nb] = B_data
        ops, keep = [], []
        for p in halo.peers_out:
            v = B_data[self.sent_pos[p]]
            keep.append(v)
            if v.numel() > 0:
                ops.append(dist.P2POp(dist.isend, v, halo._peer(p), group=halo.group))
        for p in halo.peers_in:
            a, b = self.ranges_in[p]
            if b > a:
                ops.append(dist.P2POp(dist.irecv, ext[self.nb + a:self.nb + b], halo._peer(p), group=halo.group))
        HaloPlan._run(ops)
        return ext


def _fetched_rows(A, B):
    """The cached ``_FetchedRows`` of the pair (collective on the first call for a pair of patterns:
    every rank of the group reaches it in the same call, as the patterns change on all ranks alike)."""
    key = (id(A.halo), B.indptr.data_ptr(), B.indptr._version, B.global_indices.data_ptr(), B.global_indices._version)
    cache = B.__dict__.setdefault("_fetched_rows", {})
    hit = cache.get(key)
    if hit is None:
        cache.clear()
        hit = cache[key] = _FetchedRows(A, B)
    return hit


class _DistSpGEMM(torch.autograd.Function):
    """C = A B on row blocks.  Forward: the rows of B that this rank's columns refer to are fetched
    from their owners (structure once per pair of patterns, values per call) and the local product is
    formed against ``[B_local ; fetched rows]``.  Backward: the local SpGEMM backward gives grad_A
    (local) and a gradient for every entry of the extended B; the part that belongs to fetched rows
    travels back to the owners, who add it to their own in ascending peer order (reproducible)."""

    @staticmethod
    def forward(ctx, A, B, A_data, B_data):
        halo = A.halo
        fetched = _fetched_rows(A, B)
        ext_data = fetched.values(B_data.detach())
        n_ext = halo.n_local + halo.n_halo
        C_data, C_indices, C_indptr = A.ops.spgemm_forward(A.n_rows, n_ext, A_data.detach(), A.indices, A.indptr,
                                                           n_ext, B.global_shape[1], ext_data, fetched.ext_indices,
                                                           fetched.ext_indptr)
        ctx.A, ctx.B, ctx.fetched = A, B, fetched
        ctx.save_for_backward(A_data, ext_data, C_indices, C_indptr)
        ctx.mark_non_differentiable(C_indices, C_indptr)
        return C_data, C_indices, C_indptr

    @staticmethod
    def backward(ctx, grad_C, _grad_indices, _grad_indptr):
        A, B, fetched = ctx.A, ctx.B, ctx.fetched
        halo = A.halo
        A_data, ext_data, C_indices, C_indptr = ctx.saved_tensors
        n_ext = halo.n_local + halo.n_halo
        grad_A, grad_ext = A.ops.spgemm_backward(grad_C.contiguous(), C_indices, C_indptr,
                                                 A.n_rows, n_ext, A_data.detach(), A.indices, A.indptr,
                                                 n_ext, B.global_shape[1], ext_data, fetched.ext_indices, fetched.ext_indptr)
        nb = fetched.nb
        grad_B = grad_ext[:nb].clone()
        ops, bufs = [], {}
        for p in halo.peers_in:                              # gradients of the rows fetched from p go home
            a, b = fetched.ranges_in[p]
            if b > a:
                ops.append(dist.P2POp(dist.isend, grad_ext[nb + a:nb + b], halo._peer(p), group=halo.group))
        for p in halo.peers_out:
            count = int(fetched.sent_pos[p].numel())
            if count > 0:
                bufs[p] = torch.empty(count, dtype=grad_ext.dtype, device=grad_ext.device)
                ops.append(dist.P2POp(dist.irecv, bufs[p], halo._peer(p), group=halo.group))
        HaloPlan._run(ops)
        for p in sorted(bufs):
            grad_B.index_add_(0, fetched.sent_pos[p], bufs[p])
        return None, None, grad_A, grad_B


def dist_spgemm(A, B):
    """This rank's rows of C = A B for row-partitioned A (columns partitioned like B's rows) and B.
    Returns ``(C_data, C_indices[global cols], C_indptr)``; the blocks of all ranks concatenate to
    the single-device product.  ``C_data`` is differentiable with respect to the stored values of
    both factors (every rank must then take part in the backward pass, which exchanges)."""
    return _DistSpGEMM.apply(A, B, A.data, B.data)


def rows_with_halo_columns(indices, indptr, n_local):
    """Boolean mask over the rows of a block in ``[local | halo]`` numbering: True where the row
    stores at least one entry in a halo column (>= n_local).  Empty rows, leading ones included,
    are False."""
    running = torch.zeros(int(indices.numel()) + 1, dtype=torch.int64, device=indices.device)
    torch.cumsum((indices >= n_local).to(torch.int64), 0, out=running[1:])
    return (running[indptr[1:]] - running[indptr[:-1]]) > 0


def ghost_row_extension(indices, indptr, n_local, n_ext):
    """Square, pattern-symmetric extension of a rank's block of rows.

    ``indices`` / ``indptr`` describe n_local rows over n_ext = n_local + n_halo columns in
    ``[local | halo]`` numbering.  One ghost row is appended per halo column, holding the mirror
    images (c, i) of the halo entries (i, c), sorted by i.  Returns
    ``(idx_ext, ptr_ext, in_halo)``: the extended CSR structure over n_ext rows and the mask of the
    original entries that lie in halo columns.  Ghost entries carry no values of their own: in the
    one-pass backward kernel a ghost row reads the values of the local entries it mirrors, which
    makes its row sum exactly the partial sum of grad_x owed to the neighbour that owns the column;
    a local entry in a halo column is paired with itself and multiplied by the zero that the
    extended upstream gradient holds in ghost rows.
    """
    dev = indices.device
    nnz = int(indices.numel())
    rows_of = torch.repeat_interleave(torch.arange(n_local, device=dev), indptr[1:] - indptr[:-1], output_size=nnz)
    in_halo = indices >= n_local
    ghost_r, ghost_c = indices[in_halo], rows_of[in_halo]
    order = torch.argsort(ghost_r * n_ext + ghost_c)
    counts = torch.bincount(ghost_r - n_local, minlength=n_ext - n_local)
    ptr_ext = torch.cat((indptr, nnz + torch.cumsum(counts, 0))).contiguous()
    idx_ext = torch.cat((indices, ghost_c[order])).contiguous()
    return idx_ext, ptr_ext, in_halo


def mirror_positions(idx_ext, ptr_ext, in_halo, t_indptr, t_indices, t_perm):
    """For every entry (i, c) of the extended structure, the storage position of its mirror (c, i),
    or None if the pattern is not symmetric.

    Rows of the extended matrix are stored in global column order, which is not ascending in the
    [local | halo] numbering, so symmetry is checked on sets: the entries sorted by (row, column)
    must coincide with the transposed structure ``(t_indptr, t_indices)``, whose ``t_perm`` then
    gives the mirror of the q-th sorted entry.  Local entries in halo columns are mapped to
    themselves (their mirror is a ghost entry without a value).
    """
    n_ext = int(ptr_ext.numel()) - 1
    dev = idx_ext.device
    rows_ext = torch.repeat_interleave(torch.arange(n_ext, device=dev), ptr_ext[1:] - ptr_ext[:-1],
                                       output_size=int(idx_ext.numel()))
    srt = torch.argsort(rows_ext * n_ext + idx_ext)
    if not (torch.equal(t_indptr.to(ptr_ext.dtype), ptr_ext) and torch.equal(t_indices.to(idx_ext.dtype), idx_ext[srt])):
        return None
    perm = torch.empty_like(t_perm)
    perm[srt] = t_perm
    k = torch.nonzero(in_halo).flatten()
    perm[k] = k.to(perm.dtype)
    return perm


class PeerExchange:
    """Exchange buffers of the peer-memory halo exchange (``csrc/halo.cu``): one buffer per rank,
    created by ``nb200_ipc_alloc``, mapped by every neighbour with CUDA IPC.

    Layout of a buffer (bytes): ``[flag words and scalar area: 256][packed x values: 2 halves][partial sums:
    2 halves]``; the first 256 bytes hold the three flag words (x, grad_x, scalar reductions) at offsets
    0, 4, 8 and, at offset 64, two halves of four doubles for dot products reduced across ranks.
    The packed x area holds, for every neighbour in ascending order, the entries of this rank's block
    of x that the neighbour reads; the partial-sum area holds this rank's grad_x contributions to the
    halo columns in halo-slot order (neighbour by neighbour, ascending).  The constructor is collective
    over the halo plan's group.  ``usable`` is False (on every rank alike) when the neighbour relation
    is not symmetric or a mapping failed; the caller then keeps the NCCL exchange.
    """

    FLAG_BYTES = 256
    SCALAR_OFFSET = 64

    def __init__(self, halo, dtype, device):
        import ctypes
        from . import _cabi
        self._c, self._cabi = ctypes, _cabi
        self.halo = halo
        self.device = device
        self.esize = torch.empty(0, dtype=dtype).element_size()
        self.code = _cabi.F64 if dtype == torch.float64 else _cabi.F32
        self.base = None
        self.mapped = {}
        group = halo.group
        peers = sorted(set(halo.peers_in) | set(halo.peers_out))
        symmetric = set(halo.peers_in) == set(halo.peers_out) and len(peers) > 0
        self.send_total = sum(halo.send_counts[p] for p in halo.peers_out)
        self.n_halo = halo.n_halo
        pad = lambda b: (b + 255) // 256 * 256  # noqa: E731
        self.x_off = self.FLAG_BYTES
        self.g_off = self.x_off + pad(2 * self.send_total * self.esize)
        total = self.g_off + pad(2 * self.n_halo * self.esize)
        handle = (ctypes.c_ubyte * 64)()
        ok = symmetric
        if ok:
            with torch.cuda.device(device):
                ptr = ctypes.c_void_p()
                ok = _cabi.lib().nb200_ipc_alloc(total, ctypes.byref(ptr), handle) == 0
                if ok:
                    self.base = ptr.value
        seg, off = {}, 0
        for p in halo.peers_out:
            seg[p] = (off, halo.send_counts[p])
            off += halo.send_counts[p]
        meta = {"ok": ok, "handle": bytes(handle), "x_off": self.x_off, "g_off": self.g_off, "send_total": self.send_total,
                "n_halo": self.n_halo, "x_segment": seg,
                "g_segment": {p: (halo.recv_offsets[p], halo.recv_counts[p]) for p in halo.peers_in}}
        metas = [None] * halo.world
        dist.all_gather_object(metas, meta, group=group)
        ok = all(m["ok"] for m in metas)
        if ok:
            with torch.cuda.device(device):
                for p in peers:
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(metas[p]["handle"])
                    if _cabi.lib().nb200_ipc_open(buf, ctypes.byref(ptr)) != 0:
                        ok = False
                        break
                    self.mapped[p] = ptr.value
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.usable = bool(flag.item())
        if not self.usable:
            self.close()
            return
        self.peers = peers
        self._handles = {r: metas[r]["handle"] for r in range(halo.world)}
        dev = device
        self.reduce_seq = torch.zeros(1, dtype=torch.int32, device=dev)
        self._reduce_table = None
        self.step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
        # what is packed for the neighbours: their segments, concatenated in ascending order
        self.send_index = torch.cat([halo.send[p] for p in halo.peers_out]).contiguous()
        # pull descriptors (x): one per neighbour this rank reads from
        words = []
        for p in halo.peers_in:
            m = metas[p]
            seg_off, seg_cnt = m["x_segment"][halo.rank]
            assert seg_cnt == halo.recv_counts[p]
            words += [self.mapped[p] + m["x_off"], m["send_total"], seg_off, seg_cnt,
                      halo.n_local + halo.recv_offsets[p], self.mapped[p] + 0, 0, 0]
        self.x_desc = torch.tensor(words, dtype=torch.int64, device=dev)
        self.x_largest = max([halo.recv_counts[p] for p in halo.peers_in], default=0)
        # pull-add descriptors (grad_x): neighbours that computed partial sums for columns of this rank
        words, index_of = [], {}
        for q, p in enumerate(halo.peers_out):
            m = metas[p]
            index_of[p] = q
            words += [self.mapped[p] + m["g_off"], m["n_halo"], 0, 0, 0, self.mapped[p] + 4, 0, 0]
        self.g_desc = torch.tensor(words, dtype=torch.int64, device=dev)
        tgt = torch.cat([halo.send[p] for p in halo.peers_out])
        src_peer = torch.cat([torch.full((halo.send_counts[p],), index_of[p], dtype=torch.int32, device=dev) for p in halo.peers_out])
        src_elem = torch.cat([metas[p]["g_segment"][halo.rank][0] + torch.arange(halo.send_counts[p], device=dev)
                              for p in halo.peers_out])
        # the same sums through a local staging buffer: the neighbours' partial sums are copied over NVLink while
        # the local rows are still being computed, and only a local addition is left for the end of the step
        stage_off, off = {}, 0
        for p in halo.peers_out:
            stage_off[p] = off
            off += halo.send_counts[p]
        self.g_stage = torch.zeros(max(off, 1), dtype=dtype, device=dev)
        words = []
        for p in halo.peers_out:
            m = metas[p]
            seg_off, seg_cnt = m["g_segment"][halo.rank]
            assert seg_cnt == halo.send_counts[p]
            words += [self.mapped[p] + m["g_off"], m["n_halo"], seg_off, seg_cnt, stage_off[p], self.mapped[p] + 4, 0, 0]
        self.g_pull_desc = torch.tensor(words, dtype=torch.int64, device=dev)
        self.g_largest = max([halo.send_counts[p] for p in halo.peers_out], default=0)
        # one descriptor that names the staging buffer as an "area" whose two halves coincide, flagged by this
        # rank's own gradient flag (raised by its own publish of the same step)
        self.stage_desc = torch.tensor([self.g_stage.data_ptr(), 0, 0, 0, 0, self.base + 4, 0, 0], dtype=torch.int64, device=dev)
        stage_elem = torch.cat([stage_off[p] + torch.arange(halo.send_counts[p], device=dev) for p in halo.peers_out])
        order = torch.sort(tgt, stable=True).indices            # by target; neighbours stay in ascending order
        tgt, self.src_peer, self.src_elem = tgt[order], src_peer[order].contiguous(), src_elem[order].contiguous()
        self.stage_elem = stage_elem[order].contiguous()
        self.stage_peer = torch.zeros_like(self.src_peer)
        self.targets, counts = torch.unique_consecutive(tgt, return_counts=True)
        self.target_ptr = torch.zeros(self.targets.numel() + 1, dtype=torch.int64, device=dev)
        self.target_ptr[1:] = torch.cumsum(counts, 0)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def _p(self, t):
        return self._c.c_void_p(t.data_ptr())

    def pull_g_args(self, status, budget):
        """nb200_halo_pull of the neighbours' partial sums for this rank's columns into the staging buffer."""
        return [len(self.halo.peers_out), self._p(self.g_pull_desc), self.g_largest, self._p(self.g_stage),
                self._p(self.step_word), self._p(status), budget, self.code, None]

    def add_g_args(self, grad_x, status, budget):
        """nb200_halo_pull_add over the staging buffer: the same additions in the same order, all local."""
        return [1, self._p(self.stage_desc), int(self.targets.numel()), self._p(self.targets), self._p(self.target_ptr),
                self._p(self.stage_peer), self._p(self.stage_elem), self._p(grad_x), self._p(self.step_word), self._p(status),
                budget, self.code, None]

    def publish_x_args(self, x_ext):
        """nb200_halo_publish: pack this rank's boundary entries of x and open a new step."""
        return [self.send_total, self._p(x_ext), self._p(self.send_index), self._c.c_void_p(self.base + self.x_off),
                self._c.c_void_p(self.base), self._p(self.step_word), 1, self._p(self.arrivals), self.code, None]

    def pull_x_args(self, x_ext, status, budget):
        return [len(self.halo.peers_in), self._p(self.x_desc), self.x_largest, self._p(x_ext), self._p(self.step_word),
                self._p(status), budget, self.code, None]

    def publish_g_args(self, gx_ext):
        """nb200_halo_publish of the halo part of gx_ext (the partial sums owed to the neighbours)."""
        halo_part = self._c.c_void_p(gx_ext.data_ptr() + self.halo.n_local * self.esize)
        return [self.n_halo, halo_part, None, self._c.c_void_p(self.base + self.g_off),
                self._c.c_void_p(self.base + 4), self._p(self.step_word), 0, self._p(self.arrivals), self.code, None]

    def pull_add_g_args(self, grad_x, status, budget):
        return [len(self.halo.peers_out), self._p(self.g_desc), int(self.targets.numel()), self._p(self.targets),
                self._p(self.target_ptr), self._p(self.src_peer), self._p(self.src_elem), self._p(grad_x),
                self._p(self.step_word), self._p(status), budget, self.code, None]

    def reduce_table(self):
        """Device table for reductions across all ranks (``nb200_cg_peer_phase``): per rank the address of
        its scalar area and of its reduction flag.  Maps the buffers of the ranks that are not halo
        neighbours on first use."""
        if self._reduce_table is None:
            halo, lib, c = self.halo, self._cabi.lib(), self._c
            words = []
            with torch.cuda.device(self.device):
                for r in range(halo.world):
                    if r == halo.rank:
                        base = self.base
                    else:
                        if r not in self.mapped:
                            ptr = c.c_void_p()
                            buf = (c.c_ubyte * 64).from_buffer_copy(self._handles[r])
                            if lib.nb200_ipc_open(buf, c.byref(ptr)) != 0:
                                raise RuntimeError(f"could not map the exchange buffer of rank {r}")
                            self.mapped[r] = ptr.value
                        base = self.mapped[r]
                    words += [base + self.SCALAR_OFFSET, base + 8]
            self._reduce_table = torch.tensor(words, dtype=torch.int64, device=self.device)
        return self._reduce_table

    def close(self):
        """Unmap the neighbours' buffers and free this rank's (after a barrier by the caller, so that no
        neighbour still reads it)."""
        lib = self._cabi.lib()
        for ptr in self.mapped.values():
            lib.nb200_ipc_close(self._c.c_void_p(ptr))
        self.mapped = {}
        if self.base is not None:
            lib.nb200_ipc_free(self._c.c_void_p(self.base))
            self.base = None


class PeerRowExchange:
    """Exchange of the rows of a dense operand between row blocks through peer memory, for the
    row-partitioned SpMM (``csrc/halo.cu``, the row kernels).  One buffer per rank from
    ``nb200_ipc_alloc``, mapped by every neighbour: ``[flag words: 256 bytes][this rank's block of rows,
    2 halves][partial gradient rows per halo slot, 2 halves]``.

    forward   every rank copies its block of X into its buffer once (``nb200_halo_publish``), each
              neighbour gathers the rows it needs from there straight into ``[local | halo]``
              (``nb200_halo_pull_rows``): nothing is packed per neighbour and no communication library runs;
    backward  the halo part of the extended gradient is published, and every owner adds the rows that
              belong to it, neighbours in ascending order (``nb200_halo_pull_add_rows``), which is the
              order of the send/recv path: the results are the same bit for bit.

    Collective over the halo plan's group.  ``usable`` is False on every rank alike when the neighbour
    relation is not symmetric, a row is not a multiple of 16 bytes, or a mapping failed."""

    FLAG_BYTES = 256

    def __init__(self, halo, dtype, width, device):
        import ctypes
        from . import _cabi
        self._c, self._cabi = ctypes, _cabi
        self.halo, self.device, self.width = halo, device, int(width)
        self.esize = torch.empty(0, dtype=dtype).element_size()
        self.code = _cabi.F64 if dtype == torch.float64 else _cabi.F32
        self.row_bytes = self.width * self.esize
        self.base, self.mapped = None, {}
        self.wait_budget_cycles = 4_000_000_000
        group = halo.group
        peers = sorted(set(halo.peers_in) | set(halo.peers_out))
        ok = set(halo.peers_in) == set(halo.peers_out) and len(peers) > 0 and self.row_bytes % 16 == 0 \
            and dtype in (torch.float32, torch.float64)
        pad = lambda b: (b + 255) // 256 * 256  # noqa: E731
        self.x_off = self.FLAG_BYTES
        self.g_off = self.x_off + pad(2 * halo.n_local * self.row_bytes)
        total = self.g_off + pad(2 * max(halo.n_halo, 1) * self.row_bytes)
        handle = (ctypes.c_ubyte * 64)()
        if ok:
            with torch.cuda.device(device):
                ptr = ctypes.c_void_p()
                ok = _cabi.lib().nb200_ipc_alloc(total, ctypes.byref(ptr), handle) == 0
                if ok:
                    self.base = ptr.value
        meta = {"ok": ok, "handle": bytes(handle), "x_off": self.x_off, "g_off": self.g_off, "n_local": halo.n_local,
                "n_halo": halo.n_halo, "recv_offsets": list(halo.recv_offsets)}
        metas = [None] * halo.world
        dist.all_gather_object(metas, meta, group=group)
        ok = all(m["ok"] for m in metas)
        if ok:
            with torch.cuda.device(device):
                for p in peers:
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(metas[p]["handle"])
                    if _cabi.lib().nb200_ipc_open(buf, ctypes.byref(ptr)) != 0:
                        ok = False
                        break
                    self.mapped[p] = ptr.value
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.usable = bool(flag.item())
        if not self.usable:
            self.close()
            return
        dev = device
        self.step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # forward: which row of the owner's block goes into which halo slot
        self.row_of_slot = torch.cat([halo.need[p] - halo.col_bounds[p] for p in halo.peers_in]).contiguous()
        words = []
        for p in halo.peers_in:
            m = metas[p]
            words += [self.mapped[p] + m["x_off"], m["n_local"], halo.recv_offsets[p], halo.recv_counts[p],
                      halo.n_local + halo.recv_offsets[p], self.mapped[p] + 0, 0, 0]
        self.x_desc = torch.tensor(words, dtype=torch.int64, device=dev)
        self.x_largest = max([halo.recv_counts[p] for p in halo.peers_in], default=0)
        # backward: for every local row that a neighbour reads, the halo slots (of the neighbours) that hold
        # partial gradient rows for it, neighbours ascending
        words, index_of = [], {}
        for q, p in enumerate(halo.peers_out):
            m = metas[p]
            index_of[p] = q
            words += [self.mapped[p] + m["g_off"], max(m["n_halo"], 1), 0, 0, 0, self.mapped[p] + 4, 0, 0]
        self.g_desc = torch.tensor(words, dtype=torch.int64, device=dev)
        tgt = torch.cat([halo.send[p] for p in halo.peers_out])
        src_peer = torch.cat([torch.full((halo.send_counts[p],), index_of[p], dtype=torch.int32, device=dev) for p in halo.peers_out])
        src_elem = torch.cat([metas[p]["recv_offsets"][halo.rank] + torch.arange(halo.send_counts[p], device=dev)
                              for p in halo.peers_out])
        order = torch.sort(tgt, stable=True).indices            # by target; neighbours stay in ascending order
        tgt, self.src_peer, self.src_elem = tgt[order], src_peer[order].contiguous(), src_elem[order].contiguous()
        self.targets, counts = torch.unique_consecutive(tgt, return_counts=True)
        self.target_ptr = torch.zeros(self.targets.numel() + 1, dtype=torch.int64, device=dev)
        self.target_ptr[1:] = torch.cumsum(counts, 0)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def _p(self, t):
        return self._c.c_void_p(t.data_ptr())

    def _stream(self):
        return self._c.c_void_p(torch.cuda.current_stream().cuda_stream)

    def extend(self, x_local):
        """``[x_local | rows fetched from their owners]``: the forward exchange."""
        halo, c = self.halo, self._c
        x_local = x_local.contiguous()
        x_ext = torch.empty((halo.n_local + halo.n_halo, self.width), dtype=x_local.dtype, device=x_local.device)
        main, side = torch.cuda.current_stream(), self._side_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):                       # the local part is copied beside the exchange
            x_ext.record_stream(side)
            x_ext[:halo.n_local].copy_(x_local)
        call = self._cabi.call
        call("nb200_halo_publish", halo.n_local * self.width, self._p(x_local), None, c.c_void_p(self.base + self.x_off),
             c.c_void_p(self.base), self._p(self.step_word), 1, self._p(self.arrivals), self.code, self._stream())
        call("nb200_halo_pull_rows", len(halo.peers_in), self._p(self.x_desc), self._p(self.row_of_slot), self.x_largest,
             self.row_bytes, self._p(x_ext), self._p(self.step_word), self._p(self.status), self.wait_budget_cycles,
             self._stream())
        main.wait_stream(side)
        return x_ext

    def reduce(self, g_ext):
        """The local block of the gradient: ``g_ext[:n_local]`` plus the partial rows that the neighbours
        computed for it (the backward exchange)."""
        halo, c = self.halo, self._c
        g_ext = g_ext.contiguous()
        main, side = torch.cuda.current_stream(), self._side_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):                       # copied beside the publication of the halo part
            g_local = g_ext[:halo.n_local].clone()
        call = self._cabi.call
        halo_part = c.c_void_p(g_ext.data_ptr() + halo.n_local * self.row_bytes)
        call("nb200_halo_publish", halo.n_halo * self.width, halo_part, None, c.c_void_p(self.base + self.g_off),
             c.c_void_p(self.base + 4), self._p(self.step_word), 0, self._p(self.arrivals), self.code, self._stream())
        main.wait_stream(side)
        g_local.record_stream(main)
        call("nb200_halo_pull_add_rows", len(halo.peers_out), self._p(self.g_desc), int(self.targets.numel()),
             self._p(self.targets), self._p(self.target_ptr), self._p(self.src_peer), self._p(self.src_elem), self.row_bytes,
             self._p(g_local), self._p(self.step_word), self._p(self.status), self.wait_budget_cycles, self.code,
             self._stream())
        return g_local

    def _side_stream(self):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def check(self):
        """Raise if a bounded wait of an exchange ran out (reads the status word: synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer-memory row exchange gave up waiting for a neighbour (status {code})")

    def close(self):
        lib = self._cabi.lib()
        for ptr in self.mapped.values():
            lib.nb200_ipc_close(self._c.c_void_p(ptr))
        self.mapped = {}
        if self.base is not None:
            lib.nb200_ipc_free(self._c.c_void_p(self.base))
            self.base = None


def _row_exchange(A, x_local):
    """The ``PeerRowExchange`` of A's halo plan for operands like ``x_local``, created (collectively) on
    first use, or None when the send/recv path is to be used: CPU tensors, one rank, vectors, the
    environment variable NB200_EXCHANGE=nccl, or a set-up that did not succeed on every rank."""
    halo = A.halo
    if not x_local.is_cuda or x_local.ndim != 2 or halo.world < 2 or os.environ.get("NB200_EXCHANGE", "auto") == "nccl":
        return None
    cache = halo.__dict__.setdefault("_row_exchanges", {})
    key = (x_local.dtype, int(x_local.shape[1]))
    if key not in cache:
        for old in cache.values():                       # one set of buffers at a time
            if old is not None and old.usable:
                torch.cuda.synchronize(x_local.device)
                dist.barrier(group=halo.group)
                old.close()
        cache.clear()
        ex = PeerRowExchange(halo, x_local.dtype, int(x_local.shape[1]), x_local.device)
        cache[key] = ex if ex.usable else None
    return cache[key]


class DistSpMVEngine:
    """Forward + backward of a row-partitioned SpMV as a fixed schedule of C-ABI launches over
    preallocated buffers, with the halo exchange overlapped with the rows that do not need it.

    forward:   pack -> [exchange || rows without halo columns] -> remaining rows
    backward:  grad_x partial sums of the halo columns -> [exchange || grad_A pass, local grad_x
               pass] -> add the received partial sums (peers in ascending order)

    The outputs live in the engine's buffers (``y``, ``grad_A``, ``grad_x``); x is written by the
    caller into ``x_ext[:n_local]``.  CUDA only.
    """

    def __init__(self, A, exchange="auto"):
        """``exchange``: "peer" (halo values read from the neighbours' memory by this library's own
        kernels, see ``PeerExchange``), "nccl" (grouped send/recv), or "auto" (peer when it can be set
        up on every rank, else nccl; the environment variable NB200_EXCHANGE overrides)."""
        import ctypes
        from . import _cabi, _plan
        self._c, self._cabi = ctypes, _cabi
        self.A = A
        self._exchange_request = os.environ.get("NB200_EXCHANGE", exchange)
        self.use_value_symmetry = True
        self.values_symmetric = False
        self.backward_schedule = os.environ.get("NB200_BACKWARD_SCHEDULE", "sequential")   # or "forked"
        self._side = None
        self.peer = None
        self.wait_budget_cycles = 4_000_000_000
        halo = A.halo
        dev = A.data.device
        dt = A.data.dtype
        self.n, self.n_ext, self.nnz = A.n_rows, halo.n_local + halo.n_halo, int(A.data.numel())
        self.code = _cabi.F64 if dt == torch.float64 else _cabi.F32
        plan = _plan.get_plan(self.n, self.n_ext, A.indices, A.indptr)
        self.plan = plan
        self.idx, self.ptr, self.itype = plan.csr()
        self.t_indptr, self.t_indices, self.t_perm, _ = plan.transpose()
        self.br = plan.spmv_block_rows()
        self.tbr = plan.spmv_block_rows(transposed=True)
        self.esize = self.ptr.element_size()
        self.vsize = A.data.element_size()
        # rows that reference no halo column, as one contiguous range aligned to the kernel's row blocks
        has_halo = rows_with_halo_columns(A.indices, A.indptr, halo.n_local)
        marks = [-1] + torch.nonzero(has_halo).flatten().tolist() + [self.n]
        gaps = [(marks[q + 1] - marks[q] - 1, marks[q] + 1, marks[q + 1]) for q in range(len(marks) - 1)]
        _, a, b = max(gaps)
        align = 256
        a = min(self.n, -(-a // align) * align)
        b = max(a, (b // align) * align)
        self.interior = (a, b)
        self.x_ext = torch.zeros(self.n_ext, dtype=dt, device=dev)
        self.gx_ext = torch.zeros(self.n_ext, dtype=dt, device=dev)
        self.y = torch.empty(self.n, dtype=dt, device=dev)
        self.grad_A = torch.empty(self.nnz, dtype=dt, device=dev)
        self.grad_x = self.gx_ext[:halo.n_local]
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.send_bufs = {p: torch.empty(halo.send_counts[p], dtype=dt, device=dev) for p in halo.peers_out}
        self.recv_bufs = {p: torch.empty(halo.send_counts[p], dtype=dt, device=dev) for p in halo.peers_out}
        self.launches_per_step = 3 + 3 + len(halo.peers_out)
        self.fused = False
        self.exchange = "NCCL grouped send/recv of packed halo values"
        self.schedule = "pack -> [exchange || interior rows] -> boundary rows; ghost rows -> [exchange || local rows] -> add"
        if self._exchange_request in ("auto", "peer") and A.data.is_cuda and halo.world > 1:
            peer = PeerExchange(halo, dt, dev)
            if peer.usable:
                self.peer = peer
                self.exchange = "peer memory: neighbours' packed values read over NVLink by this library's kernels, step flags with bounded waits"
                self.schedule = ("[publish -> pull -> boundary rows || interior rows]; [ghost rows -> publish -> pull into a staging"
                                 " buffer || local rows] -> local add (two streams, no communication library in the step)")
                self.launches_per_step = 4 + 5
            elif self._exchange_request == "peer":
                raise RuntimeError("the peer-memory exchange could not be set up on every rank")
        if self.br > 0 and self.n == halo.n_local and self.nnz > 0:
            self._build_symmetric_extension(_plan)

    def _build_symmetric_extension(self, _plan):
        """Switch the backward to the one-pass kernel on the ghost-row extension of the local block
        (see ``ghost_row_extension``), if the block's pattern allows it."""
        A, halo = self.A, self.A.halo
        dev = A.data.device
        nl, n_ext, nnz = halo.n_local, self.n_ext, self.nnz
        idx_ext, ptr_ext, in_halo = ghost_row_extension(A.indices, A.indptr, nl, n_ext)
        plan = _plan.get_plan(n_ext, n_ext, idx_ext, ptr_ext)
        br = plan.spmv_block_rows()
        if br == 0:
            return
        idx_n, ptr_n, itype = plan.csr()
        t_indptr, t_indices, t_perm, _ = plan.transpose()
        perm = mirror_positions(idx_ext, ptr_ext, in_halo, t_indptr, t_indices, t_perm)
        if perm is None:
            return
        self.plan_ext = plan
        self.idx, self.ptr, self.itype = idx_n, ptr_n, itype
        self.br = br
        self.perm_ext = perm
        self.nnz_ext = int(idx_ext.numel())
        self.g_ext = torch.zeros(n_ext, dtype=A.data.dtype, device=dev)
        self.grad_A_ext = torch.empty(self.nnz_ext, dtype=A.data.dtype, device=dev)
        self.grad_A = self.grad_A_ext[:nnz]
        self.fused = True
        self.launches_per_step = 3 + 2 + len(halo.peers_out) if self.peer is None else 4 + 4

    def _p(self, t, offset_elems=0):
        return self._c.c_void_p(t.data_ptr() + offset_elems * t.element_size())

    def _fwd_call(self, a, b, ptr, idx, perm, vec, out, cols, hint):
        """Argument tuple of nb200_spgemv_forward restricted to rows [a, b) (None if empty)."""
        if b <= a:
            return None
        return [b - a, cols, int(idx.numel()), self._p(self.A.data), self._p(idx), self._p(ptr, a),
                self._p(perm) if perm is not None else None, self._p(vec), self._p(out, a),
                self._row_range_hint(a, b, int(ptr.numel()) - 1, hint), self._p(self.status), self.code, self.itype, None]

    @staticmethod
    def _row_range_hint(a, b, total_rows, hint):
        """Kernel choice for rows [a, b): the pipelined kernel when the plan allows it and the range starts on one
        of its row blocks; otherwise, for a proper sub-range, the row-streaming kernel named explicitly (-1),
        because nnz / rows of a sub-range call says nothing about the rows in it."""
        if hint > 0 and a % 256 == 0:
            return hint
        return 0 if (a == 0 and b == total_rows and hint >= 0) else -1

    def _prepare(self, g):
        """Everything that does not change from step to step: ctypes argument lists and the
        point-to-point descriptors (the buffers they name are fixed)."""
        halo, lib = self.A.halo, self._cabi.lib()
        nl = halo.n_local
        a, b = self.interior
        self._g = g
        self._lib = lib
        self._pack = [[halo.send_counts[p], self._p(self.x_ext), self._p(halo.send[p]), self._p(self.send_bufs[p]),
                       self.code, self._cabi.I64, None] for p in halo.peers_out]
        self._fwd_ops = [dist.P2POp(dist.isend, self.send_bufs[p], halo._peer(p), group=halo.group) for p in halo.peers_out]
        for p in halo.peers_in:
            o = nl + halo.recv_offsets[p]
            self._fwd_ops.append(dist.P2POp(dist.irecv, self.x_ext[o:o + halo.recv_counts[p]], halo._peer(p), group=halo.group))
        fw = lambda lo, hi: self._fwd_call(lo, hi, self.ptr, self.idx, None, self.x_ext, self.y, self.n_ext, self.br)  # noqa: E731
        self._fwd_interior = fw(a, b)
        # With the peer exchange the boundary rows run beside the interior rows on a side stream.  The pipelined
        # kernel of the interior rows fills every SM's shared memory, so a second pipelined kernel would only start
        # when the first has drained; the register-staged kernel (hint 0) needs none and fits in beside it.
        small = (lambda lo, hi: self._fwd_call(lo, hi, self.ptr, self.idx, None, self.x_ext, self.y, self.n_ext, -1)) \
            if self.peer is not None else fw
        self._fwd_boundary = [c for c in (small(0, a), small(b, self.n)) if c is not None]
        tp = lambda lo, hi: self._fwd_call(lo, hi, self.t_indptr, self.t_indices, self.t_perm, g, self.gx_ext, self.n, self.tbr)  # noqa: E731
        self._t_halo = tp(nl, self.n_ext)
        self._t_local = tp(0, nl)
        self._bwd_ops = []
        for p in halo.peers_in:
            o = nl + halo.recv_offsets[p]
            self._bwd_ops.append(dist.P2POp(dist.isend, self.gx_ext[o:o + halo.recv_counts[p]], halo._peer(p), group=halo.group))
        for p in halo.peers_out:
            self._bwd_ops.append(dist.P2POp(dist.irecv, self.recv_bufs[p], halo._peer(p), group=halo.group))
        self._grad_A = [self.n, self.n_ext, self.nnz, self._p(self.idx), self._p(self.ptr), self._p(self.x_ext),
                        self._p(g), self._p(self.grad_A), self.br, self._p(self.status), self.code, self.itype, None]
        if self.fused:
            def sym(lo, hi, values_symmetric=0):
                return [self.n_ext, self.nnz_ext, lo, hi, self._p(self.A.data), self._p(self.idx), self._p(self.ptr),
                        self._p(self.perm_ext), self._p(self.x_ext), self._p(self.g_ext), self._p(self.grad_A_ext),
                        self._p(self.gx_ext), values_symmetric, self.br, self._p(self.status), self.code, self.itype, None]
            # ghost rows have no values of their own and always read their mirrors through the permutation;
            # the local rows stream their values when the local block equals its transpose in value
            self._values_key = (self.A.data.data_ptr(), self.A.data._version)
            self.values_symmetric = self._local_values_symmetric()
            self._sym_ghost = sym(nl, self.n_ext) if self.n_ext > nl else None
            self._sym_local = sym(0, nl, int(self.values_symmetric))
            # the same partial sums (row sums of the ghost rows, values through the mirror permutation, entries in
            # storage order) from the register-staged forward kernel, which runs beside the local rows' pipelined one
            self._ghost_light = self._fwd_call(nl, self.n_ext, self.ptr, self.idx, self.perm_ext, self.g_ext, self.gx_ext,
                                               self.n_ext, -1) if self.peer is not None else None
        if self.peer is not None:
            self._peer_publish_x = self.peer.publish_x_args(self.x_ext)
            self._peer_pull_x = self.peer.pull_x_args(self.x_ext, self.status, self.wait_budget_cycles)
            self._peer_publish_g = self.peer.publish_g_args(self.gx_ext)
            self._peer_pull_add = self.peer.pull_add_g_args(self.gx_ext, self.status, self.wait_budget_cycles)
            self._peer_pull_g = self.peer.pull_g_args(self.status, self.wait_budget_cycles)
            self._peer_add_g = self.peer.add_g_args(self.gx_ext, self.status, self.wait_budget_cycles)
            if self.fused and self.n_ext > nl:
                # ghost rows and publication in one launch: the row sums go straight into the exchange buffer
                pk = self.peer
                self._ghost_publish = [self.n_ext - nl, self._p(self.A.data), self._p(self.idx), self._p(self.ptr, nl),
                                       self._p(self.perm_ext), self._p(self.g_ext), self._c.c_void_p(pk.base + pk.g_off),
                                       self._c.c_void_p(pk.base + 4), self._p(pk.step_word), 0, self._p(pk.arrivals),
                                       self.code, self.itype, None]
                if self.backward_schedule == "sequential":
                    self.schedule = ("[publish -> pull -> boundary rows || interior rows]; ghost rows + publish (one launch) -> local rows"
                                     " -> pull-add over NVLink (no communication library in the step)")
                    self.launches_per_step = 4 + 3
            else:
                self._ghost_publish = None

    def _local_values_symmetric(self):
        """True if every local entry equals its mirror image bit for bit (entries in halo columns are
        their own mirrors in the extension): the test behind the value-symmetric backward pass, run on
        the device.  `_prepare` repeats it whenever the values' version counter has moved; a captured
        graph keeps the answer it was recorded with, so capture again after changing the values."""
        if not self.use_value_symmetry:
            return False
        word = torch.zeros(1, dtype=torch.int32, device=self.A.data.device)
        self._cabi.call("nb200_csr_values_symmetric", self.nnz, self._p(self.A.data), self._p(self.perm_ext), self._p(word),
                        self.code, self.itype, self._c.c_void_p(torch.cuda.current_stream().cuda_stream))
        return int(word.item()) == 0

    def close(self):
        """Release the exchange buffers (collective: a barrier first, so that no neighbour is still
        reading this rank's)."""
        if self.peer is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.A.halo.group)
            self.peer.close()
            self.peer = None

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.A.data.device)
        return self._side

    def _launch(self, fn, args, stream):
        if args is None:
            return
        args[-1] = stream
        rc = fn(*args)
        if rc != 0:
            raise self._cabi.NB200Error(fn.__name__, rc, self._lib.nb200_status_string(rc).decode())

    def forward(self):
        """y = A x with x taken from x_ext[:n_local]."""
        if not hasattr(self, "_lib"):
            self._prepare(torch.zeros(self.n, dtype=self.y.dtype, device=self.y.device))
        lib = self._lib
        stream = self._c.c_void_p(torch.cuda.current_stream().cuda_stream)
        if self.peer is not None:
            # the small kernels (publish, pull, boundary rows) go to a side stream and are issued first, so that
            # they take their few SMs at once and run under the cover of the interior rows, which need none of them
            main = torch.cuda.current_stream()
            side = self._side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                s2 = self._c.c_void_p(side.cuda_stream)
                self._launch(lib.nb200_halo_publish, self._peer_publish_x, s2)
                self._launch(lib.nb200_halo_pull, self._peer_pull_x, s2)
                for args in self._fwd_boundary:
                    self._launch(lib.nb200_spgemv_forward, args, s2)
            self._launch(lib.nb200_spgemv_forward, self._fwd_interior, stream)
            main.wait_stream(side)
            return self.y
        for args in self._pack:
            self._launch(lib.nb200_gather, args, stream)
        reqs = dist.batch_isend_irecv(self._fwd_ops) if self._fwd_ops else []
        self._launch(lib.nb200_spgemv_forward, self._fwd_interior, stream)
        for r in reqs:
            r.wait()
        for args in self._fwd_boundary:
            self._launch(lib.nb200_spgemv_forward, args, stream)
        return self.y

    def set_inputs(self, x, g):
        """Copy this rank's block of x and of the upstream gradient g into the engine's buffers; `step`
        and the captured graph read them from there."""
        self.x_ext[:self.A.halo.n_local].copy_(x)
        if self.fused:
            self.g_ext[:self.n].copy_(g)
            self._g_in = self.g_ext[:self.n]
        else:
            self._g_in = g.clone()

    def step(self):
        """forward() followed by backward() on the inputs given to `set_inputs`."""
        self.forward()
        self.backward(self._g_in)

    def capture(self, warmup=3):
        """Record step() -- kernels, packs and the exchanges -- into one CUDA graph and return a
        function that replays it.  The launch schedule is identical on every step, so replaying removes
        the per-step host work (a dozen launches and the exchange calls), which at two or more GPUs is
        as long as the GPU work itself.  Every rank must call this at the same point.  Warm-up steps run
        first on a side stream, as graph capture requires."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step()
        self._graph = graph
        return graph.replay

    def phase_times(self, reps=50):
        """Microseconds per call of the forward half alone and of the whole step, each replayed ``reps`` times
        as a CUDA graph and timed with CUDA events on this rank; the backward half is their difference.
        Collective: every rank must call it at the same point, after ``set_inputs``."""
        def replayed(fn):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            if dist.is_initialized():
                dist.barrier(group=self.A.halo.group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            e1.synchronize()
            return e0.elapsed_time(e1) * 1e3 / reps
        forward_us = replayed(self.forward)
        step_us = replayed(self.step)
        return {"forward_us": forward_us, "backward_us": step_us - forward_us, "step_us": step_us}

    def backward(self, g):
        """grad_A (pattern of the local rows) and grad_x (local block) for upstream gradient g;
        x_ext must still hold the forward's values."""
        if self.fused and g.data_ptr() != self.g_ext.data_ptr():
            self.g_ext[:self.n].copy_(g)            # callers may also write into g_ext[:n] directly
            g = self.g_ext[:self.n]
        if not hasattr(self, "_lib") or self._g.data_ptr() != g.data_ptr() or \
                (self.fused and self._values_key != (self.A.data.data_ptr(), self.A.data._version)):
            self._prepare(g)
        lib, halo = self._lib, self.A.halo
        stream = self._c.c_void_p(torch.cuda.current_stream().cuda_stream)
        # partial sums for halo columns first, so that their exchange overlaps the rest
        if self.peer is not None:
            if self.fused and self._ghost_publish is not None and self.backward_schedule == "sequential":
                # The pipelined kernel of the local rows takes every register of every SM, so nothing launched beside
                # it overlaps with it; the shortest chain is then: ghost rows + publication in one small launch, the
                # local rows, and one launch that reads the neighbours' sums over NVLink (long published by then)
                # and adds them.
                self._launch(lib.nb200_halo_publish_rowsums, self._ghost_publish, stream)
                self._launch(lib.nb200_spgemv_backward_symmetric_rows, self._sym_local, stream)
                self._launch(lib.nb200_halo_pull_add, self._peer_pull_add, stream)
                return self.grad_A, self.grad_x
            if self.fused:
                # ghost rows and the publication of their partial sums run beside the local rows
                main = torch.cuda.current_stream()
                side = self._side_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    s2 = self._c.c_void_p(side.cuda_stream)
                    if self._ghost_light is not None:
                        self._launch(lib.nb200_spgemv_forward, self._ghost_light, s2)
                    else:
                        self._launch(lib.nb200_spgemv_backward_symmetric_rows, self._sym_ghost, s2)
                    self._launch(lib.nb200_halo_publish, self._peer_publish_g, s2)
                    self._launch(lib.nb200_halo_pull, self._peer_pull_g, s2)       # NVLink reads under the local rows
                self._launch(lib.nb200_spgemv_backward_symmetric_rows, self._sym_local, stream)
                main.wait_stream(side)
                self._launch(lib.nb200_halo_pull_add, self._peer_add_g, stream)    # local additions only
                return self.grad_A, self.grad_x
            else:
                self._launch(lib.nb200_spgemv_forward, self._t_halo, stream)
                self._launch(lib.nb200_halo_publish, self._peer_publish_g, stream)
                self._launch(lib.nb200_spgemv_grad_A, self._grad_A, stream)
                self._launch(lib.nb200_spgemv_forward, self._t_local, stream)
            self._launch(lib.nb200_halo_pull_add, self._peer_pull_add, stream)
            return self.grad_A, self.grad_x
        if self.fused:
            self._launch(lib.nb200_spgemv_backward_symmetric_rows, self._sym_ghost, stream)
            reqs = dist.batch_isend_irecv(self._bwd_ops) if self._bwd_ops else []
            self._launch(lib.nb200_spgemv_backward_symmetric_rows, self._sym_local, stream)
        else:
            self._launch(lib.nb200_spgemv_forward, self._t_halo, stream)
            reqs = dist.batch_isend_irecv(self._bwd_ops) if self._bwd_ops else []
            self._launch(lib.nb200_spgemv_grad_A, self._grad_A, stream)
            self._launch(lib.nb200_spgemv_forward, self._t_local, stream)
        for r in reqs:
            r.wait()
        for p in halo.peers_out:
            self.grad_x.index_add_(0, halo.send[p], self.recv_bufs[p])
        return self.grad_A, self.grad_x


class DistCG:
    """Unpreconditioned CG with a fixed iteration count on a row-partitioned SPD matrix, driven through a
    ``DistSpMVEngine``.  The recurrence is the reference's (``numml/krylov.py:135-153``) with ``rtol = 0``;
    nothing is read back to the host inside the loop.

    With the peer-memory exchange the whole iteration is this library's kernels: the engine's forward
    (publish, [pull and boundary rows beside] the interior rows) and three vector kernels whose dot
    products are reduced across ranks through the exchange buffers, in rank order, inside the kernels
    (``nb200_cg_peer_phase``).  One iteration is recorded into a CUDA graph and replayed.  Without it the
    vector updates are torch operations and the two dot products of an iteration are all-reduced."""

    def __init__(self, engine):
        self.engine = engine
        self.group = engine.A.halo.group
        self.peer = engine.peer is not None and engine.A.halo.world <= 32
        self._graph = None
        if self.peer:
            self.schedule = ("per iteration: publish p, [pull + boundary rows || interior rows], <Ap,p>, update with <r,r>, direction;"
                             " dot products reduced through peer memory inside the kernels; one CUDA graph per iteration")
        else:
            self.schedule = "per iteration: engine forward (NCCL halo exchange) + torch vector updates + 2 all-reduced dot products"

    def _dot(self, a, b):
        s = torch.dot(a, b)
        dist.all_reduce(s, group=self.group)
        return s

    def solve(self, b_local, iterations):
        """Returns (this rank's block of x, the iterations + 1 residual norms)."""
        if self.peer:
            return self._solve_peer(b_local, iterations)
        eng = self.engine
        nl = eng.A.halo.n_local
        p = eng.x_ext[:nl]                      # the search direction lives where the engine reads x
        x = torch.zeros_like(b_local)
        r = b_local.clone()
        p.copy_(r)
        rz = self._dot(r, r)
        hist = torch.empty(iterations + 1, dtype=b_local.dtype, device=b_local.device)
        hist[0] = torch.sqrt(rz)
        zero = torch.zeros_like(rz)
        for it in range(iterations):
            Ap = eng.forward()
            done = rz == 0
            alpha = torch.where(done, zero, rz / self._dot(Ap, p))
            x.add_(alpha * p)
            r.sub_(alpha * Ap)
            rz_new = self._dot(r, r)
            beta = torch.where(done, zero, rz_new / rz)
            p.mul_(beta).add_(r)
            rz = rz_new
            hist[it + 1] = torch.sqrt(rz)
        return x, hist

    def _solve_peer(self, b_local, iterations):
        import ctypes
        from . import _cabi
        eng, halo = self.engine, self.engine.A.halo
        dev, dt = b_local.device, b_local.dtype
        nl = halo.n_local
        P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        if not hasattr(self, "_work"):
            wbytes = _cabi.lib().nb200_cg_peer_workspace_bytes()
            self._work = torch.zeros(wbytes, dtype=torch.uint8, device=dev)
            self._wbytes = wbytes
            self._x = torch.empty(nl, dtype=dt, device=dev)
            self._r = torch.empty(nl, dtype=dt, device=dev)
            self._b = torch.empty(nl, dtype=dt, device=dev)
            self._table = eng.peer.reduce_table()
        if getattr(self, "_hist", None) is None or self._hist.numel() != iterations + 1:
            self._hist = torch.empty(iterations + 1, dtype=dt, device=dev)
            self._graph = None                                   # the history buffer is part of the recording
        self._b.copy_(b_local)
        p = eng.x_ext[:nl]
        code = _cabi.F64 if dt == torch.float64 else _cabi.F32

        def phase(k, Ap=None):
            _cabi.call("nb200_cg_peer_phase", k, nl, P(self._b), P(self._x), P(self._r), P(p),
                       P(Ap) if Ap is not None else None, P(self._hist), P(self._work), self._wbytes, halo.world, halo.rank,
                       P(self._table), P(eng.peer.reduce_seq), P(eng.status), eng.wait_budget_cycles, code,
                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))

        def iteration():
            Ap = eng.forward()
            phase(2, Ap)
            phase(3, Ap)
            phase(4)

        phase(0)
        phase(1)
        if self._graph is None and iterations > 1:
            # one eager iteration warms everything up; the recording then covers one iteration
            iteration()
            done = 1
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                iteration()
            self._graph = graph
        else:
            done = 0
        for _ in range(iterations - done):
            if self._graph is not None:
                self._graph.replay()
            else:
                iteration()
        return self._x.clone(), self._hist.clone()
