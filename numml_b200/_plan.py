"""Per-sparsity-pattern plans: what can be computed once from ``(indices, indptr)`` and reused
while the values change (CG iterations, training steps).

A plan holds
  * int32 copies of ``indices`` / ``indptr`` (the reference stores int64 everywhere,
    reference ``numml/sparse/_csr.py:599-600,626-639``; the kernels read half the index bytes from
    the narrowed copy) -- only when nnz, rows and cols fit in 31 bits;
  * the transposed structure (``t_indptr``, ``t_indices``, ``t_perm``), built on first use.

Plans are looked up by the identity of the two index tensors (storage pointer, length, in-place
version counter).  A cache entry keeps the tensors alive, so a pointer can never be recycled
for a different pattern while its entry exists; an in-place edit bumps the version and misses.
"""
import collections
import ctypes

import torch

from . import _cabi

_INT32_MAX = 2 ** 31 - 1
CHECK_BAD_INDPTR, CHECK_COLUMN_RANGE, CHECK_UNSORTED, CHECK_NO_DIAGONAL = 1, 2, 4, 8   # NB200_CHECK_* of the C header
_CACHE = collections.OrderedDict()
_CACHE_SIZE = 8
force_int64 = False  # set True to make every kernel read the int64 arrays as stored (measurement aid)


def _stream():
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() > 0 else 0)


def _published(device):
    """Cached plan arrays are written once, on the stream that first needed them, and read for as long
    as the pattern lives from whatever stream is current then.  Waiting once for the producing stream,
    here, makes them safe to read from any stream afterwards."""
    torch.cuda.current_stream(device).synchronize()


class PatternPlan:
    def __init__(self, rows, cols, indices, indptr):
        self.rows, self.cols = int(rows), int(cols)
        self.indices, self.indptr = indices, indptr
        self.nnz = int(indices.numel())
        self.version = (indices._version, indptr._version)
        self._narrow = None
        self._t = None
        self.extra = {}

    # -- index-width selection -------------------------------------------------------------
    def fits_int32(self):
        return (not force_int64) and max(self.nnz, self.rows, self.cols) < _INT32_MAX

    def csr(self):
        """(indices, indptr, itype) in the width the kernels should read."""
        if not self.fits_int32():
            return self.indices, self.indptr, _cabi.I64
        if self._narrow is None:
            with torch.cuda.device(self.indices.device):
                i32 = torch.empty(self.nnz, dtype=torch.int32, device=self.indices.device)
                p32 = torch.empty(self.rows + 1, dtype=torch.int32, device=self.indices.device)
                _cabi.call("nb200_narrow_indices", self.nnz, _ptr(self.indices), _ptr(i32), _stream())
                _cabi.call("nb200_narrow_indices", self.rows + 1, _ptr(self.indptr), _ptr(p32), _stream())
                _published(self.indices.device)
            self._narrow = (i32, p32)
        return self._narrow[0], self._narrow[1], _cabi.I32

    # -- structure check ---------------------------------------------------------------------
    def check_flags(self):
        """NB200_CHECK_* bits of the pattern (0 = clean), computed once per plan by nb200_csr_check."""
        if "check" not in self.extra:
            if self.indices.dtype != torch.int64 or self.indptr.dtype != torch.int64:
                raise RuntimeError("CSR index arrays must be int64 tensors")
            dev = self.indices.device
            with torch.cuda.device(dev):
                flags = torch.zeros(1, dtype=torch.int32, device=dev)
                _cabi.call("nb200_csr_check", self.rows, self.cols, self.nnz, _ptr(self.indices), _ptr(self.indptr),
                           _cabi.I64, _ptr(flags), _stream())
                self.extra["check"] = int(flags.item())
        return self.extra["check"]

    def require(self, sorted_columns=False, diagonal=False, what="this operation"):
        """Raise (instead of reading out of bounds or answering wrongly, as the reference would) when
        the pattern is malformed, or lacks a property that ``what`` relies on."""
        flags = self.check_flags()
        if flags & CHECK_BAD_INDPTR:
            raise RuntimeError("malformed CSR matrix: indptr must start at 0, end at nnz and never decrease")
        if flags & CHECK_COLUMN_RANGE:
            raise RuntimeError(f"malformed CSR matrix: a column index lies outside [0, {self.cols})")
        if sorted_columns and flags & CHECK_UNSORTED:
            raise RuntimeError(f"{what} needs the column indices of every row strictly ascending "
                               "(sorted, without duplicates)")
        if diagonal and flags & CHECK_NO_DIAGONAL:
            raise RuntimeError(f"{what} needs a stored diagonal entry in every row")

    # -- transposed structure ----------------------------------------------------------------
    def transpose(self):
        """(t_indptr, t_indices, t_perm, itype) of the pattern, in the plan's index width."""
        if self._t is None:
            idx, ptr, itype = self.csr()
            self._t = transpose_structure(self.rows, self.cols, idx, ptr, itype, itype) + (itype,)
            _published(self.indices.device)
        return self._t


    def pattern_symmetric(self):
        """True if the sparsity pattern equals its transpose (stencils, undirected graphs)."""
        if "symmetric" not in self.extra:
            ok = self.rows == self.cols
            if ok:
                idx, ptr, _ = self.csr()
                t_indptr, t_indices, _, _ = self.transpose()
                ok = bool(torch.equal(t_indptr, ptr)) and bool(torch.equal(t_indices, idx))
            self.extra["symmetric"] = ok
        return self.extra["symmetric"]

    def values_symmetric(self, data):
        """True once ``data`` is known to equal its transpose bit for bit (``data[t_perm[k]] == data[k]``)
        on this pattern, which must be symmetric.  The one-pass SpMV backward then streams the values
        instead of gathering their mirror images.

        The test costs a pass over the matrix and a host read of one word, so it is made only for
        values that come back: the first call with a given tensor version answers False and remembers
        the version; a second call with the same version runs the test and caches its answer until the
        tensor is modified in place (torch bumps its version counter) or replaced.  Values that change
        every step therefore never pay for it.  Writes that bypass the version counter (``.data``
        views) are not seen, as with autograd's own saved-tensor checks."""
        key = (data.data_ptr(), data._version, int(data.numel()), data.dtype)
        seen = self.extra.get("values_symmetric")
        if seen is not None and seen[0] == key:
            if seen[1] is None:
                _, _, t_perm, itype = self.transpose()
                dev = data.device
                with torch.cuda.device(dev):
                    word = torch.zeros(1, dtype=torch.int32, device=dev)
                    _cabi.call("nb200_csr_values_symmetric", self.nnz, _ptr(data), _ptr(t_perm), _ptr(word),
                               _cabi.F64 if data.dtype == torch.float64 else _cabi.F32, itype, _stream())
                    seen = (key, int(word.item()) == 0, data)
                self.extra["values_symmetric"] = seen
            return seen[1]
        # keep the tensor alive so that its address cannot be reused by other values under the same key
        self.extra["values_symmetric"] = (key, None, data)
        return False

    # -- kernel choice for SpMV ---------------------------------------------------------------------
    def spmv_block_rows(self, transposed=False):
        """Rows per block for the TMA-pipelined SpMV kernels over this pattern (or over its
        transpose), or 0 when the pattern is too irregular for them: the largest R in (256, 128)
        such that every block of R consecutive rows fits one pipeline stage."""
        key = ("spmv_block_rows", bool(transposed))
        if key not in self.extra:
            if transposed:
                ptr, _, _, itype = self.transpose()
                rows = self.cols
            else:
                _, ptr, itype = self.csr()
                rows = self.rows
            dev = self.indices.device
            with torch.cuda.device(dev):
                out = torch.empty(4, dtype=torch.int64, device=dev)
                _cabi.call("nb200_csr_block_profile", rows, _ptr(ptr), itype, _ptr(out), _stream())
                maxima = out.cpu().tolist()
            tile = _cabi.lib().nb200_spmv_pipeline_tile()
            choice = 0
            for c, R in enumerate((256, 128)):
                if maxima[c] <= tile:
                    choice = R
                    break
            self.extra[key] = choice if self.nnz > 0 else 0
        return self.extra[key]

    # -- row schedule for SpMM ------------------------------------------------------------------------
    def spmm_row_order(self, transposed=False):
        """int32 permutation of the rows (of the pattern, or of its transpose) by descending length, or
        None when the lengths are even enough for the natural order (which keeps neighbouring rows, and
        the dense rows they share, together).  Skewed matrices get it: a row of thousands of entries is
        walked by one lane group alone and should start first, not last."""
        key = ("spmm_row_order", bool(transposed))
        if key not in self.extra:
            ptr = self.transpose()[0] if transposed else self.indptr
            rows = int(ptr.numel()) - 1
            order = None
            if rows >= 4096 and self.nnz > 0:
                lens = ptr[1:] - ptr[:-1]
                if int(lens.max()) > 16 * max(1.0, self.nnz / rows):
                    order = torch.argsort(lens, descending=True, stable=True).to(torch.int32)
                    _published(ptr.device)
            self.extra[key] = order
        return self.extra[key]

    # -- triangular-solve schedules ----------------------------------------------------------------
    def sptrsv_order(self, lower, transposed=False):
        """(order, nlevels) for solving with this pattern (``transposed=False``) or with its
        transpose (``transposed=True``; the triangle given is that of the transposed matrix)."""
        key = ("sptrsv", bool(lower), bool(transposed))
        if key not in self.extra:
            idx, ptr, itype = self.csr()
            if transposed:
                t_indptr, t_indices, _, _ = self.transpose()
                idx, ptr = t_indices, t_indptr
            n = self.rows
            dev = self.indices.device
            with torch.cuda.device(dev):
                order = torch.empty(n, dtype=torch.int32, device=dev)
                level_ptr = torch.empty(n + 1, dtype=torch.int32, device=dev)
                wbytes = _cabi.lib().nb200_sptrsv_analysis_workspace_bytes(n)
                work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
                nlevels = ctypes.c_int64(0)
                _cabi.call("nb200_sptrsv_analyse_levels", n, self.nnz, _ptr(idx), _ptr(ptr), itype, int(bool(lower)),
                           _ptr(order), _ptr(level_ptr), ctypes.byref(nlevels), _ptr(work), wbytes, _stream())
                self.extra[key + ("level_ptr",)] = level_ptr[:int(nlevels.value) + 1].clone()
                _published(dev)
            self.extra[key] = (order, int(nlevels.value))
        return self.extra[key]

    def sptrsv_level_plan(self, lower, transposed=False):
        """Position-ordered structure for the cluster solve (``nb200_sptrsv_level_plan``), or None for
        an empty matrix: a dict with ``level_ptr, pos_ptr, dep, src`` (device int32 arrays) and the
        host numbers ``entries, reach, longest_row, widest_level, nlevels``."""
        key = ("sptrsv_levels", bool(lower), bool(transposed))
        if key not in self.extra:
            order, nlevels = self.sptrsv_order(lower, transposed)
            n = self.rows
            if n == 0 or nlevels == 0 or self.nnz >= 2 ** 31 - 1:
                self.extra[key] = None
                return None
            level_ptr = self.extra[("sptrsv", bool(lower), bool(transposed), "level_ptr")]
            idx, ptr, itype = self.csr()
            perm = None
            if transposed:
                t_indptr, t_indices, perm, _ = self.transpose()
                idx, ptr = t_indices, t_indptr
            dev = self.indices.device
            with torch.cuda.device(dev):
                pos_ptr = torch.empty(n + 1, dtype=torch.int32, device=dev)
                dep = torch.empty(max(self.nnz, 1), dtype=torch.int32, device=dev)
                src = torch.empty(max(self.nnz, 1), dtype=torch.int32, device=dev)
                wbytes = _cabi.lib().nb200_sptrsv_level_plan_workspace_bytes(n)
                work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
                info = (ctypes.c_int64 * 4)()
                _cabi.call("nb200_sptrsv_level_plan", n, self.nnz, _ptr(idx), _ptr(ptr), _ptr(perm) if perm is not None else None,
                           itype, int(bool(lower)), _ptr(order), _ptr(level_ptr), nlevels, _ptr(pos_ptr), _ptr(dep), _ptr(src),
                           info, _ptr(work), wbytes, _stream())
                entries = int(info[0])
                self.extra[key] = {"level_ptr": level_ptr, "pos_ptr": pos_ptr, "dep": dep[:max(entries, 1)].clone(),
                                   "src": src[:max(entries, 1)].clone(), "entries": entries, "reach": int(info[1]),
                                   "longest_row": int(info[2]), "widest_level": int(info[3]), "nlevels": nlevels}
                _published(dev)
        return self.extra[key]


def transpose_structure(rows, cols, indices, indptr, itype_in, itype_out):
    """Run nb200_csr_transpose_structure; returns (t_indptr, t_indices, t_perm)."""
    nnz = int(indices.numel())
    dev = indices.device
    odt = torch.int32 if itype_out == _cabi.I32 else torch.int64
    with torch.cuda.device(dev):
        t_indptr = torch.empty(cols + 1, dtype=odt, device=dev)
        t_indices = torch.empty(nnz, dtype=odt, device=dev)
        t_perm = torch.empty(nnz, dtype=odt, device=dev)
        wbytes = _cabi.lib().nb200_csr_transpose_workspace_bytes(rows, cols, nnz)
        work = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        _cabi.call("nb200_csr_transpose_structure", rows, cols, nnz, _ptr(indices), _ptr(indptr), itype_in,
                   _ptr(t_indptr), _ptr(t_indices), _ptr(t_perm), itype_out, _ptr(work), wbytes, _stream())
    return t_indptr, t_indices, t_perm


def get_plan(rows, cols, indices, indptr):
    key = (indices.data_ptr(), indptr.data_ptr(), int(indices.numel()), int(rows), int(cols), indices.device.index)
    plan = _CACHE.get(key)
    if plan is not None and plan.version == (indices._version, indptr._version):
        _CACHE.move_to_end(key)
        return plan
    plan = PatternPlan(rows, cols, indices, indptr)
    plan.require()                     # row pointers and column range: nothing may index out of bounds later
    _CACHE[key] = plan
    while len(_CACHE) > _CACHE_SIZE:
        _CACHE.popitem(last=False)
    return plan


def clear_plan_cache():
    _CACHE.clear()
