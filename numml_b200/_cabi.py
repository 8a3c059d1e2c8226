"""ctypes binding of ``libnumml_b200.so`` (the C ABI declared in ``include/numml_b200.h``).

The library is the only compute path of this package: if it is missing, loading fails with an
error instead of falling back to anything else.
"""
import ctypes
import os

from . import build as _build

_c = ctypes
_i64, _int, _vp, _sz = _c.c_int64, _c.c_int, _c.c_void_p, _c.c_size_t

F32, F64 = 0, 1
I32, I64 = 0, 1

# name -> (restype, argtypes); mirrors include/numml_b200.h one to one
SIGNATURES = {
    "nb200_version": (_int, []),
    "nb200_status_string": (_c.c_char_p, [_int]),
    "nb200_spgemv_forward": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp, _int, _int, _vp]),
    "nb200_spgemv_backward": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int,
                                     _vp, _int, _int, _vp]),
    "nb200_spgemv_backward_symmetric_rows": (_int, [_i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int,
                                                    _vp, _int, _int, _vp]),
    "nb200_csr_values_symmetric": (_int, [_i64, _vp, _vp, _vp, _int, _int, _vp]),
    "nb200_spgemv_grad_A": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _int, _vp, _int, _int, _vp]),
    "nb200_csr_block_profile": (_int, [_i64, _vp, _int, _vp, _vp]),
    "nb200_spmv_pipeline_tile": (_int, []),
    "nb200_csr_check": (_int, [_i64, _i64, _i64, _vp, _vp, _int, _vp, _vp]),
    "nb200_csr_transpose_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "nb200_csr_transpose_structure": (_int, [_i64, _i64, _i64, _vp, _vp, _int, _vp, _vp, _vp, _int, _vp, _sz, _vp]),
    "nb200_gather": (_int, [_i64, _vp, _vp, _vp, _int, _int, _vp]),
    "nb200_scatter": (_int, [_i64, _vp, _vp, _vp, _int, _int, _vp]),
    "nb200_narrow_indices": (_int, [_i64, _vp, _vp, _vp]),
    "nb200_widen_indices": (_int, [_i64, _vp, _vp, _vp]),
    "nb200_spdmm_forward": (_int, [_i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp]),
    "nb200_spgemm_workspace_bytes": (_sz, [_i64]),
    "nb200_spgemm_plan": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _int, _int, _vp, _sz, _vp]),
    "nb200_spgemm_symbolic": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp, _sz, _vp, _i64, _vp, _vp]),
    "nb200_spgemm_numeric": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp, _sz, _vp, _i64,
                                    _vp, _vp, _vp, _vp]),
    "nb200_spgemm_backward": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp,
                                     _vp, _vp, _vp, _vp, _vp, _int, _int, _vp]),
    "nb200_sptrsv_analysis_workspace_bytes": (_sz, [_i64]),
    "nb200_sptrsv_analyse": (_int, [_i64, _i64, _vp, _vp, _vp, _vp, _int, _int, _vp, _vp, _vp, _sz, _vp]),
    "nb200_sptrsv_solve": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _i64,
                                  _int, _int, _int, _vp]),
    "nb200_sptrsv_analyse_levels": (_int, [_i64, _i64, _vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nb200_sptrsv_level_plan_workspace_bytes": (_sz, [_i64]),
    "nb200_sptrsv_level_plan": (_int, [_i64, _i64, _vp, _vp, _vp, _int, _int, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                                       _vp, _sz, _vp]),
    "nb200_sptrsv_solve_levels_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "nb200_sptrsv_solve_levels": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _vp,
                                         _vp, _sz, _int, _int, _vp]),
    "nb200_sptrsv_solve_f32_noalloc_capacity": (_i64, []),
    "nb200_sptrsv_solve_f32_noalloc": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp, _vp, _vp, _i64,
                                              _int, _vp]),
    "nb200_cg_workspace_bytes": (_sz, [_i64, _int]),
    "nb200_cg_fixed_iterations": (_int, [_i64, _i64, _vp, _vp, _vp, _int, _vp, _vp, _int, _vp, _i64, _vp, _sz, _vp,
                                         _int, _int, _vp]),
    "nb200_masked_outer": (_int, [_i64, _i64, _i64, _vp, _vp, _vp, _vp, _c.c_double, _vp, _int, _int, _vp]),
    "nb200_cg_peer_workspace_bytes": (_sz, []),
    "nb200_cg_peer_phase": (_int, [_int, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _int, _int, _vp, _vp, _vp, _i64, _int, _vp]),
    "nb200_pattern_workspace_bytes": (_sz, [_i64]),
    "nb200_csr_triangle_count": (_int, [_i64, _vp, _vp, _i64, _int, _vp, _vp, _sz, _vp]),
    "nb200_csr_triangle_fill": (_int, [_i64, _vp, _vp, _vp, _i64, _int, _vp, _vp, _vp, _vp, _int, _vp]),
    "nb200_csr_lincomb_count": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nb200_csr_lincomb_fill": (_int, [_i64, _c.c_double, _vp, _vp, _vp, _c.c_double, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "nb200_csr_lincomb_backward": (_int, [_i64, _c.c_double, _vp, _vp, _c.c_double, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "nb200_coo_workspace_bytes": (_sz, [_i64]),
    "nb200_coo_to_csr": (_int, [_i64, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "nb200_splu_workspace_bytes": (_sz, [_i64]),
    "nb200_splu_symbolic_count": (_int, [_i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nb200_splu_symbolic_fill": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _int, _vp]),
    "nb200_splu_numeric": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _i64, _int, _vp]),
    "nb200_halo_publish": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _int, _vp, _int, _vp]),
    "nb200_halo_publish_rowsums": (_int, [_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp, _int, _int, _vp]),
    "nb200_halo_pull": (_int, [_int, _vp, _i64, _vp, _vp, _vp, _i64, _int, _vp]),
    "nb200_halo_pull_add": (_int, [_int, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _vp]),
    "nb200_halo_pull_rows": (_int, [_int, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "nb200_halo_pull_add_rows": (_int, [_int, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _int, _vp]),
    "nb200_ipc_alloc": (_int, [_sz, _c.POINTER(_vp), _vp]),
    "nb200_ipc_open": (_int, [_vp, _c.POINTER(_vp)]),
    "nb200_ipc_close": (_int, [_vp]),
    "nb200_ipc_free": (_int, [_vp]),
    "nb200_spdmm_backward_grad_A": (_int, [_i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _vp]),
}

_lib = None


class NB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn, status, text):
        super().__init__(f"{fn} failed: status {status} ({text})")
        self.status = status


def library_path():
    return _build.LIB_PATH


def lib():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: the CUDA library of numml_b200 has not been built "
                "(run `python -m numml_b200.build`); there is no fallback path.")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


_functions = {}


def call(name, *args):
    """Call an int-status entry point and raise NB200Error on failure."""
    fn = _functions.get(name)
    if fn is None:
        fn = _functions[name] = getattr(lib(), name)
    status = fn(*args)
    if status != 0:
        raise NB200Error(name, status, lib().nb200_status_string(status).decode())
