"""CPU checks of the C-ABI boundary: the shared library builds, loads without a GPU, exports
every function that include/numml_b200.h declares, and the ctypes table covers the same set."""
import os
import re

from numml_b200 import _cabi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "numml_b200.h")).read()
    return sorted(set(re.findall(r"NB200_API\s+[\w\s\*]+?\b(nb200_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "nb200_spgemv_forward" in names and "nb200_spgemv_backward" in names
    assert len(names) >= 10


def test_library_exports_every_declared_symbol():
    build.build()
    handle = _cabi.lib()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_ctypes_table_matches_header():
    assert sorted(_cabi.SIGNATURES) == declared_functions()


def test_version_and_status_strings():
    handle = _cabi.lib()
    assert handle.nb200_version() >= 100
    assert handle.nb200_status_string(0) == b"ok"
    assert b"aligned" in handle.nb200_status_string(2)


def test_argument_validation_needs_no_gpu():
    # negative sizes are rejected before any CUDA call is made
    handle = _cabi.lib()
    assert handle.nb200_spgemv_forward(-1, 1, 0, None, None, None, None, None, None, 0, None, 1, 1, None) == 1
    assert handle.nb200_gather(-5, None, None, None, 0, 0, None) == 1


def test_compiled_shim_builds_and_refuses_cpu_tensors():
    """The torch extension with the per-call path of the SpMV / SpMM operators compiles against the
    installed torch, links to the CUDA library, imports without a GPU, and (like the Python shim)
    raises on CPU tensors instead of computing anything."""
    import pytest
    import torch
    from numml_b200 import numml_torch_cpp as ops
    assert os.path.exists(build.build_extension())
    ext = ops.compiled_shim()
    assert ext is not None and ext.library_version() == _cabi.lib().nb200_version()
    d, i, p, x = torch.ones(2), torch.zeros(2, dtype=torch.long), torch.tensor([0, 1, 2]), torch.ones(2)
    for call in (lambda: ops.spgemv_forward(2, 2, d, i, p, x), lambda: ops.spgemv_backward(x, 2, 2, d, i, p, x),
                 lambda: ops.spdmm_forward(2, 2, d, i, p, torch.ones(2, 3)),
                 lambda: ops.spdmm_backward(2, 2, d, i, p, torch.ones(2, 3), torch.ones(2, 3))):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()
