"""Comparison helpers shared by the parity tests.

Tolerances are the ones the task states for this path: norm-wise relative error 1e-12 for fp64
and 1e-5 for fp32 (the reference tests use the same norm-wise metric, reference
numml/tests/test_spmv.py:18-19); structure (index arrays) must match exactly.
"""
import torch

TOL = {torch.float64: 1e-12, torch.float32: 1e-5}


def relerr(ref, got):
    ref = ref.detach().double().cpu().flatten()
    got = got.detach().double().cpu().flatten()
    assert ref.shape == got.shape, (ref.shape, got.shape)
    den = torch.linalg.norm(ref)
    num = torch.linalg.norm(ref - got)
    return (num / den).item() if den > 0 else num.item()


def assert_close(ref, got, what="", tol=None):
    tol = TOL[ref.dtype] if tol is None else tol
    assert got.dtype == ref.dtype, f"{what}: dtype {got.dtype} != {ref.dtype}"
    e = relerr(ref, got)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"


def assert_same(ref, got, what=""):
    """Bit-exact equality (integers, or floats where the summation order is the reference's)."""
    assert got.dtype == ref.dtype, f"{what}: dtype {got.dtype} != {ref.dtype}"
    assert ref.shape == got.shape, f"{what}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert torch.equal(ref.cpu(), got.cpu()), f"{what}: not bit-identical"


def case(golden, name):
    """All arrays of one golden case as torch tensors."""
    out = {}
    pre = name + "/"
    for k in golden.files:
        if k.startswith(pre):
            out[k[len(pre):]] = torch.from_numpy(golden[k])
    assert out, f"golden case {name} not found"
    return out


def case_names(golden, prefix):
    return sorted({k.split("/")[0] for k in golden.files if k.startswith(prefix)})
