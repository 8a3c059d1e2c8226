"""Build the reference's own CPU operator module, unmodified, as the parity oracle.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product path; only the
tests, the smoke check and the CPU-baseline / reference arm of the benchmark may use it.

The two source files that make up the reference's non-CUDA build (``cpp/sparse_csr.cpp`` and
``cpp/sparse_csr_cpu.cpp``, the ``CppExtension`` branch of the reference ``setup.py:32-41``) are
compiled where they lie, with the reference's own flags (``-std=c++17 -DCUDA_ENABLED=0 -O2``),
by calling ``g++`` directly.  The Python module name is whatever ``TORCH_EXTENSION_NAME`` is
defined to (``cpp/sparse_csr.cpp:307``), so the module is built as ``numml_ref_cpp`` and never
clashes with this package's own operator module.  Output goes to ``oracle/_ref/`` only; no
reference source is copied.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
The reference checkout is looked for at --reference, else at $NUMML_REFERENCE, else in a directory
named ``reference`` beside this repository.
"""
import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "numml_ref_cpp"
DEFAULT_REFERENCE = os.environ.get("NUMML_REFERENCE",
                                   os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def ref_module_path():
    return os.path.join(OUT_DIR, MODULE + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference=DEFAULT_REFERENCE, force=False, verbose=True):
    """Compile the reference CPU extension into ``oracle/_ref``.  Returns the .so path, or None
    when the reference sources are not present (e.g. on a machine that only has prebuilt files)."""
    out = ref_module_path()
    srcs = [os.path.join(reference, "cpp", f) for f in ("sparse_csr.cpp", "sparse_csr_cpu.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return out if os.path.exists(out) else None
    if os.path.exists(out) and not force:
        newest = max(os.path.getmtime(s) for s in srcs)
        if os.path.getmtime(out) >= newest:
            return out
    import torch  # noqa: F401  (needed for the include / library paths)
    from torch.utils.cpp_extension import include_paths, library_paths

    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    # -DNDEBUG is what a setuptools build of the reference passes (it comes with the interpreter's own
    # compile flags, sysconfig OPT); without it an assert in the reference's queue (cpp/vector_queue.hpp:20,
    # a "full" test that fires as soon as the queue holds one element) aborts its sparse LU.
    common = ["g++", "-std=c++17", "-DCUDA_ENABLED=0", "-DNDEBUG", "-O2", "-fPIC", "-w",
              "-DTORCH_EXTENSION_NAME=" + MODULE, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    incs = ["-I" + p for p in include_paths()] + ["-I" + sysconfig.get_paths()["include"],
                                                   "-I" + os.path.join(reference, "cpp")]
    procs = []
    for s in srcs:
        o = os.path.join(OUT_DIR, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = common + incs + ["-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("reference CPU build failed")
    libdirs = library_paths()
    link = ["g++", "-shared"] + objs + ["-o", out] + ["-L" + d for d in libdirs] + \
           ["-Wl,-rpath," + d for d in libdirs] + ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.check_call(link)
    for o in objs:
        os.remove(o)
    return out


def load():
    """Import the built reference module (``numml_ref_cpp``).  Raises ImportError if not built."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    path = ref_module_path()
    if not os.path.exists(path):
        raise ImportError("oracle/_ref is not built; run python oracle/build_ref.py")
    spec = importlib.util.spec_from_file_location(MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print("built" if p else "reference sources not found", p)
    sys.exit(0 if p else 1)
