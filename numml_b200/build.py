"""Compile the CUDA sources under ``numml_b200/csrc`` into ``numml_b200/lib/libnumml_b200.so``.

One nvcc invocation per ``.cu`` file (run in parallel), sm_100a only, then one link step.  The
library has no dependency on torch or Python; it links the CUDA runtime statically, so it also
loads on a machine without a GPU (where only the symbol table can be checked).

Usage:  python -m numml_b200.build [--force] [--verbose]
"""
import argparse
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libnumml_b200.so")
HEADER = os.path.join(os.path.dirname(PKG), "include", "numml_b200.h")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _deps_mtime():
    files = glob.glob(os.path.join(SRC_DIR, "*.cuh")) + [HEADER]
    return max(os.path.getmtime(f) for f in files)


def build(force=False, verbose=False, ptxas_info=False):
    """Build the shared library if any source is newer than it.  Returns its path."""
    srcs = sorted(glob.glob(os.path.join(SRC_DIR, "*.cu")))
    if not srcs:
        raise RuntimeError("no CUDA sources found under " + SRC_DIR)
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = _deps_mtime()
    jobs = []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o")
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time)
        if stale:
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            jobs.append((s, cmd))
    objs = [os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o") for s in srcs]

    def run(job):
        s, cmd = job
        if verbose:
            print(" ".join(cmd), flush=True)
        p = subprocess.run(cmd, capture_output=True, text=True)
        return s, p.returncode, p.stdout + p.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            results = list(ex.map(run, jobs))
        for s, rc, out in results:
            if out.strip() and (verbose or ptxas_info or rc != 0):
                print(out, file=sys.stderr)
            if rc != 0:
                raise RuntimeError("nvcc failed for " + s)
    if jobs or not os.path.exists(LIB_PATH):
        link = [_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-cudart", "static"]
        if verbose:
            print(" ".join(link), flush=True)
        subprocess.check_call(link)
    return LIB_PATH


EXT_SRC = os.path.join(PKG, "csrc_ext", "ops_ext.cpp")
EXT_NAME = "numml_b200_ext"


def extension_path():
    import sysconfig
    return os.path.join(LIB_DIR, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_extension(force=False, verbose=False):
    """Compile the torch extension with the per-call path of the SpMV / SpMM operators
    (``csrc_ext/ops_ext.cpp``) against the installed torch and link it to ``libnumml_b200.so`` (found at
    run time next to itself).  Returns its path."""
    import sysconfig
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    build()
    out = extension_path()
    newest = max(os.path.getmtime(EXT_SRC), os.path.getmtime(HEADER))
    if os.path.exists(out) and not force and os.path.getmtime(out) >= newest:
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = ["-I" + p for p in include_paths()] + ["-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(cuda_home, "include")]
    libdirs = library_paths()
    cmd = (["g++", "-std=c++17", "-O2", "-fPIC", "-w", "-shared", "-DNDEBUG", "-DTORCH_EXTENSION_NAME=" + EXT_NAME,
            "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
           + incs + [EXT_SRC, "-o", out] + ["-L" + d for d in libdirs] + ["-Wl,-rpath," + d for d in libdirs]
           + ["-L" + LIB_DIR, "-Wl,-rpath,$ORIGIN", "-lnumml_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
              "-ltorch", "-ltorch_python"])
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--no-extension", action="store_true", help="skip the compiled operator shim")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.ptxas_info))
    if not a.no_extension:
        print(build_extension(a.force, a.verbose))
