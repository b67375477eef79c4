#!/usr/bin/env python
"""Build the native parts in-tree.

  libffk.so   -- the sm_100a CUDA kernel library (csrc/kernels/*.cu), plain C API
  _ffcore.so  -- the C++ compiler core (csrc/core/*.cc), pybind11 module

Both are compiled straight with nvcc / g++ (no JIT cache), so the shared
objects sit inside the package and travel with a copy of the tree.
Usage: python build.py [--force] [--kernels-only|--core-only] [--sanitize] [--ptxas-info] [-v]
"""
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flexflow_train_b200")
KSRC = os.path.join(PKG, "csrc", "kernels")
CSRC = os.path.join(PKG, "csrc", "core")
BUILD = os.path.join(ROOT, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("command failed: " + " ".join(cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build_kernels(force=False, verbose=False, ptxas_info=False):
    os.makedirs(os.path.join(BUILD, "kernels"), exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(KSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(KSRC, "*.cuh")) + glob.glob(os.path.join(KSRC, "*.h"))
    out = os.path.join(PKG, "libffk.so")
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(BUILD, "kernels", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    if jobs or force or _stale(out, objs):
        # link beside the target and rename: a reader (an import, a copy of the tree) never sees a half-written library
        _run([NVCC, "-shared", "-o", out + ".tmp"] + objs + ["-lcudart"], verbose)
        os.replace(out + ".tmp", out)
    return out


def build_core(force=False, verbose=False, sanitize=False):
    """The compiler core.  ``sanitize``: a second copy instrumented with UBSan (undefined behaviour aborts the
    process), written to build/core_ubsan/ and never into the package; the test suite loads it by path."""
    import pybind11

    sub = "core_ubsan" if sanitize else "core"
    os.makedirs(os.path.join(BUILD, sub), exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cc")))
    if not srcs:
        return None
    hdrs = glob.glob(os.path.join(CSRC, "*.h"))
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = os.path.join(BUILD, sub, "_ffcore" + ext) if sanitize else os.path.join(PKG, "_ffcore" + ext)
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + CSRC]
    opt = ["-O1", "-g", "-fsanitize=undefined", "-fno-sanitize-recover=undefined"] if sanitize else ["-O2"]
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(BUILD, sub, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(["g++"] + opt + ["-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-sign-compare"] + inc + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or _stale(out, objs):
        _run(["g++", "-shared", "-o", out + ".tmp"] + objs + (["-fsanitize=undefined"] if sanitize else []), verbose)
        os.replace(out + ".tmp", out)
    return out


def build_all(force=False, verbose=False):
    return build_kernels(force, verbose), build_core(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    if "--core-only" not in sys.argv:
        print(build_kernels(force, verbose, ptxas_info="--ptxas-info" in sys.argv))
    if "--kernels-only" not in sys.argv:
        print(build_core(force, verbose))
        if "--sanitize" in sys.argv:
            print(build_core(force, verbose, sanitize=True))
