"""Builds libcdeep.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run as ``python -m complexity_deep_b200.build``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libcdeep.so")
# the checking build: same sources with -DCDEEP_CHECKS (device-side validation of indices that
# kernels read from device memory; see include/cdeep.h, cd_checks_enabled)
CHECKS_LIB_PATH = os.path.join(PKG_DIR, "libcdeep_checks.so")
SOURCES = ["api.cu", "gemm.cu", "route.cu", "rowwise.cu", "attention_decode.cu", "attention_prefill.cu", "pack.cu", "ep_plan.cu"]
HEADERS = ["ptx.cuh", "checks.cuh", "gemm_sm100.cuh", "kernels.h", os.path.join("..", "..", "include", "cdeep.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libcdeep.so cannot be built")


def is_stale(checks: bool = False) -> bool:
    lib = CHECKS_LIB_PATH if checks else LIB_PATH
    if not os.path.exists(lib):
        return True
    built = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > built for d in deps)


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool, checks: bool = False):
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-c", src, "-o", obj]
    if checks:
        cmd[1:1] = ["-DCDEEP_CHECKS"]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    return src, subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)


def build(force: bool = False, verbose: bool = False, checks: bool = False) -> str:
    """Compiles every CUDA source of the package (in parallel, one object per source, objects
    of unchanged sources are re-used) and links them into one shared library.  checks=True
    builds the checking variant (libcdeep_checks.so) instead."""
    lib_path = CHECKS_LIB_PATH if checks else LIB_PATH
    if not force and not is_stale(checks):
        return lib_path
    from concurrent.futures import ThreadPoolExecutor
    nvcc = _nvcc()
    obj_dir = os.path.join(CSRC, "build_checks" if checks else "build")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    newest_header = max(os.path.getmtime(h) for h in headers if os.path.exists(h))
    jobs, objs = [], []
    for src in SOURCES:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        src_time = max(os.path.getmtime(os.path.join(CSRC, src)), newest_header)
        if force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < src_time:
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        results = list(pool.map(lambda j: _compile_one(nvcc, j[0], j[1], verbose, checks), jobs))
    for src, proc in results:
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + proc.stdout + proc.stderr)
        if verbose:
            sys.stderr.write(proc.stderr)
    link = subprocess.run([nvcc, "-shared", "-Xcompiler", "-fPIC", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-o", lib_path] + objs,
                          cwd=CSRC, capture_output=True, text=True)
    if link.returncode != 0:
        raise RuntimeError("link failed:\n" + link.stdout + link.stderr)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checks="--checks" in sys.argv))
