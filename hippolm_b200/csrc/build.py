"""Builds ``libhippo_kernels.so`` (all sm_100a kernels) and ``libhippo_host.so`` (host-side fused
accumulator / optimizer math) in-tree with nvcc / g++. No torch headers are involved: kernels take
raw device pointers and a stream, Python calls them through ctypes.

    python -m hippolm_b200.csrc.build [--force] [--verbose]
    HIPPO_DEBUG_BOUNDS=1 python -m hippolm_b200.csrc.build     # second library with checked data-dependent indices

With ``HIPPO_DEBUG_BOUNDS=1`` in the environment the kernels are compiled with ``-DHIPPO_DEBUG_BOUNDS`` into
``libhippo_kernels_dbg.so`` and ``ops/_ext.py`` loads that library: token / target ids and positions are range-checked on
the device, a bad one is recorded in the status word (``_ext.device_status()``: code 8, detail = which check) and the
access is skipped. This stands in for a memory checker where none can be run.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "..", "lib")
DEBUG_BOUNDS = os.environ.get("HIPPO_DEBUG_BOUNDS", "0") not in ("", "0")
KERNEL_LIB = os.path.abspath(os.path.join(OUT_DIR, "libhippo_kernels_dbg.so" if DEBUG_BOUNDS else "libhippo_kernels.so"))
HOST_LIB = os.path.abspath(os.path.join(OUT_DIR, "libhippo_host.so"))
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-rdc=true"]


def _sources(ext):
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(ext))


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode()); h.update(f.read())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    cus = _sources(".cu")
    deps = cus + _sources(".cuh") + _sources(".h")
    stamp = KERNEL_LIB + ".sha"
    dig = _digest(deps)
    if not force and os.path.exists(KERNEL_LIB) and os.path.exists(stamp) and open(stamp).read() == dig:
        return KERNEL_LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    obj_dir = os.path.join(OUT_DIR, "obj_dbg" if DEBUG_BOUNDS else "obj")
    os.makedirs(obj_dir, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DHIPPO_DEBUG_BOUNDS"] if DEBUG_BOUNDS else [])

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        _run([nvcc] + NVCC_FLAGS + extra + ["-dc", src, "-o", obj], verbose)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(cus))) as ex:
        objs = list(ex.map(compile_one, cus))
    _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-rdc=true"]
         + objs + ["-o", KERNEL_LIB, "-lcudart"], verbose)
    with open(stamp, "w") as f:
        f.write(dig)
    return KERNEL_LIB


def build_host(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = _sources(".cpp")
    if not srcs:
        return ""
    stamp = HOST_LIB + ".sha"
    dig = _digest(srcs + _sources(".inl") + [os.path.abspath(__file__)])
    if not force and os.path.exists(HOST_LIB) and os.path.exists(stamp) and open(stamp).read() == dig:
        return HOST_LIB
    # -fno-math-errno: sqrtf must not write errno, or the AdamW loop is not vectorised
    _run(["g++", "-O3", "-march=x86-64-v3", "-fno-math-errno", "-fopenmp", "-fPIC", "-shared", "-std=c++17"] + srcs
         + ["-o", HOST_LIB], verbose)
    with open(stamp, "w") as f:
        f.write(dig)
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_host(force, verbose)


if __name__ == "__main__":
    print(build_all("--force" in sys.argv, "--verbose" in sys.argv))
