"""Build libckv_b200.so in-tree with nvcc for sm_100a (no torch C++ extension involved)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libckv_b200.so")
OBJ_DIR = os.path.join(PKG_DIR, "build")
# debug build with bounds checks in the update kernels (see ckv_bounds_status in the header)
BOUNDS_LIB_PATH = os.path.join(PKG_DIR, "libckv_b200_bounds.so")
BOUNDS_OBJ_DIR = os.path.join(PKG_DIR, "build", "bounds")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_source_mtime():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(os.path.dirname(PKG_DIR), "include", "cascade_kv_b200.h"))
    return max(os.path.getmtime(f) for f in files)


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    """Compile every .cu under csrc/ and link libckv_b200.so next to this file (``bounds``: the debug
    build libckv_b200_bounds.so, compiled with -DCKV_BOUNDS)."""
    lib_path, obj_dir = (BOUNDS_LIB_PATH, BOUNDS_OBJ_DIR) if bounds else (LIB_PATH, OBJ_DIR)
    if not force and os.path.exists(lib_path) and os.path.getmtime(lib_path) >= _newest_source_mtime():
        return lib_path
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libckv_b200.so must be built where the CUDA toolkit is installed")
    os.makedirs(obj_dir, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DCKV_BOUNDS"] if bounds else [])

    def compile_one(src):
        obj = os.path.join(obj_dir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds="--bounds" in sys.argv))
