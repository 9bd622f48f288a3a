"""Ahead-of-time build of the sm_100a kernel library.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an
object and linked into one shared library next to this file (``libkb200.so``).  The sources do not
include PyTorch headers: each exports ``extern "C"`` launchers that take raw device pointers and a
``cudaStream_t``, and Python calls them through ``ctypes`` (see ``loader.py``).  Compiling needs no
GPU.  A stamp file records the hash of the sources and flags so an up-to-date library is reused.
"""

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(HERE, "libkb200.so")
STAMP = os.path.join(HERE, "libkb200.stamp")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the sm_100a kernel library cannot be built.")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in sorted(os.listdir(CSRC)):
        if path.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, path), "rb") as f:
                h.update(path.encode())
                h.update(f.read())
    return h.hexdigest()


def is_current():
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _digest()


def build(force=False, verbose=False):
    """Compile and link; returns the library path."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    os.makedirs(BUILD_DIR, exist_ok=True)
    logs = {}

    def compile_one(src):
        obj = os.path.join(BUILD_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, "-c", src, "-o", obj, "-I", CSRC] + NVCC_FLAGS
        r = subprocess.run(cmd, capture_output=True, text=True)
        logs[src] = r.stdout + r.stderr
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, sources()))
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-L", cuda_lib, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(os.path.join(BUILD_DIR, "ptxas.log"), "w") as f:
        for src, log in logs.items():
            f.write(f"==== {os.path.basename(src)}\n{log}\n")
    with open(STAMP, "w") as f:
        f.write(_digest())
    if verbose:
        for src, log in logs.items():
            print(f"==== {os.path.basename(src)}\n{log}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
