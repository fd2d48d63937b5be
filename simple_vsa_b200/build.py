"""Build the CUDA library in-tree: ``python simple_vsa_b200/build.py`` (run as a script, so that
it works before the library exists).

Compiles every ``csrc/*.cu`` for sm_100a with nvcc and links
``simple_vsa_b200/libvsa_b200.so`` (plain C ABI, static CUDA runtime, no
dependency on PyTorch).  Objects are rebuilt only when a source or header is
newer than them.
"""

from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libvsa_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link; returns the path of the shared library."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(CSRC, "*.inl")) + \
        glob.glob(os.path.join(os.path.dirname(PKG), "include", "*.h"))
    objects = []
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        extra = os.environ.get("VSA_EXTRA_NVCC_FLAGS", "").split()
        proc = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, proc

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs)))) as pool:
        for src, proc in pool.map(compile_one, jobs):
            if verbose or proc.returncode:
                sys.stderr.write(proc.stdout + proc.stderr)
            if proc.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
            with open(os.path.join(OBJ, os.path.basename(src)[:-3] + ".ptxas.txt"), "w") as fh:
                fh.write(proc.stderr)
    if force or jobs or _stale(LIB, objects):
        proc = subprocess.run([nvcc, "-shared", "-o", LIB, *objects, "-gencode", "arch=compute_100a,code=sm_100a"],
                              capture_output=True, text=True)
        if proc.returncode:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
