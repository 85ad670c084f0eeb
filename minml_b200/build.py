"""Builds libminml_b200.so in-tree with nvcc for sm_100a.

Usage:  python -m minml_b200.build [--force] [--verbose]

Each .cu file under minml_b200/csrc is compiled to an object file (in parallel) and the objects are linked into
minml_b200/libminml_b200.so.  Objects are rebuilt only when their source or a header is newer.  The library links
the CUDA runtime statically and fetches the one driver entry point it needs (cuTensorMapEncodeTiled) at run time,
so it has no link-time dependency on libcuda.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
OBJ = os.path.join(ROOT, "build")
LIB = os.path.join(ROOT, "libminml_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def find_nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put it on PATH")


def _newest_header():
    times = [os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    times.append(os.path.getmtime(os.path.join(ROOT, "..", "include", "minml_b200.h")))
    return max(times)


def build(force=False, verbose=False):
    nvcc = find_nvcc()
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    header_time = _newest_header()
    jobs = []
    for src in sources:
        src_path = os.path.join(CSRC, src)
        obj_path = os.path.join(OBJ, src[:-3] + ".o")
        stale = force or not os.path.exists(obj_path) or os.path.getmtime(obj_path) < max(os.path.getmtime(src_path), header_time)
        jobs.append((src_path, obj_path, stale))

    def compile_one(job):
        src_path, obj_path, stale = job
        if not stale:
            return obj_path, ""
        cmd = [nvcc] + NVCC_FLAGS + ["-c", src_path, "-o", obj_path]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (src_path, proc.stdout, proc.stderr))
        return obj_path, proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, jobs))
    if verbose:
        for _, log in results:
            if log:
                print(log)
    objects = [obj for obj, _ in results]
    relink = force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objects)
    if relink:
        cmd = [nvcc, "-shared", "-o", LIB] + objects + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
