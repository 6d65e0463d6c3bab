"""Builds hiptensor_b200/libhiptensor_b200.so in-tree with nvcc for sm_100a.

    python -m hiptensor_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The shared object links the CUDA runtime statically and
resolves the one driver symbol it needs at run time, so it loads on machines with no driver.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libhiptensor_b200.so")

SOURCES = ["planner.cpp", "runtime.cpp", "api.cpp", "c_abi.cpp", "permutation.cu", "reduction.cu",
           "contraction_tiled.cu", "contraction_tcgen05.cu", "contraction_tf32x3.cu", "contraction_complex.cu",
           "contraction_pack.cu"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
              "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_header():
    t = 0
    for d in (CSRC, os.path.join(ROOT, "include"), os.path.join(ROOT, "include", "hiptensor")):
        for f in os.listdir(d):
            if f.endswith((".hpp", ".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr = _newest_header()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", s, "-o", o]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p.returncode, p.stdout + p.stderr

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, rc, out in ex.map(run, jobs):
            if verbose or rc != 0:
                sys.stderr.write("== %s ==\n%s\n" % (src, out))
            failed |= rc != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or not os.path.exists(LIB):
        # link under another name and rename: a reader never sees a half-written library
        tmp = LIB + ".tmp"
        cmd = [_nvcc(), "-shared", "-o", tmp] + objs + ["-Xcompiler", "-fPIC"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
