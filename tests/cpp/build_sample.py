"""Compiles tests/cpp/dropin_sample.cpp against include/hiptensor/hiptensor.hpp and links it with
libhiptensor_b200.so (nvcc as the host-compiler driver; no GPU needed to build)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
EXE = os.path.join(HERE, "dropin_sample")


def build():
    src = os.path.join(HERE, "dropin_sample.cpp")
    lib = os.path.join(ROOT, "hiptensor_b200", "libhiptensor_b200.so")
    if os.path.exists(EXE) and os.path.getmtime(EXE) > max(os.path.getmtime(src), os.path.getmtime(lib)):
        return EXE
    libdir = os.path.dirname(lib)
    subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), src, "-o", EXE,
                           "-L", libdir, "-lhiptensor_b200", "-Xlinker", "-rpath," + libdir])
    return EXE


if __name__ == "__main__":
    print(build())
