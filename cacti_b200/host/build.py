"""Build libcacti_b200_host.so (the C++ host shim) next to libcacti_b200.so."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIBDIR = os.path.join(HERE, "..", "lib")
LIB = os.path.join(LIBDIR, "libcacti_b200_host.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "thunk_shim.cpp"), os.path.join(HERE, "thunk_shim.hpp")]
    kern = os.path.join(LIBDIR, "libcacti_b200.so")
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs + [kern]):
        return LIB
    # nvcc as the host compiler driver only (no device code here); links the kernel library by rpath
    cmd = [NVCC, "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-o", LIB, srcs[0],
           "-L" + LIBDIR, "-lcacti_b200", "-Xlinker", "-rpath,$ORIGIN", "-Wno-deprecated-gpu-targets"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
