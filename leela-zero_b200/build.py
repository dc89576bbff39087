"""Build liblzb200.so (the CUDA kernels and the C ABI) and libcudapipe.so (the
C++ ForwardPipe implementation on top of it) in-tree for sm_100a.

Usage: python leela-zero_b200/build.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
LIB = os.path.join(HERE, "liblzb200.so")
HOSTLIB = os.path.join(HERE, "libcudapipe.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-cudart", "static"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(d, exts):
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = _sources(CSRC, (".cu", ".cuh")) + [os.path.join(ROOT, "include", "lzb200.h")]
    if force or not _newer(LIB, srcs):
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
            "-o", LIB, os.path.join(CSRC, "lzb200.cu")]
        subprocess.run(cmd, check=True)
    if os.path.isdir(HOST):
        hsrcs = _sources(HOST, (".cpp", ".h"))
        cpps = [s for s in hsrcs if s.endswith(".cpp") and not s.endswith("netbench.cpp")]
        if cpps and (force or not _newer(HOSTLIB, hsrcs + [LIB])):
            cmd = ["g++", "-std=c++14", "-O2", "-fPIC", "-shared", "-pthread",
                   "-I" + os.path.join(ROOT, "include"), "-I" + HOST, "-o", HOSTLIB] + cpps + [
                   "-L" + HERE, "-llzb200", "-Wl,-rpath,$ORIGIN"]
            subprocess.run(cmd, check=True)
        nb = os.path.join(HOST, "netbench.cpp")
        exe = os.path.join(HERE, "netbench")
        if os.path.exists(nb) and (force or not _newer(exe, hsrcs + [LIB])):
            subprocess.run(["g++", "-std=c++14", "-O2", "-pthread", "-I" + os.path.join(ROOT, "include"),
                            "-I" + HOST, nb, os.path.join(HOST, "CUDAPipe.cpp"), "-L" + HERE, "-llzb200",
                            "-Wl,-rpath,$ORIGIN", "-o", exe], check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
