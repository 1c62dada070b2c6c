"""Builds libvdnn_b200.so (kernels + C ABI + host driver) and the `vdnn` command-line binary.

In-tree build with nvcc for sm_100a only.  Run as `python -m vdnn_implementation_b200.build`.
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libvdnn_b200.so")
CLI = os.path.join(PKG, "vdnn")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
          "-ccbin", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"]

CUDA_SOURCES = ["elementwise.cu", "conv_api.cu", "dp_peer.cu", "layer.cu", "network.cu"]
HOST_SOURCES = ["pool_alloc.cpp", "host_rng.cpp", "dp_nccl.cpp", "network_abi.cpp"]
# every header under csrc/ (a source is rebuilt when any of them is newer) plus the two public ones
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))) + [
    os.path.join(ROOT, "include", "vdnn_b200.h"), os.path.join(ROOT, "include", "cnmem", "include", "cnmem.h")]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout)
        raise RuntimeError("build failed: " + os.path.basename(cmd[-1]))
    return proc.stdout


def build(force=False, verbose=False):
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    objects = []
    log = []
    for src in CUDA_SOURCES + HOST_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(objdir, src + ".o")
        objects.append(obj)
        if force or _newer(obj, [path] + headers):
            host_flags = "-fPIC,-ffp-contract=off" if src == "host_rng.cpp" else "-fPIC"
            extra = ["-Xptxas", "-v"] if src.endswith(".cu") else []
            log.append(_run([NVCC] + ARCH + COMMON + extra + ["-Xcompiler", host_flags, "-c", path, "-o", obj]))
    if force or _newer(LIB, objects):
        _run([NVCC] + ARCH + ["-shared", "-o", LIB] + objects + ["-ldl", "-lpthread"])
    main_src = os.path.join(CSRC, "vdnn_main.cu")
    if force or _newer(CLI, [main_src, LIB] + headers):
        _run([NVCC] + ARCH + COMMON + [main_src, "-o", CLI, "-L", PKG, "-lvdnn_b200", "-Xlinker", "-rpath=$ORIGIN"])
    if verbose:
        sys.stdout.write("".join(log))
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
