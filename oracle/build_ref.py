"""Builds the reference itself, unmodified, from its sources where they lie (the read-only checkout named by
VDNN_REFERENCE_DIR, or a directory `reference` beside this repository), into oracle/_ref/ (git-ignored binaries).
TEST INFRASTRUCTURE ONLY.

  oracle/_ref/vdnn_ref      the reference's command-line program (vdnn.cu + network.cu + layer.cu)
  oracle/_ref/ref_harness   oracle/ref/ref_harness.cu linked against the reference's Layer class
  oracle/_ref/ref_warm      oracle/ref/ref_warm.cu: the reference's Network run for several iterations in one process
  oracle/_ref/vdnn_dropin   the reference's vdnn.cu + network.cu, unmodified, driving this library's Layer class
                            (libvdnn_b200.so) through csrc/ref_dropin.h: the drop-in claim, compiled

What the reference needs and does not ship is supplied from this repository:
  * cuDNN 7's algorithm-preference calls (removed in cuDNN 8): oracle/ref/ref_compat.h, force-included;
  * cnmem (not vendored by the reference, layer.h:21): the cnmem-compatible pool of this library
    (include/cnmem/include/cnmem.h + csrc/pool_alloc.cpp); VDNN_POOL_BYTES caps its reservation, since the
    reference asks for the whole device (network.cu:49).
Run the binaries with NVIDIA_TF32_OVERRIDE=0 so that cuDNN's fp32 convolutions use FMA arithmetic: the
reference never sets a math type, and on this architecture the default would be TF32.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
# Where the reference checkout is: VDNN_REFERENCE_DIR, else a directory named `reference` beside this repository.
REF = os.environ.get("VDNN_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
OUT = os.path.join(HERE, "_ref")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def run(cmd):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + p.stdout[-4000:])
        raise RuntimeError("reference build failed")


def build():
    if not os.path.isdir(REF):
        print("reference sources not present; keeping prebuilt oracle/_ref if any")
        return False
    os.makedirs(OUT, exist_ok=True)
    common = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-w",
              "-ccbin", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++",
              "-include", os.path.join(HERE, "ref", "ref_compat.h"),
              "-I", os.path.join(ROOT, "include"), "-I", REF, "-I", "/usr/include/x86_64-linux-gnu"]
    objs = []
    for src in ("layer.cu", "network.cu"):
        obj = os.path.join(OUT, src + ".o")
        run(common + ["-c", os.path.join(REF, src), "-o", obj])
        objs.append(obj)
    pool = os.path.join(OUT, "pool_alloc.o")
    run(common + ["-c", os.path.join(ROOT, "vdnn_implementation_b200", "csrc", "pool_alloc.cpp"), "-o", pool])
    rng = os.path.join(OUT, "host_rng.o")
    run(common + ["-Xcompiler", "-ffp-contract=off", "-c", os.path.join(ROOT, "vdnn_implementation_b200", "csrc", "host_rng.cpp"), "-o", rng])
    libs = ["-lcudnn", "-lcublas", "-lpthread"]
    run(common + [os.path.join(REF, "vdnn.cu")] + objs + [pool, "-o", os.path.join(OUT, "vdnn_ref")] + libs)
    run(common + [os.path.join(HERE, "ref", "ref_harness.cu"), objs[0], pool, rng, "-o", os.path.join(OUT, "ref_harness")] + libs)
    run(common + [os.path.join(HERE, "ref", "ref_warm.cu")] + objs + [pool, "-o", os.path.join(OUT, "ref_warm")] + libs)
    # the reference's driver (vdnn.cu + network.cu, unmodified) on top of THIS library's Layer class: its layer.h / vdnn.h are
    # displaced by the force-included csrc/ref_dropin.h, layer.cu is not compiled at all, and cuDNN / cuBLAS are not linked
    pkg = os.path.join(ROOT, "vdnn_implementation_b200")
    if os.path.exists(os.path.join(pkg, "libvdnn_b200.so")):
        run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-w",
             "-ccbin", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++",
             "-include", os.path.join(pkg, "csrc", "ref_dropin.h"), "-I", os.path.join(pkg, "csrc"), "-I", os.path.join(ROOT, "include"),
             os.path.join(REF, "vdnn.cu"), os.path.join(REF, "network.cu"), "-o", os.path.join(OUT, "vdnn_dropin"),
             "-L", pkg, "-lvdnn_b200", "-Xlinker", "-rpath=$ORIGIN/../../vdnn_implementation_b200"])
    for o in objs + [pool, rng]:
        os.remove(o)
    return True


if __name__ == "__main__":
    if build():
        print(os.path.join(OUT, "vdnn_ref"))
        print(os.path.join(OUT, "ref_harness"))
        print(os.path.join(OUT, "ref_warm"))
        print(os.path.join(OUT, "vdnn_dropin"))
