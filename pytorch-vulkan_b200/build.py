"""Build the in-tree native artefacts with nvcc for sm_100a.

  python pytorch-vulkan_b200/build.py            # libb200conv.so (the C-ABI library)
  python pytorch-vulkan_b200/build.py --torch    # also the PrivateUse1 extension torch_vulkan/_C.so

Outputs live next to the sources (git-ignored) so they travel with a snapshot of the tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200conv.so")
SOURCES = ["runtime.cu", "conv_simt.cu", "conv_tc.cu", "conv_api.cu", "conv_static.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++", "--use_fast_math=false"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_lib(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "b200conv.h"))
    if not (force or _newer(LIB, deps)):
        return LIB
    objs = []
    procs = []
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    if verbose:
        flags += ["-Xptxas", "-v"]
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for s in srcs:
        o = os.path.join(HERE, "build", os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer(o, deps):
            procs.append(subprocess.Popen(["nvcc", *flags, "-c", s, "-o", o]))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed")
    subprocess.check_call(["nvcc", "-shared", "-o", LIB, *objs, "-ccbin", "/usr/bin/g++", "-lcudart", "-lcuda"])
    return LIB


if __name__ == "__main__":
    build_lib(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if "--torch" in sys.argv:
        sys.path.insert(0, HERE)
        from torch_backend_build import build_torch_extension
        build_torch_extension()
    print("built", LIB)
