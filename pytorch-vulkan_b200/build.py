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
SOURCES = ["runtime.cu", "conv_simt.cu", "conv_group_small.cu", "conv_tc.cu", "conv_tc_strip.cu", "conv_tc_tstrip.cu", "dweight_tc_strip.cu", "winograd.cu", "conv_api.cu", "conv_static.cu", "conv_nd.cu", "batch_norm.cu", "group_norm.cu", "attention.cu", "comm.cu"]
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
    subprocess.check_call(["nvcc", "-shared", "-o", LIB, *objs, "-ccbin", "/usr/bin/g++", "-lcudart", "-lcuda", "-ldl"])
    return LIB


def build_torch_extension(force=False):
    """g++ build of the PrivateUse1 extension torch_vulkan/_C.so (host code only; it links
    libb200conv.so and the installed torch libraries)."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    build_lib()
    src_dir = os.path.join(CSRC, "torch_backend")
    srcs = [os.path.join(src_dir, f) for f in sorted(os.listdir(src_dir)) if f.endswith(".cpp")]
    deps = srcs + [os.path.join(src_dir, "backend.h"), os.path.join(HERE, "..", "include", "b200conv.h")]
    out = os.path.join(HERE, "torch_vulkan", "_C.so")
    if not (force or _newer(out, deps)):
        return out
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    incs = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    flags = ["-std=c++17", "-O2", "-fPIC", "-shared", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(HERE, "build", os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer(o, deps):
            procs.append(subprocess.Popen(["/usr/bin/g++", *[f for f in flags if f != "-shared"], *incs, "-c", s, "-o", o]))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("g++ failed")
    subprocess.check_call(["/usr/bin/g++", "-shared", "-o", out, *objs, f"-L{HERE}", "-lb200conv", f"-L{torch_lib}",
                           "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
                           "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{torch_lib}"])
    return out


if __name__ == "__main__":
    build_lib(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if "--torch" in sys.argv:
        build_torch_extension(force="--force" in sys.argv)
    print("built", LIB)
