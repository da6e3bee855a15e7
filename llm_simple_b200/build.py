"""Build libgpu_ops.so (CUDA kernels + C ABI + C++ host layer) in-tree for sm_100a.

    python -m llm_simple_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is written next to this file so
that it travels with the source tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libgpu_ops.so")
OBJ = os.path.join(HERE, "csrc", "_obj")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_SOURCES = ["rope_append.cu", "attn_mma.cu", "attn_tc5.cu", "attn_tc5p.cu", "gpu_ops.cu", "decode_noalloc.cu", "xchg_merge.cu",
                "attn_decode_tma.cu"]
CXX_SOURCES = ["decode_plan.cpp", "host/device_gpu.cpp", "host/attention_layer_gpu.cpp", "host/host_abi.cpp"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"),
          "-I", CSRC, "-I", os.path.join(CSRC, "host"), "-ccbin", "g++"]


def _newer(src_paths, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_paths)


def _deps():
    out = []
    for d in (CSRC, os.path.join(CSRC, "host"), os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".hpp", ".cuh")):
                out.append(os.path.join(d, f))
    return out


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    deps = _deps()
    objs = []
    procs = []
    for src in CUDA_SOURCES + CXX_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, os.path.splitext(src)[0].replace("/", "_") + ".o")
        objs.append(o)
        if force or _newer([s] + deps, o):
            cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            if src.endswith(".cpp"):
                cmd = [NVCC] + COMMON + ["-x", "cu"] + ARCH + ["-c", s, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write("== %s ==\n%s\n" % (src, out))
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _newer(objs, LIB):
        cmd = [NVCC] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcudart", "-ccbin", "g++"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
