"""Build libnengo_b200.so in-tree with nvcc for sm_100a.

Usage: ``python -m nengo_ocl_b200.csrc.build [--force] [--verbose]``.
Every translation unit is compiled separately (the neuron and elementwise
units with ``-fmad=false``) and linked into one shared library next to the
Python package, so the built library travels with the source tree.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libnengo_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]

# (source, extra flags)
UNITS = [
    ("nb2_runtime.cu", []),
    ("nb2_gemv.cu", []),
    ("nb2_gemv_pipe.cu", []),
    ("nb2_gemv_block.cu", []),
    ("nb2_spmv.cu", []),
    ("nb2_elementwise.cu", ["-fmad=false"]),
    ("nb2_neurons.cu", ["-fmad=false"]),
    ("nb2_direct.cu", ["-fmad=false"]),
    ("nb2_whitenoise.cu", ["-fmad=false"]),
    ("nb2_conv.cu", ["-fmad=false"]),
    ("nb2_fused.cu", ["-fmad=false"]),
    ("nb2_fused_stream.cu", ["-fmad=false"]),
    ("nb2_exchange.cu", []),
    # the persistent step loop reads what other CTAs wrote earlier in the same launch: global loads in L2 only
    ("nb2_step_loop.cu", ["-fmad=false", "-Xptxas", "-dlcm=cg"]),
    ("nb2_step_loop_single.cu", ["-fmad=false"]),
]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "nengo_b200.h"))
    headers.append(os.path.abspath(__file__))
    objs = []
    rebuilt = False
    for src, extra in UNITS:
        src_path = os.path.join(HERE, src)
        if not os.path.exists(src_path):
            continue
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if not force and _newer(obj, [src_path] + headers):
            continue
        cmd = [nvcc, "-c", src_path, "-o", obj] + ARCH + COMMON + extra
        if verbose:
            cmd += ["-Xptxas", "-v"]
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        rebuilt = True
    if rebuilt or not os.path.exists(LIB) or force:
        tmp = LIB + ".tmp"  # link beside the target and rename: a reader never sees a half-written library
        cmd = [nvcc, "-shared", "-o", tmp] + objs + ARCH + ["-Xcompiler", "-fPIC"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
