"""Run the reference's own OpenCL kernel source on the CPU.

TEST INFRASTRUCTURE ONLY.  Works only where the reference source tree is
mounted: the reference's ``plan_*`` functions are executed under the stand-in
modules of ``tests/golden/refstubs.py``, the kernel text they render is written
to ``oracle/_ref/`` (git-ignored; reference-derived text never enters the
repository), compiled as C++ with a small NDRange shim and driven over the
plan's global/local sizes.  OpenCL C of these kernels is plain C once
``get_global_id`` is a function, and compiling as C++ makes ``expm1`` /
``log1p`` / ``max`` resolve to their float overloads as in OpenCL.

Work-items run sequentially.  Kernels without barriers are exact.  Kernels
whose barriers only separate "fill local memory" from "use it" are run in
``passes`` sweeps: the first sweeps execute on scratch copies of the buffers
just to fill the (static) local arrays, the last sweep on the real buffers.
"""

import ctypes
import hashlib
import os
import re
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

SHIM = r"""
#include <cmath>
#include <algorithm>
#include <cstdio>
using std::max; using std::min;
#define __kernel static
#define __global
#define __local static
#define CLK_LOCAL_MEM_FENCE 0
#define barrier(x) do {} while (0)
typedef unsigned int uint; typedef unsigned long ulong;
static int g_gid[3], g_gsz[3], g_lsz[3];
static inline int get_global_id(int d) { return g_gid[d]; }
static inline int get_global_size(int d) { return g_gsz[d]; }
static inline int get_local_size(int d) { return g_lsz[d]; }
static inline int get_local_id(int d) { return g_gid[d] % g_lsz[d]; }
static inline int get_group_id(int d) { return g_gid[d] / g_lsz[d]; }
"""


def _signature(text, name):
    mt = re.search(r"__kernel\s+void\s+%s\s*\((.*?)\)\s*\{" % re.escape(name), text, flags=re.S)
    assert mt, "kernel %s not found" % name
    args = [a.strip() for a in mt.group(1).split(",") if a.strip()]
    types = []
    for a in args:
        a = re.sub(r"\b(__global|const)\b", "", a).strip()
        ctype = a[: a.rindex("*") + 1] if "*" in a else " ".join(a.split()[:-1])
        types.append(ctype.replace(" ", ""))
    return types


def compile_kernel(text, name):
    """Compile rendered kernel ``name`` and return a driver
    ``run(args, gsize, lsize, reverse0)`` that sweeps the NDRange once."""
    os.makedirs(REF_DIR, exist_ok=True)
    types = _signature(text, name)
    casts = ", ".join("(%s)a[%d]" % (t, i) for i, t in enumerate(types))
    driver = """
extern "C" void run(void** a, const int* gsize, const int* lsize, int reverse0) {
  for (int d = 0; d < 3; ++d) { g_gsz[d] = gsize[d]; g_lsz[d] = lsize[d]; }
  for (int z = 0; z < gsize[2]; ++z) for (int y = 0; y < gsize[1]; ++y)
    for (int xx = 0; xx < gsize[0]; ++xx) {
      int x = reverse0 ? gsize[0] - 1 - xx : xx;
      g_gid[0] = x; g_gid[1] = y; g_gid[2] = z;
      %s(%s);
    }
}
""" % (name, casts)
    src = SHIM + text + driver
    tag = hashlib.sha1(src.encode()).hexdigest()[:12]
    cpp = os.path.join(REF_DIR, "%s_%s.cpp" % (name, tag))
    so = os.path.join(REF_DIR, "%s_%s.so" % (name, tag))
    if not os.path.exists(so):
        with open(cpp, "w") as f:
            f.write(src)
        subprocess.run(["g++", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", "-w",
                        "-o", so, cpp], check=True)
    lib = ctypes.CDLL(so)
    lib.run.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int),
                        ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    lib.run.restype = None
    return lib.run


def run_plan(plan, text, name, passes=1, reverse0=False):
    """Execute ``plan`` (a reference Plan built under the stubs): its kernel's
    recorded ``set_args`` buffers are the host arrays the stubs captured, so the
    results land in those arrays in place."""
    run = compile_kernel(text, name)
    arrays = [buf.arr for buf in plan.kern.args]
    for arr in arrays:
        assert arr.flags.c_contiguous
    gsize = list(plan.gsize) + [1] * (3 - len(plan.gsize))
    lsize = list(plan.lsize) + [1] * (3 - len(plan.lsize)) if plan.lsize is not None else gsize
    G = (ctypes.c_int * 3)(*gsize)
    L = (ctypes.c_int * 3)(*lsize)

    def sweep(arrs, g, goff):
        ptrs = (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
        run(ptrs, g, L, int(reverse0))

    if passes == 1:
        sweep(arrays, G, None)
        return
    # one work-group at a time: scratch sweeps fill its local memory, the last sweep is real
    raise NotImplementedError("multi-pass execution is driven per group by run_plan_grouped")


def run_plan_grouped(plan, text, name, passes, group_axis=1):
    """Barrier kernels: run each work-group ``passes`` times, all but the last
    on scratch copies, so static local arrays are filled before they are used.
    Groups are the slices of ``group_axis`` (local size 1 along that axis)."""
    os.makedirs(REF_DIR, exist_ok=True)
    types = _signature(text, name)
    casts = ", ".join("(%s)a[%d]" % (t, i) for i, t in enumerate(types))
    driver = """
extern "C" void run_group(void** a, const int* gsize, const int* lsize, int axis, int group) {
  for (int d = 0; d < 3; ++d) { g_gsz[d] = gsize[d]; g_lsz[d] = lsize[d]; }
  int lo[3] = {0, 0, 0}, hi[3] = {gsize[0], gsize[1], gsize[2]};
  lo[axis] = group * lsize[axis]; hi[axis] = lo[axis] + lsize[axis];
  for (int z = lo[2]; z < hi[2]; ++z) for (int y = lo[1]; y < hi[1]; ++y)
    for (int x = lo[0]; x < hi[0]; ++x) {
      g_gid[0] = x; g_gid[1] = y; g_gid[2] = z;
      %s(%s);
    }
}
""" % (name, casts)
    src = SHIM + text + driver
    tag = hashlib.sha1(src.encode()).hexdigest()[:12]
    cpp = os.path.join(REF_DIR, "%s_g_%s.cpp" % (name, tag))
    so = os.path.join(REF_DIR, "%s_g_%s.so" % (name, tag))
    if not os.path.exists(so):
        with open(cpp, "w") as f:
            f.write(src)
        subprocess.run(["g++", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", "-w",
                        "-o", so, cpp], check=True)
    lib = ctypes.CDLL(so)
    lib.run_group.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int),
                              ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int]
    lib.run_group.restype = None
    arrays = [buf.arr for buf in plan.kern.args]
    gsize = list(plan.gsize) + [1] * (3 - len(plan.gsize))
    lsize = list(plan.lsize) + [1] * (3 - len(plan.lsize))
    G = (ctypes.c_int * 3)(*gsize)
    L = (ctypes.c_int * 3)(*lsize)
    n_groups = gsize[group_axis] // lsize[group_axis]
    for grp in range(n_groups):
        for p in range(passes):
            arrs = arrays if p == passes - 1 else [np.array(a) for a in arrays]
            ptrs = (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
            lib.run_group(ptrs, G, L, group_axis, grp)
