"""Stand-ins for pyopencl / mako / nengo so the reference's planning modules
can be imported from their source tree and run on the host.

Used only by ``make_golden.py`` (fixture generation, run where the reference
source tree is mounted).  ``to_device`` records every uploaded host array and
``Program`` records every rendered kernel text, which is how index tables and
kernel sources are captured.  The template class implements the small subset
of Mako the reference's kernel strings use.
"""

import importlib.util
import os
import re
import sys
import types

import numpy as np

CAPTURE = []  # host arrays handed to to_device, in call order
PROGRAMS = []  # rendered kernel sources, in build order


class FakeBuf:
    def __init__(self, arr):
        self.arr = arr


class FakeArray:
    def __init__(self, queue, shape=None, dtype=None, strides=None, data=None, offset=0, _arr=None):
        self.queue = queue
        if _arr is not None:
            self._arr = _arr
            self.shape, self.dtype, self.offset = _arr.shape, _arr.dtype, 0
            self.data = FakeBuf(_arr)
            self.base_data = self.data
            self.strides = _arr.strides
        else:
            self.shape, self.dtype, self.strides = tuple(shape), np.dtype(dtype), strides
            self.data = self.base_data = data
            self.offset = offset

    @property
    def nbytes(self):
        return int(np.prod(self.shape)) * self.dtype.itemsize

    @property
    def size(self):
        return int(np.prod(self.shape))

    def __len__(self):
        return self.shape[0]

    def get(self):
        return self._arr.copy()

    def fill(self, v):
        self._arr[...] = v

    def set(self, a):
        self._arr[...] = a


def to_device(queue, arr):
    arr = np.array(arr)
    CAPTURE.append(arr)
    return FakeArray(queue, _arr=arr)


class FakeKernel:
    def __init__(self, name):
        self.name = name
        self.args = None

    def set_args(self, *a):
        self.args = a


class FakeBuilt:
    def __init__(self, text):
        self.text = text

    def __getattr__(self, name):
        return FakeKernel(name)


class FakeProgram:
    def __init__(self, ctx, text):
        self.text = text
        PROGRAMS.append(text)

    def build(self, **kwargs):
        return FakeBuilt(self.text)


class Device:
    max_work_group_size = 1024
    global_mem_size = 180 * 2 ** 30
    local_mem_size = 48 * 1024


class Queue:
    device = Device()
    context = object()

    def finish(self):
        pass


class Template:
    """``${expr}``, ``% if/elif/else/endif``, ``% for/endfor``, backslash-newline."""

    def __init__(self, text, output_encoding=None):
        self.text = text

    def render(self, **ctx):
        text = self.text.replace("\\\n", "")
        src, depth = ["def __render(__out):"], 1
        for line in text.split("\n"):
            mt = re.match(r"^\s*%\s*(.*)$", line)
            if mt and not line.lstrip().startswith("%%"):
                stmt = re.sub(r"\s+#.*$", "", mt.group(1)).strip()
                kw = stmt.split()[0].rstrip(":")
                if kw in ("endif", "endfor"):
                    depth -= 1
                elif kw in ("else", "elif"):
                    src.append("    " * (depth - 1) + stmt)
                else:
                    src.append("    " * depth + stmt)
                    depth += 1
                    src.append("    " * depth + "pass")
                continue
            parts = re.split(r"\$\{(.*?)\}", line)
            pieces = [repr(p) if i % 2 == 0 else "str(%s)" % p for i, p in enumerate(parts)]
            src.append("    " * depth + "__out.append(%s + '\\n')" % " + ".join(pieces))
        ns = dict(ctx)
        exec("\n".join(src), ns)
        out = []
        ns["__render"](out)
        return "".join(out)


def install(reference_root):
    """Register the fake modules and load the reference's modules by path."""
    cl = types.ModuleType("pyopencl")
    cl.Program = FakeProgram
    cl.command_queue_properties = types.SimpleNamespace(PROFILING_ENABLE=1)
    cl.tools = types.SimpleNamespace(
        dtype_to_ctype=lambda d: {"float32": "float", "int32": "int"}[np.dtype(d).name])
    cl.enqueue_nd_range_kernel = lambda *a, **k: None
    cl.enqueue_copy = lambda *a, **k: None
    cla = types.ModuleType("pyopencl.array")
    cla.Array = FakeArray
    cla.to_device = to_device
    cl.array = cla
    mako = types.ModuleType("mako")
    mt = types.ModuleType("mako.template")
    mt.Template = Template
    mako.template = mt
    nengo = types.ModuleType("nengo")
    nu = types.ModuleType("nengo.utils")
    nun = types.ModuleType("nengo.utils.numpy")

    def is_iterable(x):
        if isinstance(x, np.ndarray):
            return x.ndim > 0
        try:
            iter(x)
            return True
        except TypeError:
            return False

    nun.is_iterable = is_iterable
    nun.is_number = lambda x: isinstance(x, (int, float, np.number))
    import scipy.sparse as sp

    nun.scipy_sparse = sp
    nd = types.ModuleType("nengo.dists")
    nd.Uniform = type("Uniform", (), {})
    nd.Gaussian = type("Gaussian", (), {})
    nengo.dists = nd
    pkg = types.ModuleType("nengo_ocl")
    pkg.__path__ = [os.path.join(reference_root, "nengo_ocl")]
    sys.modules.update({"pyopencl": cl, "pyopencl.array": cla, "mako": mako, "mako.template": mt,
                        "nengo": nengo, "nengo.utils": nu, "nengo.utils.numpy": nun, "nengo.dists": nd,
                        "nengo_ocl": pkg})
    mods = {}
    for name in ("utils", "raggedarray", "clraggedarray", "plan", "ast_conversion", "clra_gemv",
                 "clra_nonlinearities"):
        path = os.path.join(reference_root, "nengo_ocl", name + ".py")
        spec = importlib.util.spec_from_file_location("nengo_ocl." + name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["nengo_ocl." + name] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods
