"""Small host-side helpers shared by the planning code.

Mirrors the helper surface of the reference's ``nengo_ocl/utils.py:16-90``
(``round_up``, ``stable_unique``, ``split``, ``equal_strides`` ...) without
its pyopencl / nengo imports.
"""

import numpy as np


def is_iterable(obj):
    """True for lists/tuples/ranges and ndarrays with ndim > 0 (not scalars)."""
    if isinstance(obj, np.ndarray):
        return obj.ndim > 0
    if isinstance(obj, (str, bytes)):
        return False
    try:
        iter(obj)
    except TypeError:
        return False
    return True


def is_number(obj):
    return isinstance(obj, (int, float, np.integer, np.floating)) and not isinstance(
        obj, bool
    )


def as_ascii(s):
    if isinstance(s, bytes):
        return s.decode("ascii")
    return s if isinstance(s, str) else str(s)


def round_up(x, n):
    """Smallest multiple of ``n`` that is >= ``x`` (reference utils.py:50-51)."""
    return int(np.ceil(float(x) / n)) * n


def round_up_power_of_2(x):
    if abs(x) < 1:
        return 1
    return int(np.sign(x)) * 2 ** int(np.ceil(np.log2(abs(x))))


def equal_strides(strides1, strides2, shape):
    """Strides agree on every axis whose extent is not 1."""
    if not len(strides1) == len(strides2) == len(shape):
        return False
    return all(n == 1 or a == b for n, a, b in zip(shape, strides1, strides2))


def indent(text, n):
    pad = " " * n
    return "\n".join(pad + line for line in text.split("\n"))


def nonelist(*args):
    return [a for a in args if a is not None]


def split(iterable, criterion):
    """Partition into (matching, not matching), order preserved."""
    yes, no = [], []
    for x in iterable:
        (yes if criterion(x) else no).append(x)
    return yes, no


def stable_unique(seq):
    seen = set()
    out = []
    for x in seq:
        if x not in seen:
            seen.add(x)
            out.append(x)
    return out


def groupby(objects, key):
    """Group ``objects`` by ``key(obj)`` using ``==``; first-seen key order.

    Stand-in for ``nengo.utils.stdlib.groupby`` used at
    ``nengo_ocl/simulator.py:895,1036,1161``.
    """
    keys, groups = [], []
    for obj in objects:
        k = key(obj)
        for i, k2 in enumerate(keys):
            if k2 == k:
                groups[i].append(obj)
                break
        else:
            keys.append(k)
            groups.append([obj])
    return list(zip(keys, groups))


def get_closures(f):
    return dict(zip(f.__code__.co_freevars, (c.cell_contents for c in f.__closure__)))
