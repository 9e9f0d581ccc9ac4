"""Every entry of the reference's function tables through the device path.

Follows nengo_ocl/tests/test_ast_conversion.py:160-328: each function of
``direct_funcs`` / ``indirect_funcs`` / ``vector_funcs`` (ast_conversion.py:62-262)
is used in a node function that must be translated (``if_python_code="error"``:
no host fallback allowed), run for a few steps, and compared with the Python
function itself.  The device interpreter evaluates in double precision and
rounds when it stores, as Python does before the cast to float32, so the
tolerance is float32 round-off (2e-7 relative, the reference's own bound is an
absolute 2e-7 on O(1) values)."""

import math

import numpy as np
import pytest

from nengo_ocl_b200 import model as m
from nengo_ocl_b200.simulator import Simulator

pytestmark = pytest.mark.gpu


def run_node(fn, x_dim, steps=6):
    """``out = fn(x)`` with ``x = sin/cos ramps of t`` produced by a first (translated) node."""
    mdl = m.Model(dt=0.001)
    src = m.Signal(np.zeros(x_dim), name="<Node src>.out")
    freqs = np.arange(1, x_dim + 1)
    if x_dim == 1:
        mdl.add_op(m.SimPyFunc(src, lambda t: 0.9 * np.sin(400 * t + 0.3), mdl.time, None))
    elif x_dim == 2:
        mdl.add_op(m.SimPyFunc(src, lambda t: [0.9 * np.sin(400 * t + 0.3), 0.8 * np.cos(300 * t)], mdl.time, None))
    else:
        mdl.add_op(m.SimPyFunc(src, lambda t: [0.9 * np.sin(400 * t + 0.3), 0.8 * np.cos(300 * t),
                                               0.7 * np.sin(500 * t + 1.0)], mdl.time, None))
    probe_in = np.atleast_1d(fn(np.full(x_dim, 0.5)))
    out = m.Signal(np.zeros(probe_in.size), name="<Node f>.out")
    mdl.add_op(m.SimPyFunc(out, fn, None, src))
    p_src, p_out = mdl.add_probe(src), mdl.add_probe(out)
    with Simulator(None, model=mdl, if_python_code="error") as sim:
        assert all(type(p).__name__ != "PythonPlan" for p in sim._plans)
        sim.run_steps(steps)
        xs, ys = sim.data[p_src], sim.data[p_out]
    # the second node reads the first node's output of the same step
    want = np.array([np.atleast_1d(np.asarray(fn(x.astype(np.float64)), dtype=np.float64)) for x in xs])
    return xs, ys, want.astype(np.float32)


# name -> (function of a vector x with |x_i| < 1, input dimension)
UNARY = {
    "abs": lambda x: abs(x[0]), "math.acos": lambda x: math.acos(x[0]), "math.acosh": lambda x: math.acosh(x[0] + 2),
    "math.asin": lambda x: math.asin(x[0]), "math.asinh": lambda x: math.asinh(x[0]),
    "math.atan": lambda x: math.atan(x[0]), "math.atanh": lambda x: math.atanh(x[0]),
    "math.ceil": lambda x: math.ceil(3 * x[0]), "math.cos": lambda x: math.cos(x[0]),
    "math.cosh": lambda x: math.cosh(x[0]), "math.exp": lambda x: math.exp(x[0]), "math.fabs": lambda x: math.fabs(x[0]),
    "math.floor": lambda x: math.floor(3 * x[0]), "math.isinf": lambda x: math.isinf(x[0]),
    "math.isnan": lambda x: math.isnan(x[0]), "math.log": lambda x: math.log(x[0] + 2),
    "math.log10": lambda x: math.log10(x[0] + 2), "math.log1p": lambda x: math.log1p(x[0]),
    "math.sin": lambda x: math.sin(x[0]), "math.sinh": lambda x: math.sinh(x[0]), "math.sqrt": lambda x: math.sqrt(x[0] + 1),
    "math.tan": lambda x: math.tan(x[0]), "math.tanh": lambda x: math.tanh(x[0]), "math.expm1": lambda x: math.expm1(x[0]),
    "math.erf": lambda x: math.erf(x[0]), "math.erfc": lambda x: math.erfc(x[0]),
    "math.lgamma": lambda x: math.lgamma(x[0] + 2), "math.gamma": lambda x: math.gamma(x[0] + 2),
    "math.degrees": lambda x: math.degrees(x[0]), "math.radians": lambda x: math.radians(x[0]),
    "np.abs": lambda x: np.abs(x), "np.absolute": lambda x: np.absolute(x), "np.arccos": lambda x: np.arccos(x),
    "np.arccosh": lambda x: np.arccosh(x + 2), "np.arcsin": lambda x: np.arcsin(x), "np.arcsinh": lambda x: np.arcsinh(x),
    "np.arctan": lambda x: np.arctan(x), "np.arctanh": lambda x: np.arctanh(x), "np.ceil": lambda x: np.ceil(3 * x),
    "np.cos": lambda x: np.cos(x), "np.cosh": lambda x: np.cosh(x), "np.exp": lambda x: np.exp(x),
    "np.exp2": lambda x: np.exp2(x), "np.expm1": lambda x: np.expm1(x), "np.fabs": lambda x: np.fabs(x),
    "np.floor": lambda x: np.floor(3 * x), "np.isfinite": lambda x: np.isfinite(x), "np.isinf": lambda x: np.isinf(x),
    "np.isnan": lambda x: np.isnan(x), "np.log": lambda x: np.log(x + 2), "np.log10": lambda x: np.log10(x + 2),
    "np.log1p": lambda x: np.log1p(x), "np.log2": lambda x: np.log2(x + 2), "np.sin": lambda x: np.sin(x),
    "np.sinh": lambda x: np.sinh(x), "np.sqrt": lambda x: np.sqrt(x + 1), "np.tan": lambda x: np.tan(x),
    "np.tanh": lambda x: np.tanh(x), "np.deg2rad": lambda x: np.deg2rad(x), "np.degrees": lambda x: np.degrees(x),
    "np.rad2deg": lambda x: np.rad2deg(x), "np.radians": lambda x: np.radians(x), "np.negative": lambda x: np.negative(x),
    "np.reciprocal": lambda x: np.reciprocal(x + 2), "np.sign": lambda x: np.sign(x), "np.signbit": lambda x: np.signbit(x),
    "np.square": lambda x: np.square(x), "np.asarray": lambda x: np.asarray(x) * 2,
}
BINARY = {
    "math.atan2": lambda x: math.atan2(x[0], x[1]), "math.fmod": lambda x: math.fmod(x[0], 0.3 + abs(x[1])),
    "math.hypot": lambda x: math.hypot(x[0], x[1]), "math.ldexp": lambda x: math.ldexp(x[0], 3),
    "math.pow": lambda x: math.pow(x[0] + 2, x[1]), "np.add": lambda x: np.add(x[0], x[1]),
    "np.arctan2": lambda x: np.arctan2(x[0], x[1]), "np.divide": lambda x: np.divide(x[0], x[1] + 2),
    "np.equal": lambda x: np.equal(x[0], x[1]), "np.floor_divide": lambda x: np.floor_divide(x[0], 0.3 + abs(x[1])),
    "np.fmax": lambda x: np.fmax(x[0], x[1]), "np.fmin": lambda x: np.fmin(x[0], x[1]),
    "np.fmod": lambda x: np.fmod(x[0], 0.3 + abs(x[1])), "np.greater": lambda x: np.greater(x[0], x[1]),
    "np.greater_equal": lambda x: np.greater_equal(x[0], x[1]), "np.hypot": lambda x: np.hypot(x[0], x[1]),
    "np.less": lambda x: np.less(x[0], x[1]), "np.less_equal": lambda x: np.less_equal(x[0], x[1]),
    "np.logaddexp": lambda x: np.logaddexp(x[0], x[1]), "np.logaddexp2": lambda x: np.logaddexp2(x[0], x[1]),
    "np.maximum": lambda x: np.maximum(x[0], x[1]), "np.minimum": lambda x: np.minimum(x[0], x[1]),
    "np.multiply": lambda x: np.multiply(x[0], x[1]), "np.power": lambda x: np.power(x[0] + 2, x[1]),
    "np.remainder": lambda x: np.remainder(x[0], 0.3 + abs(x[1])), "np.subtract": lambda x: np.subtract(x[0], x[1]),
}
VECTOR = {
    "all": lambda x: all(x), "any": lambda x: any(x), "len": lambda x: len(x), "max": lambda x: max(x),
    "min": lambda x: min(x), "sum": lambda x: sum(x), "np.all": lambda x: np.all(x), "np.any": lambda x: np.any(x),
    "np.max": lambda x: np.max(x), "np.min": lambda x: np.min(x), "np.mean": lambda x: np.mean(x),
    "np.prod": lambda x: np.prod(x), "np.sum": lambda x: np.sum(x), ".all": lambda x: (x > -2).all(),
    ".any": lambda x: (x > 0.5).any(), ".max": lambda x: x.max(), ".min": lambda x: x.min(), ".mean": lambda x: x.mean(),
    ".prod": lambda x: x.prod(), ".sum": lambda x: (x * x).sum(),
}
CASES = ([(k, f, 1) for k, f in UNARY.items()] + [(k, f, 2) for k, f in BINARY.items()]
         + [(k, f, 3) for k, f in VECTOR.items()])


@pytest.mark.parametrize("name,fn,dim", CASES, ids=[c[0] for c in CASES])
def test_function_table_entry_on_device(name, fn, dim):
    xs, got, want = run_node(fn, dim)
    assert np.abs(xs).max() > 0.1
    assert got.shape == want.shape
    assert np.allclose(got, want, rtol=2e-7, atol=2e-7), (name, got[:2], want[:2])


def test_untranslatable_function_falls_back_to_the_host():
    """What the translator does not take (loops, side effects, library calls outside the
    tables) raises NotImplementedError inside the planner and runs as a host plan."""
    from nengo_ocl_b200.ast_conversion import is_translatable

    for fn, dims in [(lambda x: sorted(x), [3]), (lambda x: np.linalg.norm(x), [3]),
                     (lambda x: [v for v in x], [2]), (lambda t: np.random.rand(), [1])]:
        assert not is_translatable(fn, dims)
    mdl = m.Model(dt=0.001)
    out = m.Signal(np.zeros(1), name="<Node host>.out")
    mdl.add_op(m.SimPyFunc(out, lambda t: np.linalg.norm([t, 1.0]), mdl.time, None))
    with pytest.raises(RuntimeError):
        Simulator(None, model=mdl, if_python_code="error")
    with Simulator(None, model=mdl) as sim:
        assert any(type(p).__name__ == "PythonPlan" for p in sim._plans)
        sim.run_steps(3)
        assert np.allclose(sim.signals[out], np.sqrt(0.003 ** 2 + 1), rtol=1e-6)
