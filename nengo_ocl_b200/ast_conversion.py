"""Translate simple Python functions (node outputs, connection functions) into
postfix programs for the device interpreter (csrc/nb2_direct.cu).

Role of the reference's ``nengo_ocl/ast_conversion.py`` (``OclFunction``
:845-931 and the function tables :62-262): there the Python AST becomes OpenCL
C text compiled per function; here it becomes a list of ``(opcode, operand)``
pairs evaluated by one generic kernel, so no run-time compiler is involved.

Supported: arithmetic, comparisons, boolean and/or/not, conditional
expressions, unary minus, constants from closures / globals / default
arguments, indexing of the vector argument with constant indices, whole-vector
arithmetic with broadcasting, tuple / list / ``np.array([...])`` results, and
every entry of the reference's three function tables (``direct_funcs``,
``indirect_funcs``, ``vector_funcs`` / ``vector_attr``, ast_conversion.py:62-262):
the elementary functions in ``FUNCS``, the composite ones in ``COMPOSITES``
(degrees, hypot, logaddexp, ...) and the reductions over a vector in
``REDUCTIONS`` (sum, prod, mean, max, min, all, any, len; also as methods,
``x.sum()``), expanded like the reference expands them.  Anything else raises
``NotImplementedError`` (the simulator then falls back to running the function
on the host, depending on ``if_python_code``).
"""

import ast
import inspect
import math
import os
import re
import textwrap

import numpy as np

OUTPUT_NAME = "OUTPUT__"


def _load_opcodes():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "nb2_direct_ops.h")
    with open(path) as f:
        text = f.read()
    ops = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define NB2_OP_(\w+) (\d+)", text)}
    return ops, int(re.search(r"#define NB2_DIRECT_STACK (\d+)", text).group(1))


OPS, MAX_STACK = _load_opcodes()

BINOPS = {ast.Add: "ADD", ast.Sub: "SUB", ast.Mult: "MUL", ast.Div: "DIV", ast.Pow: "POW", ast.Mod: "MOD"}
CMPOPS = {ast.Lt: "LT", ast.LtE: "LE", ast.Gt: "GT", ast.GtE: "GE", ast.Eq: "EQ", ast.NotEq: "NE"}
# python / numpy function name -> (opcode, arity)
FUNCS = {
    "sin": ("SIN", 1), "cos": ("COS", 1), "tan": ("TAN", 1), "arcsin": ("ASIN", 1), "asin": ("ASIN", 1),
    "arccos": ("ACOS", 1), "acos": ("ACOS", 1), "arctan": ("ATAN", 1), "atan": ("ATAN", 1),
    "sinh": ("SINH", 1), "cosh": ("COSH", 1), "tanh": ("TANH", 1), "exp": ("EXP", 1), "expm1": ("EXPM1", 1),
    "log": ("LOG", 1), "log2": ("LOG2", 1), "log10": ("LOG10", 1), "log1p": ("LOG1P", 1), "sqrt": ("SQRT", 1),
    "abs": ("ABS", 1), "absolute": ("ABS", 1), "fabs": ("ABS", 1), "floor": ("FLOOR", 1), "ceil": ("CEIL", 1),
    "round": ("ROUND", 1), "rint": ("ROUND", 1), "sign": ("SIGN", 1), "square": (None, 1), "negative": ("NEG", 1),
    "arctan2": ("ATAN2", 2), "atan2": ("ATAN2", 2), "power": ("POW", 2), "pow": ("POW", 2),
    "minimum": ("MIN", 2), "maximum": ("MAX", 2), "min": ("MIN", 2), "max": ("MAX", 2), "fmod": ("MOD", 2),
    "where": ("SELECT", 3),
    "arccosh": ("ACOSH", 1), "acosh": ("ACOSH", 1), "arcsinh": ("ASINH", 1), "asinh": ("ASINH", 1),
    "arctanh": ("ATANH", 1), "atanh": ("ATANH", 1), "exp2": ("EXP2", 1), "isinf": ("ISINF", 1),
    "isnan": ("ISNAN", 1), "isfinite": ("ISFINITE", 1), "erf": ("ERF", 1), "erfc": ("ERFC", 1),
    "lgamma": ("LGAMMA", 1), "fmax": ("MAX", 2), "fmin": ("MIN", 2), "mod": ("FMOD", 2),
    "add": ("ADD", 2), "subtract": ("SUB", 2), "multiply": ("MUL", 2), "divide": ("DIV", 2),
    "true_divide": ("DIV", 2), "equal": ("EQ", 2), "not_equal": ("NE", 2), "greater": ("GT", 2),
    "greater_equal": ("GE", 2), "less": ("LT", 2), "less_equal": ("LE", 2), "remainder": ("MOD", 2),
}
FUNCS["fmod"] = ("FMOD", 2)  # C fmod: the result has the sign of the dividend (math.fmod, np.fmod)

# functions the reference expands into expressions (indirect_funcs, ast_conversion.py:131-195):
# name -> (arity, builder(translator, *argument values))
COMPOSITES = {
    "degrees": (1, lambda t, x: t._apply("MUL", x, t._const(180.0 / math.pi))),
    "rad2deg": (1, lambda t, x: t._apply("MUL", x, t._const(180.0 / math.pi))),
    "radians": (1, lambda t, x: t._apply("MUL", x, t._const(math.pi / 180.0))),
    "deg2rad": (1, lambda t, x: t._apply("MUL", x, t._const(math.pi / 180.0))),
    "hypot": (2, lambda t, x, y: t._apply("SQRT", t._apply("ADD", t._apply("MUL", x, x), t._apply("MUL", y, y)))),
    "ldexp": (2, lambda t, x, y: t._apply("MUL", x, t._apply("POW", t._const(2.0), y))),
    "reciprocal": (1, lambda t, x: t._apply("DIV", t._const(1.0), x)),
    "signbit": (1, lambda t, x: t._apply("LT", x, t._const(0.0))),
    "floor_divide": (2, lambda t, x, y: t._apply("FLOOR", t._apply("DIV", x, y))),
    "logaddexp": (2, lambda t, x, y: t._apply("LOG", t._apply("ADD", t._apply("EXP", x), t._apply("EXP", y)))),
    "logaddexp2": (2, lambda t, x, y: t._apply("LOG2", t._apply("ADD", t._apply("EXP2", x), t._apply("EXP2", y)))),
    "gamma": (1, lambda t, x: t._apply("EXP", t._apply("LGAMMA", x))),
}


def _fold(op):
    """x0 op (x1 op (x2 op ...)): the right-nested expansion of the reference (_recurse_binexp)."""
    def build(t, elems):
        out = [elems[-1]]
        for e in reversed(elems[:-1]):
            out = t._apply(op, [e], out)
        return out
    return build


# reductions over the elements of one vector argument (vector_funcs / vector_attr, :198-262)
REDUCTIONS = {
    "sum": _fold("ADD"), "prod": _fold("MUL"), "max": _fold("MAX"), "min": _fold("MIN"), "amax": _fold("MAX"),
    "amin": _fold("MIN"), "all": _fold("AND"), "any": _fold("OR"),
    "len": lambda t, elems: t._const(len(elems)),
    "mean": lambda t, elems: t._apply("DIV", _fold("ADD")(t, elems), t._const(len(elems))),
}


class DeviceFunction:
    """A translated function: ``program`` = [(opcode, operand)], ``constants``."""

    def __init__(self, fn, in_dims=None, out_dim=None):
        self.fn = fn
        self.in_dims = list(in_dims or [])
        self.out_dim = out_dim
        self.translator = _Translator(fn, self.in_dims)
        self.program, self.constants, n_out = self.translator.translate()
        # the interpreter evaluates on a fixed-size stack: a program that needs more is not run
        # on the device (the caller then evaluates the function on the host)
        self.max_depth = stack_depth(self.program)
        if self.max_depth > MAX_STACK:
            raise NotImplementedError("expression needs %d stack slots, the device interpreter has %d"
                                      % (self.max_depth, MAX_STACK))
        if out_dim is not None and n_out != out_dim:
            raise NotImplementedError("function returns %d values, expected %d" % (n_out, out_dim))
        self.out_dim = n_out

    # names kept for signature parity with the reference's OclFunction
    @property
    def code(self):
        return self

    @property
    def init(self):
        return ""


OclFunction = DeviceFunction


class _Translator(ast.NodeVisitor):
    MAX_VECTOR_LENGTH = 25  # as in the reference (ast_conversion.py:492)

    def __init__(self, fn, in_dims):
        self.fn = fn
        self.in_dims = in_dims
        self.constants = []
        if isinstance(fn, np.ufunc):
            self.arg_names = ["x%d" % i for i in range(len(in_dims))]
            self.tree = None
            self.namespace = {}
            return
        node = self._lambda_from_file(fn) if getattr(fn, "__name__", "") == "<lambda>" else None
        if node is not None:
            tree = ast.Module(body=[ast.Expr(node)], type_ignores=[])
            self.tree, self.func_node = tree, node
        else:
            src = textwrap.dedent(inspect.getsource(fn)).strip()
            try:
                tree = ast.parse(src)
            except SyntaxError:
                tree = self._parse_embedded_lambda(src)
            self.tree = tree
            self.func_node = self._find_function(tree, fn)
        args = self.func_node.args
        self.arg_names = [a.arg for a in args.args]
        if inspect.ismethod(fn):
            self.arg_names = self.arg_names[1:]
        self.namespace = dict(getattr(fn, "__globals__", {}))
        if getattr(fn, "__closure__", None):
            self.namespace.update(zip(fn.__code__.co_freevars, (c.cell_contents for c in fn.__closure__)))
        defaults = fn.__defaults__ or ()
        for name, value in zip(self.arg_names[len(self.arg_names) - len(defaults):], defaults):
            self.namespace[name] = value
        self.arg_names = self.arg_names[: len(in_dims)]
        self.locals = {}

    @staticmethod
    def _lambda_from_file(fn):
        """The ``ast.Lambda`` of ``fn`` located in its source file by line number; several lambdas
        on one line (a table of functions) are told apart by their compiled code."""
        try:
            path = inspect.getsourcefile(fn)
            with open(path) as f:
                tree = ast.parse(f.read())
        except (TypeError, OSError, SyntaxError):
            return None
        line = fn.__code__.co_firstlineno
        found = [n for n in ast.walk(tree) if isinstance(n, ast.Lambda) and n.lineno == line]
        if len(found) == 1:
            return found[0]
        # the code object records the columns of its instructions: the lambda whose body spans them
        cols = [(c0, c1) for l0, _, c0, c1 in fn.__code__.co_positions()
                if l0 == line and c0 is not None and c1 is not None and c1 > c0]
        if cols:
            lo, hi = min(c for c, _ in cols), max(c for _, c in cols)
            inside = [n for n in found if n.body.lineno == line and n.body.col_offset <= lo
                      and (n.body.end_lineno > line or hi <= n.body.end_col_offset)]
            if len(inside) == 1:
                return inside[0]
        return None

    @staticmethod
    def _parse_embedded_lambda(src):
        """The source line of a lambda may be a fragment of a larger statement:
        cut at 'lambda' and drop trailing characters until it parses."""
        if "lambda" not in src:
            raise NotImplementedError("unparsable function source")
        sub = src[src.index("lambda"):]
        for end in range(len(sub), 6, -1):
            try:
                return ast.parse(sub[:end].strip())
            except SyntaxError:
                continue
        raise NotImplementedError("unparsable lambda source")

    @staticmethod
    def _find_function(tree, fn):
        name = getattr(fn, "__name__", None)
        lambdas = [n for n in ast.walk(tree) if isinstance(n, ast.Lambda)]
        if name == "<lambda>":
            if len(lambdas) != 1:
                raise NotImplementedError("cannot isolate the lambda in its source line")
            return lambdas[0]
        for n in ast.walk(tree):
            if isinstance(n, ast.FunctionDef) and n.name == name:
                return n
        raise NotImplementedError("function source not found")

    # ---- values are lists of token lists (one per vector element) -------------
    def _const(self, value):
        value = float(value)
        if value not in self.constants:
            self.constants.append(value)
        return [[(OPS["CONST"], self.constants.index(value))]]

    def _from_python(self, value):
        arr = np.asarray(value, dtype=np.float64)
        if arr.ndim == 0:
            return self._const(arr)
        if arr.ndim == 1 and arr.size <= self.MAX_VECTOR_LENGTH:
            return [self._const(v)[0] for v in arr]
        raise NotImplementedError("only scalars and short vectors can be embedded")

    @staticmethod
    def _broadcast(*values):
        n = max(len(v) for v in values)
        out = []
        for v in values:
            if len(v) not in (1, n):
                raise NotImplementedError("shape mismatch in vector expression")
            out.append(v * n if len(v) == 1 else v)
        return out

    def _apply(self, op, *values):
        values = self._broadcast(*values)
        return [sum((list(v[i]) for v in values), []) + [(OPS[op], 0)] for i in range(len(values[0]))]

    def translate(self):
        if self.tree is None and isinstance(self.fn, np.ufunc):
            name = self.fn.__name__
            if name not in FUNCS:
                raise NotImplementedError(name)
            args = [self._arg_value(i) for i in range(len(self.in_dims))]
            result = self._call(name, args)
        elif isinstance(self.func_node, ast.Lambda):
            result = self.visit(self.func_node.body)
        else:
            result = None
            for stmt in self.func_node.body:
                if isinstance(stmt, ast.Return):
                    result = self.visit(stmt.value)
                    break
                if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name):
                    self.locals[stmt.targets[0].id] = self.visit(stmt.value)
                elif isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
                    continue  # docstring
                else:
                    raise NotImplementedError("statement %s" % type(stmt).__name__)
            if result is None:
                raise NotImplementedError("function has no return value")
        program = []
        for i, tokens in enumerate(result):
            program.extend(tokens)
            program.append((OPS["STORE"], i))
        return program, self.constants, len(result)

    def _arg_value(self, index):
        op = OPS["IN0"] if index == 0 else OPS["IN1"]
        return [[(op, j)] for j in range(self.in_dims[index])]

    def _call(self, name, args):
        # a reduction takes one vector (max / min with several scalars are the binary functions)
        if name in REDUCTIONS and len(args) == 1 and (len(args[0]) > 1 or name not in FUNCS):
            out = REDUCTIONS[name](self, args[0])
            if name in ("all", "any"):  # truth value of the (possibly single) element
                out = self._apply("NE", out, self._const(0.0))
            return out
        if name in COMPOSITES:
            arity, build = COMPOSITES[name]
            if len(args) != arity:
                raise NotImplementedError("%s with %d arguments" % (name, len(args)))
            return build(self, *args)
        if name not in FUNCS:
            raise NotImplementedError("function %r" % name)
        op, arity = FUNCS[name]
        if len(args) != arity:
            raise NotImplementedError("%s with %d arguments" % (name, len(args)))
        if name == "square":
            return self._apply("MUL", args[0], args[0])
        return self._apply(op, *args)

    # ---- visitors ---------------------------------------------------------------
    def generic_visit(self, node):
        raise NotImplementedError("expression %s" % type(node).__name__)

    def visit_Constant(self, node):
        if isinstance(node.value, (int, float, bool)):
            return self._const(node.value)
        raise NotImplementedError("constant %r" % (node.value,))

    def visit_Name(self, node):
        if node.id in self.locals:
            return self.locals[node.id]
        if node.id in self.arg_names:
            return self._arg_value(self.arg_names.index(node.id))
        if node.id in self.namespace:
            return self._from_python(self.namespace[node.id])
        if node.id in ("True", "False"):
            return self._const(node.id == "True")
        raise NotImplementedError("name %r" % node.id)

    def visit_Attribute(self, node):
        # constants such as np.pi / math.e
        if isinstance(node.value, ast.Name) and node.value.id in self.namespace:
            value = getattr(self.namespace[node.value.id], node.attr, None)
            if isinstance(value, (int, float)):
                return self._const(value)
        raise NotImplementedError("attribute %s" % node.attr)

    def visit_UnaryOp(self, node):
        v = self.visit(node.operand)
        if isinstance(node.op, ast.USub):
            return self._apply("NEG", v)
        if isinstance(node.op, ast.UAdd):
            return v
        if isinstance(node.op, ast.Not):
            return self._apply("NOT", v)
        raise NotImplementedError("unary %s" % type(node.op).__name__)

    def visit_BinOp(self, node):
        if type(node.op) not in BINOPS:
            raise NotImplementedError("operator %s" % type(node.op).__name__)
        left, right = self.visit(node.left), self.visit(node.right)
        if isinstance(node.op, ast.Pow) and isinstance(node.right, ast.Constant) and node.right.value == 2:
            return self._apply("MUL", left, left)
        return self._apply(BINOPS[type(node.op)], left, right)

    def visit_Compare(self, node):
        if len(node.ops) != 1 or type(node.ops[0]) not in CMPOPS:
            raise NotImplementedError("comparison")
        return self._apply(CMPOPS[type(node.ops[0])], self.visit(node.left), self.visit(node.comparators[0]))

    def visit_BoolOp(self, node):
        op = "AND" if isinstance(node.op, ast.And) else "OR"
        out = self.visit(node.values[0])
        for v in node.values[1:]:
            out = self._apply(op, out, self.visit(v))
        return out

    def visit_IfExp(self, node):
        return self._apply("SELECT", self.visit(node.test), self.visit(node.body), self.visit(node.orelse))

    def visit_Subscript(self, node):
        base = self.visit(node.value)
        idx = node.slice
        if isinstance(idx, ast.Constant) and isinstance(idx.value, int):
            return [base[idx.value]]
        if isinstance(idx, ast.UnaryOp) and isinstance(idx.op, ast.USub) and isinstance(idx.operand, ast.Constant):
            return [base[-idx.operand.value]]
        if isinstance(idx, ast.Slice):
            get = lambda n: None if n is None else ast.literal_eval(n)
            return base[slice(get(idx.lower), get(idx.upper), get(idx.step))]
        raise NotImplementedError("only constant indices are supported")

    def _sequence(self, elts):
        out = []
        for e in elts:
            out.extend(self.visit(e))
        return out

    def visit_Tuple(self, node):
        return self._sequence(node.elts)

    visit_List = visit_Tuple

    def visit_Call(self, node):
        if node.keywords:
            raise NotImplementedError("keyword arguments")
        fname = node.func.attr if isinstance(node.func, ast.Attribute) else getattr(node.func, "id", None)
        if fname in ("array", "asarray", "float", "float32", "float64"):
            return self.visit(node.args[0])
        # a reduction as a method of a vector value: x.sum(), (x * x).mean()
        if (isinstance(node.func, ast.Attribute) and fname in REDUCTIONS and not node.args
                and not (isinstance(node.func.value, ast.Name) and node.func.value.id in self.namespace
                         and node.func.value.id not in self.arg_names and node.func.value.id not in self.locals)):
            return self._call(fname, [self.visit(node.func.value)])
        args = [self.visit(a) for a in node.args]
        return self._call(fname, args)


_PUSHES = {OPS["CONST"], OPS["IN0"], OPS["IN1"]}
_UNARY = {OPS[name] for name in ("NEG", "NOT", "SIN", "COS", "TAN", "ASIN", "ACOS", "ATAN", "SINH", "COSH", "TANH",
                                 "EXP", "EXPM1", "LOG", "LOG2", "LOG10", "LOG1P", "SQRT", "ABS", "FLOOR", "CEIL",
                                 "ROUND", "SIGN", "ACOSH", "ASINH", "ATANH", "EXP2", "ISINF", "ISNAN", "ISFINITE",
                                 "ERF", "ERFC", "LGAMMA")}


def stack_depth(program):
    """Largest number of values a postfix program holds on the evaluation stack."""
    depth = deepest = 0
    for op, _ in program:
        if op in _PUSHES:
            depth += 1
        elif op == OPS["SELECT"]:
            depth -= 2
        elif op == OPS["STORE"] or op not in _UNARY:
            depth -= 1  # a store pops one value, a binary operator replaces two by one
        deepest = max(deepest, depth)
    assert depth == 0, "unbalanced program"
    return deepest


def is_translatable(fn, in_dims, out_dim=None):
    try:
        DeviceFunction(fn, in_dims, out_dim)
        return True
    except (NotImplementedError, OSError, TypeError, SyntaxError, IndexError, ValueError):
        return False


__all__ = ["DeviceFunction", "OclFunction", "OUTPUT_NAME", "OPS", "FUNCS", "MAX_STACK", "stack_depth",
           "is_translatable", "math"]
