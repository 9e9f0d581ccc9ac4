"""Operator merging and simplification applied before planning.

Planning-surface equivalents of the reference's ``nengo_ocl/operators.py``:
``MultiDotInc`` (:19-194) with ``convert_to`` / ``compress`` / ``get_views``,
``signal_io_dicts`` (:197-228), ``remove_unmodified_resets`` (:231-272),
``remove_zero_incs`` (:275-330), ``simplify_operators`` and the mutable
``simplifications`` list (:333-350).
"""

import numpy as np

from nengo_ocl_b200.model import Copy, DotInc, ElementwiseInc, Operator, Reset, Signal


class MultiDotInc(Operator):
    r"""``y <- gamma + beta * y_in + \sum_i dot(A_i, x_i)``"""

    def __init__(self, Y, Y_in, beta, gamma, tag=None):
        Operator.__init__(self, tag=tag)
        assert Y.ndim == 1
        if Y.shape != Y_in.shape:
            raise TypeError()
        self.Y = Y
        self.Y_in = Y_in
        if isinstance(beta, Signal):
            if beta.shape != Y.shape:
                raise NotImplementedError("", (beta.shape, Y.shape))
            self._float_beta, self._signal_beta = None, beta
        else:
            self._float_beta, self._signal_beta = float(getattr(beta, "value", beta)), None
        self.gamma = float(gamma)
        self.As = []
        self.Xs = []
        # beta == 1 on Y itself is an increment of Y; anything else sets Y
        self._incs_Y = self._signal_beta is None and self._float_beta == 1 and self.Y_in is self.Y

    @classmethod
    def convert_to(cls, op):
        """Wrap a plain ``DotInc`` as a one-term MultiDotInc; pass others through."""
        if type(op).__name__ == "BsrDotInc":
            raise NotImplementedError("Optimized BsrDotInc operations not yet supported")
        if type(op).__name__ != "DotInc":
            return op
        new = cls(op.Y, op.Y, beta=1, gamma=0, tag=op.tag)
        new.add_AX(op.A, op.X)
        assert set(op.reads).issuperset(new.reads)
        assert list(new.incs) == list(op.incs) and list(new.sets) == list(op.sets)
        assert all(s.size for s in new.all_signals), op
        return new

    def add_AX(self, A, X):
        assert X.ndim == 1
        self.As.append(A)
        self.Xs.append(X)

    # sets/incs/reads/updates are derived, not stored
    @property
    def reads(self):
        out = self.As + self.Xs
        if not self._incs_Y:
            if self._signal_beta is not None:
                out = out + [self._signal_beta]
                if self.Y_in is not self.Y:
                    out = out + [self.Y_in]
            elif self._float_beta != 0 and self.Y_in is not self.Y:
                out = out + [self.Y_in]
        return out

    @reads.setter
    def reads(self, value):
        pass

    @property
    def incs(self):
        return [self.Y] if self._incs_Y else []

    @incs.setter
    def incs(self, value):
        pass

    @property
    def sets(self):
        return [] if self._incs_Y else [self.Y]

    @sets.setter
    def sets(self, value):
        pass

    @property
    def updates(self):
        return []

    @updates.setter
    def updates(self, value):
        pass

    def __str__(self):
        beta = self._float_beta if self._signal_beta is None else self._signal_beta
        dots = ", ".join("dot(%s, %s)" % (A, X) for A, X in zip(self.As, self.Xs))
        return "<MultiDotInc(tag=%s, Y=%s, Y_in=%s, beta=%s, gamma=%s, dots=[%s]) at 0x%x>" % (
            self.tag, self.Y, self.Y_in, beta, self.gamma, dots, id(self))

    __repr__ = __str__

    @classmethod
    def compress(cls, operators):
        """Merge all MultiDotIncs that target the same Y view into one op."""
        setters, incrementers, others = {}, {}, []
        for op in operators:
            if not isinstance(op, cls):
                others.append(op)
            elif op.sets:
                assert len(op.sets) == 1 and not op.incs
                setters.setdefault(op.sets[0], []).append(op)
            else:
                assert len(op.incs) == 1 and not op.sets
                incrementers.setdefault(op.incs[0], []).append(op)

        merged = list(others)
        for view, ops in setters.items():
            (set_op,) = ops
            for inc_op in incrementers.pop(view, []):
                set_op.As.extend(inc_op.As)
                set_op.Xs.extend(inc_op.Xs)
            merged.append(set_op)
        for view, ops in incrementers.items():
            if not ops:
                continue
            head = ops[0]
            for other in ops[1:]:
                head.As.extend(other.As)
                head.Xs.extend(other.Xs)
            merged.append(head)
        return merged

    @staticmethod
    def _as2d(view):
        if view.ndim == 0:
            return view.reshape(1, 1)
        if view.ndim == 1:
            return view.reshape(view.shape[0], 1)
        if view.ndim == 2:
            return view
        raise ValueError("No support for tensors with %d dimensions" % view.ndim)

    def get_views(self):
        """2-D views of every operand; a (1,1) ``A`` swaps roles with its ``X``."""
        Y_view = self._as2d(self.Y)
        Y_in_view = self._as2d(self.Y_in)
        beta_view = self._as2d(self._signal_beta) if self._signal_beta is not None else None
        A_views, X_views = [], []
        for A, X in zip(self.As, self.Xs):
            X_view = self._as2d(X)
            A_view = A.reshape((1, A.shape[0])) if (A.ndim == 1 and X.ndim == 1) else self._as2d(A)
            if A_view.shape == (1, 1):
                A_view, X_view = X_view, A_view
            elif not (X_view.shape[0] == A_view.shape[1] and X_view.shape[1] == Y_view.shape[1]
                      and A_view.shape[0] == Y_view.shape[0]):
                raise ValueError("shape mismach (A: %s, X: %s, Y: %s)" % (A.shape, X.shape, self.Y.shape))
            A_views.append(A_view)
            X_views.append(X_view)
        return A_views, X_views, Y_view, Y_in_view, beta_view


def signal_io_dicts(operators):
    """base signal -> operators that set / inc / read / update it."""
    bases = {s.base for op in operators for s in op.all_signals}
    sets = {b: [] for b in bases}
    incs = {b: [] for b in bases}
    reads = {b: [] for b in bases}
    updates = {b: [] for b in bases}
    for op in operators:
        for s in op.sets:
            sets[s.base].append(op)
        for s in op.incs:
            incs[s.base].append(op)
        for s in op.reads:
            reads[s.base].append(op)
        for s in op.updates:
            updates[s.base].append(op)
    return sets, incs, reads, updates


def remove_unmodified_resets(operators):
    """Drop ``Reset`` ops whose target is never incremented or updated: the
    reset value becomes the signal's initial value instead."""
    _, incs, _, updates = signal_io_dicts(operators)
    kept = []
    for op in operators:
        if type(op).__name__ == "Reset" and not incs[op.dst.base] and not updates[op.dst.base]:
            init = op.dst.initial_value
            writable = init.flags.writeable
            if not writable:
                init.setflags(write=True)
            init[...] = op.value
            if not writable:
                init.setflags(write=False)
        else:
            kept.append(op)
    return kept


def remove_zero_incs(operators):
    """Drop DotInc / ElementwiseInc / Copy ops whose input is known to be zero
    (only ever reset to 0, or a constant all-zero signal that nothing writes)."""
    sets, incs, _, updates = signal_io_dicts(operators)
    writers_of = {}  # base -> its writers (looked up once per base: a graph model reads one base thousands of times)

    def writers_list(base):
        if base not in writers_of:
            writers_of[base] = sets[base] + incs[base] + updates[base]
        return writers_of[base]

    kept = []
    for op in operators:
        if type(op).__name__ not in ("DotInc", "ElementwiseInc", "Copy", "ConvInc"):
            kept.append(op)
            continue
        drop = False
        for src in op.reads:
            if src.name.startswith("<Node"):
                continue  # node outputs may change at run time
            writers = writers_list(src.base)
            only_zero_reset = (len(writers) == 1 and type(writers[0]).__name__ == "Reset"
                               and np.all(writers[0].value == 0))
            constant_zero = len(writers) == 0 and np.all(np.asarray(src.initial_value) == 0)
            if only_zero_reset or constant_zero:
                drop = True
                break
        if not drop:
            kept.append(op)
        elif op.sets:
            kept.append(Reset(op.sets[0]))
    return kept


def simplify_operators(operators):
    """Apply every function in ``simplifications`` in turn."""
    for simplification in simplifications:
        operators = simplification(operators)
    return operators


# Modify this list to change which simplifications the simulator applies.
simplifications = [remove_unmodified_resets, remove_zero_incs]

__all__ = ["MultiDotInc", "signal_io_dicts", "remove_unmodified_resets", "remove_zero_incs",
           "simplify_operators", "simplifications", "Copy", "DotInc", "ElementwiseInc"]
