"""Scheduling of operators into groups that one ragged kernel launch can run.

``greedy_planner`` follows the reference's ``nengo_ocl/planners.py:9-95``:
repeatedly take the operator type with the most ready instances, keep the
instances whose written views do not overlap, and emit ``(type, [ops])``.
``operator_dependency_graph`` is the ordering rule nengo supplies there
(``nengo.utils.simulator``): on each base signal, per step,
sets -> incs -> reads -> updates.
"""

import bisect
from collections import defaultdict


def operator_dependency_graph(operators):
    """Edges ``op -> {ops that must run after it}``."""
    by_base = defaultdict(lambda: {"sets": [], "incs": [], "reads": [], "updates": []})
    for op in operators:
        for kind in ("sets", "incs", "reads", "updates"):
            for sig in getattr(op, kind):
                by_base[sig.base][kind].append((sig, op))

    edges = {op: set() for op in operators}

    def link(firsts, seconds):
        for s1, op1 in firsts:
            for s2, op2 in seconds:
                if op1 is not op2 and s1.may_share_memory(s2):
                    edges[op1].add(op2)

    for groups in by_base.values():
        link(groups["sets"], groups["incs"])
        link(groups["sets"], groups["reads"])
        link(groups["sets"], groups["updates"])
        link(groups["incs"], groups["reads"])
        link(groups["incs"], groups["updates"])
        link(groups["reads"], groups["updates"])
    return edges


def _dependency_graph_fast(operators):
    """Same edges as ``operator_dependency_graph`` with interval bucketing, so
    bases touched by thousands of views do not cost a quadratic scan."""
    import numpy as np

    by_base = defaultdict(lambda: {"sets": [], "incs": [], "reads": [], "updates": []})
    index = {}
    for i, op in enumerate(operators):
        index[op] = i
        for kind in ("sets", "incs", "reads", "updates"):
            for sig in getattr(op, kind):
                lo = sig.elemoffset
                hi = lo + sum((n - 1) * abs(st) for n, st in zip(sig.shape, sig.elemstrides)) + 1
                by_base[sig.base][kind].append((lo, hi, i))

    edges = [set() for _ in operators]
    order = ("sets", "incs", "reads", "updates")
    for groups in by_base.values():
        arrs = {}
        for kind in order:
            g = groups[kind]
            if g:
                a = np.array(g, dtype=np.int64)
                arrs[kind] = a[np.argsort(a[:, 0], kind="stable")]
        for ai, first in enumerate(order):
            if first not in arrs:
                continue
            fa = arrs[first]
            for second in order[ai + 1:]:
                if second not in arrs:
                    continue
                sa = arrs[second]
                if len(fa) * len(sa) <= 64:
                    for lo1, hi1, i1 in fa:
                        for lo2, hi2, i2 in sa:
                            if i1 != i2 and lo1 < hi2 and lo2 < hi1:
                                edges[i1].add(int(i2))
                    continue
                # second intervals sorted by lo: candidates have lo2 < hi1; filter hi2 > lo1
                lo2s = sa[:, 0]
                max_len = int((sa[:, 1] - sa[:, 0]).max())
                for lo1, hi1, i1 in fa:
                    a = np.searchsorted(lo2s, lo1 - max_len, side="left")
                    b = np.searchsorted(lo2s, hi1, side="left")
                    if b <= a:
                        continue
                    cand = sa[a:b]
                    hit = cand[cand[:, 1] > lo1][:, 2]
                    for i2 in hit:
                        if i2 != i1:
                            edges[i1].add(int(i2))
    return {op: {operators[j] for j in edges[i]} for i, op in enumerate(operators)}


def _extent(sig):
    """[lo, hi) element range of a signal inside its base (what ``Signal.may_share_memory`` compares)."""
    lo = sig.elemoffset
    return lo, lo + sum((n - 1) * abs(st) for n, st in zip(sig.shape, sig.elemstrides)) + 1


class _Extents:
    """Element ranges already written in one base signal: ``overlaps`` in O(log n) (the plain
    pairwise test is quadratic in the thousands of slices that a graph model copies into one
    signal).  Ranges are kept sorted by start; as long as they are pairwise disjoint -- always,
    unless one operator writes overlapping views itself -- only the last range that starts before
    ``hi`` can overlap [lo, hi)."""

    def __init__(self):
        self.los, self.his, self.disjoint = [], [], True

    def overlaps(self, lo, hi):
        if not self.disjoint:
            return any(l < hi and lo < h for l, h in zip(self.los, self.his))
        k = bisect.bisect_left(self.los, hi)  # ranges [0, k) start before hi
        return k > 0 and self.his[k - 1] > lo

    def add(self, lo, hi):
        if self.disjoint and self.overlaps(lo, hi):
            self.disjoint = False
        k = bisect.bisect_right(self.los, lo)
        self.los.insert(k, lo)
        self.his.insert(k, hi)


def greedy_planner(operators, dependency_graph=_dependency_graph_fast):
    """Group operators by type in a dependency-respecting order."""
    edges = dependency_graph(operators)

    # Successors are visited in operator-list order, so that operators that become ready together
    # (e.g. the increments of one signal after its reset) are scheduled in the order the model
    # lists them: float32 sums of several increments then do not depend on object hashes, as
    # they do when the successors are walked as a set.
    position = {op: i for i, op in enumerate(operators)}
    predecessors_of = {op: set() for op in operators}
    successors_of = {op: [] for op in operators}
    for op, dests in edges.items():
        successors_of[op] = sorted(dests, key=position.__getitem__)
        for op2 in dests:
            predecessors_of[op2].add(op)

    available = defaultdict(list)  # type -> ready ops, in first-ready order
    for op in operators:
        if not predecessors_of[op]:
            available[type(op)].append(op)

    schedule = []
    remaining = len(operators)
    while remaining > 0:
        if not available:
            raise ValueError("Cycles in the op graph")
        # the type with the most ready instances; among ties the one that became
        # available last (what a stable ascending sort followed by [-1] picks)
        chosen_type = None
        for t, ready in available.items():
            if chosen_type is None or len(ready) >= len(available[chosen_type]):
                chosen_type = t
        candidates = available[chosen_type]

        written = {"sets": defaultdict(_Extents), "incs": defaultdict(_Extents), "updates": defaultdict(_Extents)}

        def overlaps(op):
            for kind in ("sets", "incs", "updates"):
                for s in getattr(op, kind):
                    if written[kind][s.base].overlaps(*_extent(s)):
                        return True
            return False

        chosen = []
        left = []
        for op in candidates:
            if overlaps(op):
                left.append(op)
                continue
            chosen.append(op)
            for kind in ("sets", "incs", "updates"):
                for s in getattr(op, kind):
                    written[kind][s.base].add(*_extent(s))
        assert chosen
        schedule.append((chosen_type, chosen))

        if left:
            available[chosen_type] = left
        else:
            del available[chosen_type]
        for op in chosen:
            for op2 in successors_of[op]:
                preds = predecessors_of[op2]
                preds.discard(op)
                if not preds:
                    available[type(op2)].append(op2)
            del predecessors_of[op], successors_of[op]
        remaining -= len(chosen)

    assert len(operators) == sum(len(ops) for _, ops in schedule)
    return schedule
