"""Host logic of the graph capture along signal dependencies (``Plans._capture_branches``) and of
the grouping of tiny plans, checked on the CPU with a recording stand-in for the C library:
every pair of plans that conflicts on a signal must be ordered in the captured graph (by stream
order or by an event edge), in every step of an unrolled capture."""

import ctypes
import itertools

import numpy as np
import pytest

from nengo_ocl_b200 import _capi, plan as plan_mod


class Recorder:
    """Stand-in for the library: hands out stream / event handles and records the calls."""

    def __init__(self):
        self.calls = []
        self.handles = itertools.count(100)

    def call(self, name, *args):
        if name in ("nb2_stream_create", "nb2_event_create"):
            args[0]._obj.value = next(self.handles)
            return 0
        if name == "nb2_graph_end":
            args[1]._obj.value = next(self.handles)
        self.calls.append((name,) + tuple(self._plain(a) for a in args))
        return 0

    @staticmethod
    def _plain(a):
        if isinstance(a, ctypes.c_void_p):
            return a.value
        return a

    def lib(self):
        rec = self

        class _L:
            def __getattr__(self, name):
                return lambda *args: rec.call(name, *args)

        return _L()


class FakeQueue:
    stream = ctypes.c_void_p(1)

    def finish(self):
        pass


def make_plan(queue, rec, name, reads, writes, blocks=1):
    def kern(stream):
        rec.calls.append(("launch", name, rec._plain(stream)))

    p = plan_mod.Plan(queue, kern, (256, blocks), name=name)
    p.signal_use = (set(reads), set(writes))
    return p


def ordered_pairs(calls, n_plans, repeat):
    """Reachability between launches of one capture: node = (step, plan index)."""
    order = []         # launches in capture order
    stream_tail = {}   # stream -> last node on it
    event_node = {}    # event -> node it was recorded after (None: the fork)
    pending = {}       # stream -> nodes it waits for before its next launch
    preds = {}
    for c in calls:
        if c[0] == "nb2_event_record":
            event_node[c[1]] = stream_tail.get(c[2])
        elif c[0] == "nb2_stream_wait_event":
            pending.setdefault(c[1], set()).add(event_node[c[2]])
        elif c[0] == "launch":
            node = len(order)
            order.append(c[1])
            p = set(pending.pop(c[2], set()))
            if c[2] in stream_tail:
                p.add(stream_tail[c[2]])
            preds[node] = {q for q in p if q is not None}
            stream_tail[c[2]] = node
    assert len(order) == n_plans * repeat
    reach = {}
    for node in range(len(order)):
        r = set()
        for q in preds[node]:
            r |= {q} | reach[q]
        reach[node] = r
    return order, reach


@pytest.mark.parametrize("repeat", [1, 3])
def test_branch_capture_orders_every_conflicting_pair(monkeypatch, repeat):
    rec = Recorder()
    monkeypatch.setattr(_capi, "call", rec.call)
    monkeypatch.setattr(_capi, "lib", rec.lib)
    q = FakeQueue()
    # the shape of a graph model's step: gather | clock -> node function -> gather | ensembles | probes
    specs = [("gather1", {"f"}, {"x"}, 16), ("clock", set(), {"t"}, 1), ("direct", {"t"}, {"u"}, 1),
             ("gather2", {"u"}, {"x0"}, 1), ("fused", {"x", "x0", "v"}, {"f", "v"}, 512), ("probes", {"f"}, {"ring"}, 3)]
    plans = [make_plan(q, rec, *s) for s in specs]
    pl = plan_mod.Plans(plans, profiling=False, parallel=True)
    pl._capture(plans, repeat)
    order, reach = ordered_pairs(rec.calls, len(plans), repeat)
    uses = [p.signal_use for p in plans] * repeat
    n_parallel = 0
    for j in range(len(order)):
        for i in range(j):
            (ri, wi), (rj, wj) = uses[i], uses[j]
            conflict = bool(wi & (rj | wj) or ri & wj)
            if conflict:
                assert i in reach[j], (order[i], order[j], i, j)
            elif i not in reach[j]:
                n_parallel += 1
    assert n_parallel > 0  # something does run beside something else
    # the clock and the first gather of a step are independent of each other
    assert 0 not in reach[1] and 1 not in reach[0]
    # every branch is joined back into the origin stream before the capture ends
    end = [k for k, c in enumerate(rec.calls) if c[0] == "nb2_graph_end"][0]
    tail_streams = {c[2] for c in rec.calls[:end] if c[0] == "launch"} - {1}
    joined = {rec_c[1] for rec_c in rec.calls[:end] if rec_c[0] == "nb2_stream_wait_event" and rec_c[1] == 1}
    assert not tail_streams or joined == {1}


def test_chain_capture_without_declared_signals(monkeypatch):
    rec = Recorder()
    monkeypatch.setattr(_capi, "call", rec.call)
    monkeypatch.setattr(_capi, "lib", rec.lib)
    q = FakeQueue()
    plans = [make_plan(q, rec, "a", {"x"}, {"y"}), make_plan(q, rec, "b", {"y"}, {"z"})]
    plans[1].signal_use = None  # a plan that does not say what it touches: plain in-order capture
    pl = plan_mod.Plans(plans, profiling=False, parallel=True)
    pl._capture(plans, 2)
    assert [c[1] for c in rec.calls if c[0] == "launch"] == ["a", "b", "a", "b"]
    assert not [c for c in rec.calls if c[0] == "nb2_stream_wait_event"]


def test_tiny_plans_are_grouped_in_runs(monkeypatch):
    blocks = {"a": 1, "b": 2, "c": 40, "d": 1, "e": 1, "f": 3, "g": None}
    monkeypatch.setattr(plan_mod, "phase_blocks", lambda p: blocks[p.name])

    class Group:
        def __init__(self, queue, members):
            self.members = members
            self.name = "phase_group"

    monkeypatch.setattr(plan_mod, "PhaseGroup", Group)
    q = FakeQueue()
    rec = Recorder()
    plans = [make_plan(q, rec, n, set(), {n}) for n in "abcdefg"]
    out = plan_mod.group_tiny_plans(plans, max_blocks=4)
    shape = [[m.name for m in p.members] if isinstance(p, Group) else p.name for p in out]
    # a + b fit in four blocks; c is large; d + e fit, f would exceed four; g has no phase form
    assert shape == [["a", "b"], "c", ["d", "e"], "f", "g"]
