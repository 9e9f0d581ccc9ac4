"""Operator simplification, MultiDotInc merging and the greedy planner on the
host (cases of the reference's nengo_ocl/tests/test_operators.py:9-86,
test_planners.py:41-47 and the merge in test_simulator.py:14-38)."""

import numpy as np
import pytest

from nengo_ocl_b200 import model as m
from nengo_ocl_b200 import operators as ops_mod
from nengo_ocl_b200 import synth
from nengo_ocl_b200.operators import MultiDotInc, remove_unmodified_resets, remove_zero_incs, simplify_operators
from nengo_ocl_b200.planners import greedy_planner, operator_dependency_graph, _dependency_graph_fast


def test_signal_views():
    base = m.Signal(np.arange(24.0).reshape(4, 6), name="base")
    v = base[1:3, ::2]
    assert v.is_view and v.base is base and v.shape == (2, 3)
    assert v.elemoffset == 6 and v.elemstrides == (6, 2)
    assert np.array_equal(v.initial_value, np.arange(24.0).reshape(4, 6)[1:3, ::2])
    col = base[:, 2]
    assert col.shape == (4,) and col.elemstrides == (6,) and col.elemoffset == 2
    r = col.reshape(4, 1)
    assert r.elemstrides == (6, 6) and r.shape == (4, 1)
    assert base[0].may_share_memory(base[0, 2:4]) and not base[0].may_share_memory(base[1])
    assert not base.may_share_memory(m.Signal(np.zeros(3)))
    with pytest.raises(ValueError):
        v.reshape(6)


def test_multidotinc_convert_and_compress():
    a = m.Signal(np.zeros(2), name="a")
    A, B = m.Signal(np.eye(2)), m.Signal(np.eye(2))
    x, y = m.Signal(np.ones(2)), m.Signal(np.ones(2))
    d1, d2 = m.DotInc(A, x, a), m.DotInc(B, y, a)
    other = m.Reset(a)
    converted = [MultiDotInc.convert_to(op) for op in (other, d1, d2)]
    assert converted[0] is other and all(isinstance(c, MultiDotInc) for c in converted[1:])
    assert converted[1].incs == [a] and converted[1].sets == [] and set(converted[1].reads) == {A, x}
    merged = MultiDotInc.compress(converted)
    mdis = [op for op in merged if isinstance(op, MultiDotInc)]
    assert len(mdis) == 1 and mdis[0].As == [A, B] and mdis[0].Xs == [x, y]
    # a beta != 1 op sets its target, and absorbs increments of the same view
    setter = MultiDotInc(a, a, beta=0.5, gamma=1.0)
    setter.add_AX(A, x)
    inc = MultiDotInc.convert_to(m.DotInc(B, y, a))
    out = MultiDotInc.compress([setter, inc])
    assert out == [setter] and setter.As == [A, B] and setter.sets == [a]


def test_multidotinc_views_swap_scalar_a():
    y = m.Signal(np.zeros(3))
    s = m.Signal(np.array(2.0))
    x = m.Signal(np.ones(3))
    op = MultiDotInc.convert_to(m.DotInc(s.reshape(1, 1), x, y)) if False else None
    mdi = MultiDotInc(y, y, 1, 0)
    mdi.As.append(s.reshape(1, 1)), mdi.Xs.append(x)
    A_views, X_views, Y_view, Y_in_view, beta_view = mdi.get_views()
    assert A_views[0].shape == (3, 1) and X_views[0].shape == (1, 1)  # roles swapped
    assert Y_view.shape == (3, 1) and beta_view is None
    bad = MultiDotInc(y, y, 1, 0)
    bad.As.append(m.Signal(np.zeros((2, 3)))), bad.Xs.append(x)
    with pytest.raises(ValueError):
        bad.get_views()


def test_remove_unmodified_resets_and_zero_incs():
    a = m.Signal(np.zeros(2), name="a")
    b = m.Signal(np.zeros(2), name="b")
    zero = m.Signal(np.zeros(2), name="zero")
    x = m.Signal(np.ones(2), name="x")
    A = m.Signal(np.eye(2))
    ops = [m.Reset(a, value=3.0), m.Reset(b), m.DotInc(A, zero, b), m.DotInc(A, x, b), m.Copy(zero, a, inc=False)]
    out = remove_zero_incs(ops)
    # the zero-input DotInc disappears; the zero-input Copy (a set) becomes a Reset of its target
    assert sum(isinstance(o, m.DotInc) for o in out) == 1
    assert sum(isinstance(o, m.Copy) for o in out) == 0 and sum(isinstance(o, m.Reset) for o in out) == 3
    out = remove_unmodified_resets([m.Reset(a, value=3.0), m.Reset(b), m.DotInc(A, x, b)])
    assert len(out) == 2 and np.all(a.initial_value == 3.0)
    assert ops_mod.simplifications == [remove_unmodified_resets, remove_zero_incs]
    assert len(simplify_operators([m.Reset(a)])) == 0


def test_dependency_graph_fast_equals_reference_rule():
    mdl = synth.pes_learning_model(n_ensembles=6, n_neurons=16, dimensions=2, n_templates=2, n_probes=1,
                                   sim_time=0.05)
    ops = MultiDotInc.compress(list(map(MultiDotInc.convert_to, simplify_operators(list(mdl.operators)))))
    slow = operator_dependency_graph(ops)
    fast = _dependency_graph_fast(ops)
    assert {k: set(v) for k, v in slow.items()} == {k: set(v) for k, v in fast.items()}


def test_greedy_planner_groups_respect_dependencies():
    mdl = synth.two_ensemble_model()
    ops = MultiDotInc.compress(list(map(MultiDotInc.convert_to, simplify_operators(list(mdl.operators)))))
    groups = greedy_planner(ops)
    assert sum(len(g) for _, g in groups) == len(ops)
    assert len([t for t, _ in groups if t is m.Reset]) == 1  # all resets planned together
    position = {op: i for i, (_, g) in enumerate(groups) for op in g}
    for op, later in operator_dependency_graph(ops).items():
        for op2 in later:
            assert position[op] < position[op2]
    for typ, g in groups:
        assert all(type(op) is typ for op in g)
        written = [s for op in g for s in list(op.sets) + list(op.incs) + list(op.updates)]
        for i, s in enumerate(written):
            assert not any(s.may_share_memory(s2) for s2 in written[i + 1:])
    cyc_a, cyc_b = m.Signal(np.zeros(1)), m.Signal(np.zeros(1))
    with pytest.raises(ValueError):
        greedy_planner([m.Copy(cyc_a, cyc_b), m.Copy(cyc_b, cyc_a)])


def test_lowpass_and_linear_filter_coefficients():
    num, den = m.Lowpass(0.01).discrete_tf(0.001)
    a = np.exp(-0.1)
    assert np.allclose(num, [1 - a]) and np.allclose(den, [-a])
    num2, den2 = m.LinearFilter([1.0], [0.01, 1.0]).discrete_tf(0.001)
    assert np.allclose(num2, num) and np.allclose(den2, den)
    num3, den3 = m.Alpha(0.01).discrete_tf(0.001)
    assert len(num3) == 2 and len(den3) == 2
    assert np.isclose(num3.sum() / (1 + den3.sum()), 1.0)  # unit DC gain


def test_function_translation_to_postfix():
    from nengo_ocl_b200.ast_conversion import DeviceFunction, OPS

    f = DeviceFunction(lambda t: np.sin(t), [1])
    assert f.program == [(OPS["IN0"], 0), (OPS["SIN"], 0), (OPS["STORE"], 0)]
    g = DeviceFunction(lambda t, x: [x[0] * x[1], t + 2.5], [1, 2])
    assert g.out_dim == 2 and g.constants == [2.5]
    with pytest.raises(NotImplementedError):
        DeviceFunction(lambda x: sorted(x), [3])
    with pytest.raises(NotImplementedError):
        DeviceFunction(lambda t: [t, t], [1], out_dim=3)


def test_deep_expression_is_not_sent_to_the_device():
    """The device interpreter evaluates on a fixed-size stack; the translator computes the depth
    a program needs and refuses deeper ones (the simulator then runs the function on the host).
    Checked on the host only: such a program must never reach the kernel."""
    from nengo_ocl_b200.ast_conversion import DeviceFunction, MAX_STACK, stack_depth

    shallow = DeviceFunction(lambda t, x: [x[0] * x[1], t + 2.5], [1, 2])
    assert shallow.max_depth == 2 == stack_depth(shallow.program)

    def horner(x):
        return x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (
            1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (
                1 + x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1])))))))))))))))))))

    with pytest.raises(NotImplementedError, match="stack"):
        DeviceFunction(horner, [2])
    assert MAX_STACK == 32

    def medium(x):
        return x[0] * (1 + x[1] * (1 + x[0] * (1 + x[1] * (1 + x[0]))))

    assert DeviceFunction(medium, [2]).max_depth == 9


def test_gather_sum_over_slices_and_reset_folding():
    """The fusion passes on operator lists: copies into slices of a reset signal become one
    gather-sum with one part per slice (gaps are only zeroed); a reset followed by one merged
    product becomes the product in set form."""
    from nengo_ocl_b200 import fusion

    a = m.Signal(np.zeros(6), name="a")
    s1, s2, s3 = (m.Signal(np.ones(2) * k, name="s%d" % k) for k in (1, 2, 3))
    ops = [m.Reset(a), m.Copy(s1, a[0:2], inc=True), m.Copy(s2, a[4:6], inc=True), m.Copy(s3, a[0:2], inc=True)]
    gathers, consumed = fusion.find_gather_sums(ops)
    assert len(gathers) == 1 and consumed == set(ops)
    parts = gathers[0].parts
    assert [(off, size) for off, size, _ in parts] == [(0, 2), (2, 2), (4, 2)]
    assert parts[0][2] == [s1, s3] and parts[1][2] == [] and parts[2][2] == [s2]
    # partially overlapping slices are left alone
    bad = [m.Reset(a), m.Copy(s1, a[0:2], inc=True), m.Copy(s2, a[1:3], inc=True)]
    assert fusion.find_gather_sums(bad)[0] == []

    y = m.Signal(np.zeros(3), name="y")
    A = m.Signal(np.eye(3), name="A", readonly=True)
    x = m.Signal(np.ones(3), name="x")
    reset, dot = m.Reset(y), MultiDotInc.convert_to(m.DotInc(A, x, y))
    dropped = fusion.fold_resets_into_products([reset, dot])
    assert dropped == {reset}
    assert dot._float_beta == 0 and dot.gamma == 0 and dot.sets == [y] and dot.incs == []
    # a reset to another value stays: "value + terms" and "terms + value" round differently
    reset_h, dot_h = m.Reset(y, value=0.5), MultiDotInc.convert_to(m.DotInc(A, x, y))
    assert fusion.fold_resets_into_products([reset_h, dot_h]) == set() and dot_h._float_beta == 1
    # a second writer of y keeps the reset
    reset2, dot2 = m.Reset(y), MultiDotInc.convert_to(m.DotInc(A, x, y))
    assert fusion.fold_resets_into_products([reset2, dot2, m.Copy(x, y, inc=True)]) == set()
    assert dot2._float_beta == 1


def test_member_reading_a_fused_output_is_not_fused():
    """An ensemble whose encoder product reads a signal that the fused kernel writes (here: the
    filtered output of another ensemble's connection, directly, without an input signal in
    between) must stay un-fused: inside one kernel it could see the old or the new value."""
    from types import SimpleNamespace

    from nengo_ocl_b200 import fusion, synth
    from nengo_ocl_b200.operators import simplify_operators

    nb = synth.NetBuilder(dt=0.001, seed=1)
    a = nb.ensemble(40, 2, label="a")
    b = nb.ensemble(40, 2, label="b")
    conn = nb.connect_decoded(a, None, nb.solve_decoders(a), synapse=0.005, label="a->b")
    # b's encoders read the filtered value itself (and a constant keeps a's input alive)
    nb.model.operators = [op for op in nb.model.operators
                          if not (type(op).__name__ == "DotInc" and op.Y is b.sig_J)]
    nb.model.add_op(m.DotInc(b.sig_enc, conn["out"], b.sig_J, tag="b.encode"))
    nb.model.add_op(m.Copy(nb.node_const([0.3, -0.2]), a.sig_in, inc=True))
    ops = simplify_operators(list(nb.model.operators))
    ops = MultiDotInc.compress(list(map(MultiDotInc.convert_to, ops)))
    views = {}
    for op in ops:
        if isinstance(op, MultiDotInc):
            A_views, X_views, *_ = op.get_views()
            views[op] = (A_views, X_views)
    sim = SimpleNamespace(_A_views={op: v[0] for op, v in views.items()},
                          _X_views={op: v[1] for op, v in views.items()},
                          model=SimpleNamespace(sig={}, probes=[], dt=0.001),
                          linear_filter_coefficients=lambda op: op.process.discrete_tf(0.001))
    members, consumed = fusion.find_fusable(sim, ops)
    fused = {mem["neurons"].J for mem in members}
    assert a.sig_J in fused and b.sig_J not in fused
    assert not any(getattr(op, "J", None) is b.sig_J for op in consumed)


def test_step_loop_barriers_follow_the_signal_dependencies():
    """Grid barriers of the persistent step loop: one before every phase that touches what an
    earlier phase since the last barrier wrote (or writes what it read), the previous step's
    phases included."""
    from nengo_ocl_b200.plan import phase_barriers

    # clock | gather x <- f | ensembles x -> f (state v) | probes f -> ring
    uses = [(set(), {"t"}), ({"f"}, {"x"}), ({"x", "v"}, {"f", "v"}), ({"f"}, {"ring"})]
    assert phase_barriers(uses) == [False, False, True, True]
    # the gather of the next step reads f while the probes only read it: no barrier at the step boundary,
    # but a phase that overwrites what the last phase of the previous step read needs one
    uses = [({"a"}, {"b"}), ({"b"}, {"c"}), ({"c"}, {"a"})]
    assert phase_barriers(uses) == [True, True, True]
    # independent phases that only rewrite their own outputs: one barrier per step keeps the steps apart
    assert phase_barriers([(set(), {"a"}), (set(), {"b"})]) == [True, False]
    assert phase_barriers([({"k"}, {"a"}), ({"k"}, {"b"}), ({"a", "b"}, {"c"})]) == [True, False, True]


def test_phase_barriers_of_a_single_pass():
    """A group of plans launched once per step is not a ring: only conflicts inside the pass count."""
    from nengo_ocl_b200.plan import phase_barriers

    uses = [(set(), {"t"}), ({"t"}, {"y"}), ({"q"}, {"z"})]
    assert phase_barriers(uses, ring=False) == [False, True, False]
    assert phase_barriers(uses, ring=True) == [True, True, False]


def test_planner_extents_agree_with_pairwise_overlap():
    """The sorted-range structure of the planner against the pairwise test it replaces."""
    from nengo_ocl_b200.planners import _Extents

    rng = np.random.RandomState(0)
    for trial in range(50):
        ext, ranges = _Extents(), []
        for _ in range(60):
            lo = int(rng.randint(0, 400))
            hi = lo + int(rng.randint(1, 12))
            want = any(l < hi and lo < h for l, h in ranges)
            assert ext.overlaps(lo, hi) == want
            if not want or trial % 5 == 0:  # every fifth trial also stores overlapping ranges
                ext.add(lo, hi)
                ranges.append((lo, hi))
