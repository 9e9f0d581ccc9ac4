"""Planning of whole models without a GPU (tests/fake_library.py stands in for the C library):
which plans a model becomes, what the fused tables contain, how the captured step is shaped.
The arithmetic is checked on the GPU (tests/*_gpu.py); here the host logic."""

import numpy as np
import pytest

from nengo_ocl_b200 import simulator as sim_mod
from nengo_ocl_b200 import synth
from nengo_ocl_b200.plan import PhaseGroup

import fake_library


@pytest.fixture
def fake(monkeypatch):
    lib = fake_library.install(monkeypatch)
    monkeypatch.setattr(sim_mod.Simulator, "some_context", None)
    from nengo_ocl_b200 import runtime

    monkeypatch.setattr(runtime, "_default_context", None, raising=False)
    return lib


def names(plans):
    return [p.name for p in plans]


def test_pes_model_is_one_streamed_kernel_and_four_helpers(fake, monkeypatch):
    from nengo_ocl_b200 import plan as plan_mod

    # (block counts as at the benchmark size, where no plan but the clock is tiny)
    monkeypatch.setattr(plan_mod, "phase_blocks", lambda p: 1 if p.name == "cl_timeupdate" else 100)
    mdl = synth.pes_learning_model(seed=3, n_ensembles=12, n_neurons=1024, dimensions=16, n_templates=2, n_probes=3,
                                   sim_time=0.05)
    sim = sim_mod.Simulator(None, model=mdl, step_loop=False)
    assert sorted(names(sim._plans)) == sorted(["gather_sum", "cl_timeupdate", "cl_presentinput", "fused_ensemble_step",
                                                 "cl_probes"])
    fused = [p for p in sim._plans if p.name == "fused_ensemble_step"][0]
    t = fused.tables
    assert len(t["streamed"]) == 12 and len(t["small"]) == 0 and len(t["large"]) == 0
    # E records start on multiples of 32 neurons and hold at most a stage's worth (96 neurons with the
    # 16 encoder columns of this model, more for an ensemble without input), D records are whole rows
    rec = t["records"]
    e_rec, d_rec = rec[rec[:, 0] == 1], rec[rec[:, 0] == 2]
    assert len(e_rec) and len(d_rec)
    from nengo_ocl_b200 import fusion

    assert (e_rec[:, 3] % 32 == 0).all() and (e_rec[:, 4] <= fusion.STREAM_CHUNK).all()
    with_input = t["ens"][e_rec[:, 1], 6] > 0
    assert (e_rec[with_input, 4] <= 96).all() and (e_rec[with_input, 4] * 20 <= fusion.STREAM_STAGE_FLOATS).all()
    assert (d_rec[:, 7] * ((d_rec[:, 11] + 127) // 128) <= 16).all()
    # every plan says what it touches; the PES error gather was folded away (read in place)
    assert all(p.signal_use is not None for p in sim._plans)
    assert names(sim._plans).count("gather_sum") == 1
    # one step = five launches: a single tiny plan is not a group
    assert sim._plans.launches_per_step == 5
    sim.close()


def test_graph_model_groups_its_tiny_plans(fake, monkeypatch):
    mdl = synth.watts_strogatz_model(seed=2, n_ensembles=64, n_neurons=50, k=4, n_templates=4, n_probes=3)
    # (the stand-in library reports one block for every plan: give the real counts of the tiny ones)
    from nengo_ocl_b200 import plan as plan_mod

    blocks = {"cl_timeupdate": 1, "cl_direct": 1, "gather_sum": 16, "fused_ensemble_step": 8, "cl_probes": 3}
    monkeypatch.setattr(plan_mod, "phase_blocks", lambda p: blocks.get(p.name))
    sim = sim_mod.Simulator(None, model=mdl, step_loop=False)
    assert "fused_ensemble_step" in names(sim._plans) and "cl_direct" in names(sim._plans)
    launch = sim._plans.launch_plans()
    groups = [p for p in launch if isinstance(p, PhaseGroup)]
    assert len(groups) == 1 and names(groups[0].members) == ["cl_timeupdate", "cl_direct"]
    assert len(launch) == len(sim._plans) - 1
    # the group touches what its members touch
    reads, writes = groups[0].signal_use
    assert reads >= set(groups[0].members[1].signal_use[0]) and writes >= set(groups[0].members[0].signal_use[1])
    sim.close()


def test_step_loop_is_built_from_the_plans_phase_forms(fake):
    mdl = synth.two_ensemble_model(seed=0)
    sim = sim_mod.Simulator(None, model=mdl, step_loop="single")
    loop = sim._plans.step_loop
    assert loop is not None
    added = [c[0] for c in fake.calls if c[0].startswith("nb2_step_loop_add_")]
    # one phase per plan, in plan order
    want = {"cl_timeupdate": "timeupdate", "gather_sum": "gather_sum", "cl_direct": "direct",
            "fused_ensemble_step": "ensemble_step", "cl_probes": "probes"}
    assert added == ["nb2_step_loop_add_" + want[n] for n in names(sim._plans)]
    sim.run_steps(3)  # three steps: one launch of the loop (plus the status read)
    assert [c[0] for c in fake.calls].count("nb2_step_loop_run") == 1
    sim.close()


def test_models_with_host_code_or_ring_buffers_keep_the_graph_path(fake):
    mdl = synth.circular_convolution_model(seed=4, dimensions=16, n_neurons=64, n_templates=3)
    sim = sim_mod.Simulator(None, model=mdl, step_loop=True)
    assert sim._plans.step_loop is not None  # every plan of this model has a phase form
    sim.close()
    from nengo_ocl_b200 import model as m

    mdl2 = synth.white_noise_model(seed=21, n=64)
    sim2 = sim_mod.Simulator(None, model=mdl2, step_loop=True)
    assert "cl_whitenoise" in names(sim2._plans)
    assert sim2._plans.step_loop is None  # the noise plan has no phase form
    sim2.close()


def test_host_clock_matches_the_clock_kernel(fake):
    """``run_steps`` advances ``n_steps`` / ``time`` on the host between probe drains; the values must
    be the ones the clock kernel leaves in the step and time signals (oracle: K.timeupdate)."""
    from nengo_ocl_b200.raggedarray import RaggedArray
    from oracle import kernels as K

    mdl = synth.two_ensemble_model(seed=0)
    sim = sim_mod.Simulator(None, model=mdl, step_loop=False)
    step = RaggedArray([np.zeros((1, 1))], dtype=np.float32)
    time = RaggedArray([np.zeros((1, 1))], dtype=np.float32)
    done = 0
    for batch in (1, 2, 7, 256, 256, 1000, 33):
        sim._probe(steps_run=batch)  # (the stand-in library runs nothing: only the host arithmetic)
        for _ in range(batch):
            K.timeupdate(step, time, mdl.dt)
        done += batch
        assert sim.n_steps == done == int(step[0][0, 0])
        assert np.float32(sim.time) == time[0][0, 0]
    sim.close()


def test_plan_functions_keep_the_reference_error_conventions(fake):
    """Argument checks of the plan functions that have no kernel-side counterpart: an unsupported
    padding is a ValueError (clra_nonlinearities.py:1886-1893), biases are asserted absent (:1787),
    a noise plan needs one key, one enum and two parameters per item."""
    from nengo_ocl_b200 import cura_nonlinearities as nl
    from nengo_ocl_b200 import model as m
    from nengo_ocl_b200.curaggedarray import CUDARaggedArray
    from nengo_ocl_b200.raggedarray import RaggedArray
    from nengo_ocl_b200.runtime import CommandQueue, create_some_context, to_device

    queue = CommandQueue(create_some_context())
    data = CUDARaggedArray(queue, RaggedArray([np.zeros(2 * 5 * 5), np.zeros(3 * 3 * 2 * 4), np.zeros(4 * 3 * 3)],
                                              dtype=np.float32))
    X, F, Y = (data.getitem_device(i) for i in range(3))
    args = dict(shape_in=(5, 5, 2), shape_out=(3, 3, 4), kernel_shape=(3, 3))
    plan = nl.plan_conv2d(queue, X, Y, F, padding="valid", **args)
    assert plan.name == "cl_conv2d" and plan.flops_per_call == 2 * 3 * 3 * 4 * 2 * 3 * 3
    plan()
    assert ("nb2_conv2d", 19) in fake.calls
    with pytest.raises(ValueError):
        nl.plan_conv2d(queue, X, Y, F, padding="full", **args)
    with pytest.raises(AssertionError):
        nl.plan_conv2d(queue, X, Y, F, biases=Y, **args)
    with pytest.raises(AssertionError):  # the output does not have the size the shapes imply
        nl.plan_conv2d(queue, X, Y, F, shape_in=(5, 5, 2), shape_out=(3, 3, 5), kernel_shape=(3, 3))

    Yn = CUDARaggedArray(queue, RaggedArray([np.zeros(5), np.zeros(3)], dtype=np.float32))
    step = CUDARaggedArray(queue, RaggedArray([np.zeros((1, 1))], dtype=np.float32))
    enums, params = nl.get_dist_enums_params([m.Uniform(-1, 1), m.Gaussian(0, 2)])
    assert [int(e[0, 0]) for e in enums] == [0, 1] and params[1][:, 0].tolist() == [0.0, 2.0]
    rngs = nl.create_rngs(queue, 2)
    nl.init_rngs(queue, rngs, [7, (5 << 32) | 9])
    assert rngs.get().view(np.uint32).tolist() == [[7, 0], [9, 5]]
    plan = nl.plan_whitenoise(queue, Yn, CUDARaggedArray(queue, enums), CUDARaggedArray(queue, params),
                              to_device(queue, np.zeros(2, np.int32)), to_device(queue, np.ones(2, np.int32)), 0.001,
                              rngs, step[[0, 0]])
    plan()
    assert plan.name == "cl_whitenoise" and ("nb2_whitenoise", 14) in fake.calls
    with pytest.raises(AssertionError):
        nl.plan_whitenoise(queue, Yn, CUDARaggedArray(queue, enums), CUDARaggedArray(queue, params),
                           to_device(queue, np.zeros(3, np.int32)), to_device(queue, np.ones(2, np.int32)), 0.001,
                           rngs, step[[0, 0]])
