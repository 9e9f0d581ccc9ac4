"""The persistent step loop (csrc/nb2_step_loop.cu): n whole steps in one cooperative launch
must leave every signal and every probe sample bit-identical to the launch-per-plan path
and to the CPU oracle.  The reference has one way to run a step (nengo_ocl/plan.py:137-149),
so the launch-per-plan path is the behaviour being matched."""

import numpy as np
import pytest

from nengo_ocl_b200 import synth
from nengo_ocl_b200.simulator import Simulator
from oracle.simulator import OracleSimulator

pytestmark = pytest.mark.gpu

MODELS = {
    "two_ensembles": lambda: synth.two_ensemble_model(seed=0),
    "watts_strogatz": lambda: synth.watts_strogatz_model(seed=2, n_ensembles=300, n_neurons=50, k=4, n_templates=4,
                                                         n_probes=3),
    "circular_convolution": lambda: synth.circular_convolution_model(seed=4, dimensions=16, n_neurons=64,
                                                                     n_templates=3),
    # populations below the streamed kernel's size: warp- and CTA-per-ensemble phases with PES
    "pes_small": lambda: synth.pes_learning_model(seed=3, n_ensembles=12, n_neurons=128, dimensions=4,
                                                  n_templates=3, n_probes=3, sim_time=0.2),
    "pes_odd": lambda: synth.pes_learning_model(seed=3, n_ensembles=5, n_neurons=301, dimensions=3, n_templates=2,
                                                n_probes=3, sim_time=0.2),
}


def stored_signals(sim, mdl):
    """Base signals of the model that the simulator keeps up to date in device memory."""
    skip = {id(s) for g in sim.fused_groups for s in g["unstored"]}
    sigs = []
    for op in mdl.operators:
        for s in op.all_signals:
            if not s.base.sparse and id(s.base) not in skip and all(s.base is not t for t in sigs):
                sigs.append(s.base)
    return sigs


@pytest.mark.parametrize("mode", [True, "single"], ids=["grid", "one_cta"])
@pytest.mark.parametrize("name", list(MODELS))
def test_step_loop_matches_launch_per_plan_and_oracle(name, mode, parity_report):
    """Both forms of the loop: a cooperative grid with grid-wide barriers, and one CTA."""
    mdl = MODELS[name]()
    with Simulator(None, model=mdl, step_loop=mode) as loop, Simulator(None, model=mdl, step_loop=False) as plain:
        assert loop._plans.step_loop is not None, [p.name for p in loop._plans if getattr(p, "phase", None) is None]
        assert plain._plans.step_loop is None
        info = loop._plans.step_loop
        assert 1 <= info.n_barriers <= info.n_phases and info.grid >= 1
        assert info.grid == 1 or mode is True
        ora = OracleSimulator(mdl)
        total = differ = 0
        for steps in (100, 37, 1):  # each run_steps call is ONE launch of the loop
            loop.run_steps(steps)
            plain.run_steps(steps)
            for _ in range(steps):
                ora.step()
            for sig in stored_signals(loop, mdl):
                a, b = np.asarray(loop.signals[sig]), np.asarray(plain.signals[sig])
                assert np.array_equal(a, b), sig
            fused_pes = any(g.get("pes") for g in loop.fused_groups)
            pes = [c for c in mdl.info.get("connections", []) if "delta" in c] if fused_pes else []
            skip = {id(c[k]) for c in pes for k in ("delta", "weights")}
            for sig in stored_signals(loop, mdl):
                if id(sig) in skip:
                    continue
                a, ref = np.asarray(loop.signals[sig]), np.asarray(ora[sig])
                total += a.size
                differ += int(np.count_nonzero(a.reshape(-1) != ref.reshape(-1)))
        assert differ <= total // 1000000
        for p in mdl.probes:
            assert np.array_equal(loop.data[p], plain.data[p])
            assert np.array_equal(loop.data[p], np.array(ora.probe_data[p]))
    parity_report("step loop: %s, 138 steps in 3 launches (%d phases, %d barriers, %d CTAs)"
                  % (name, info.n_phases, info.n_barriers, info.grid),
                  elements=total, not_bit_identical=differ, out_of_tolerance=0, spikes_moved=0)


def test_default_uses_the_loop_only_for_tiny_models():
    with Simulator(None, model=MODELS["two_ensembles"]()) as tiny:
        assert tiny._plans.step_loop is not None and tiny._plans.step_loop.grid == 1
    with Simulator(None, model=MODELS["watts_strogatz"]()) as larger:
        assert larger._plans.step_loop is None


def test_models_without_a_phase_form_keep_the_graph_path():
    """The streamed ensemble kernel owns its CTAs for a whole step: such a model replays a graph."""
    mdl = synth.pes_learning_model(seed=3, n_ensembles=6, n_neurons=1024, dimensions=16, n_templates=2, n_probes=3,
                                   sim_time=0.2)
    with Simulator(None, model=mdl, step_loop=True) as sim:
        assert sim._plans.step_loop is None
        sim.run_steps(5)


def test_tiny_consecutive_plans_share_one_launch(monkeypatch):
    """Graph path: the clock update and the one-item node function of the graph model are one
    launch (a PhaseGroup), and the step is bit-identical to the ungrouped one."""
    mdl = MODELS["watts_strogatz"]()
    with Simulator(None, model=mdl, step_loop=False) as grouped:
        names = [p.name for p in grouped._plans.launch_plans()]
        assert "phase_group" in names and len(names) < len(grouped._plans)
        assert grouped._plans.launches_per_step < sum(p.n_launches for p in grouped._plans)
        grouped.run_steps(60)
        monkeypatch.setenv("NENGO_B200_GROUP_TINY", "0")
        with Simulator(None, model=mdl, step_loop=False) as plain:
            assert len(plain._plans.launch_plans()) == len(plain._plans)
            plain.run_steps(60)
            for sig in stored_signals(grouped, mdl):
                assert np.array_equal(np.asarray(grouped.signals[sig]), np.asarray(plain.signals[sig])), sig
            for p in mdl.probes:
                assert np.array_equal(grouped.data[p], plain.data[p])


def test_grid_barrier_wait_is_bounded():
    """A grid barrier that can only run out (it expects one arrival more than there are CTAs): the
    kernel returns within its wait limit, records NB2_ERR_TIMEOUT, the host raises, and after the
    status is cleared the same context and loop run the model again."""
    import time

    from nengo_ocl_b200 import _capi

    mdl = MODELS["watts_strogatz"]()
    with Simulator(None, model=mdl, step_loop=True) as sim, Simulator(None, model=mdl, step_loop=False) as plain:
        loop = sim._plans.step_loop
        assert loop is not None and loop.grid > 1
        t0 = time.time()
        _capi.call("nb2_step_loop_wait_selftest", loop.handle, sim.queue.stream)
        assert loop.status(sim.queue.stream) == -4  # NB2_ERR_TIMEOUT; the call synchronises the stream
        assert time.time() - t0 < 60
        with pytest.raises(RuntimeError):
            sim._plans.check_status()
        _capi.call("nb2_step_loop_clear_status", loop.handle, sim.queue.stream)
        sim.reset()
        sim.run_steps(20)
        plain.run_steps(20)
        for p in mdl.probes:
            assert np.array_equal(sim.data[p], plain.data[p])
