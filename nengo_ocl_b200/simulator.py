"""Simulator: runs an operator-level model on one B200 through the C ABI.

Public surface of the reference's ``nengo_ocl.Simulator``
(nengo_ocl/simulator.py:145-1449): same constructor arguments, context-manager
use, ``run / run_steps / step / reset / close / clear_probes / trange``,
``data``, ``signals``, ``sim[signal]``, ``dt / n_steps / time``,
``print_plans / print_profiling``.  Build = simplify operators, merge DotIncs
into MultiDotIncs, group with the planner, pack every dense signal into ONE
float32 ragged array in HBM (views become extra ragged items), and turn each
operator group into a plan (``_plan_<OperatorType>``).  What differs is the
device layer: plans launch hand-written CUDA kernels, the step list is replayed
as a CUDA graph, groups that form the ensemble pattern (bias copy, encoder
GEMV, neuron update, decoder GEMV, synapse, PES) are fused into one kernel, and
probe buffers are drained with one bounded copy per probe.
"""

import ctypes
import logging
import os
import warnings
from collections import defaultdict
from collections.abc import Mapping
from io import StringIO

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.ast_conversion import DeviceFunction
from nengo_ocl_b200.cura_gemv import plan_block_gemv
from nengo_ocl_b200.cura_nonlinearities import (
    plan_bcm,
    plan_copy,
    plan_direct,
    plan_elementwise_inc,
    plan_lif,
    plan_lif_rate,
    plan_linearfilter,
    plan_oja,
    plan_presentinput,
    plan_probes,
    plan_rectified_linear,
    plan_reset,
    plan_sigmoid,
    plan_slicedcopy,
    plan_spiking_rectified_linear,
    plan_timeupdate,
    plan_voja,
)
from nengo_ocl_b200.curaggedarray import CUDARaggedArray, to_device
from nengo_ocl_b200.operators import MultiDotInc, simplify_operators
from nengo_ocl_b200.plan import BasePlan, Plans, PythonPlan
from nengo_ocl_b200.planners import greedy_planner
from nengo_ocl_b200.raggedarray import RaggedArray
from nengo_ocl_b200.runtime import CommandQueue, DeviceArray, create_some_context
from nengo_ocl_b200.utils import groupby, indent, stable_unique

logger = logging.getLogger(__name__)


class SimulatorClosed(RuntimeError):
    """Raised by run/step/reset on a closed simulator."""


class ReadonlyError(AttributeError):
    pass


class ValidationError(ValueError):
    pass


class ViewBuilder:
    """Maps every signal (base or view) to an item of the packed ragged array.

    Views become extra items that alias their base: ``start = base.start +
    elemoffset`` with the view's element strides (reference simulator.py:72-142)."""

    def __init__(self, bases, rarray):
        self.sidx = {bb: ii for ii, bb in enumerate(bases)}
        assert len(bases) == len(self.sidx)
        self.rarray = rarray
        self.starts, self.shape0s, self.shape1s, self.stride0s, self.stride1s, self.names = [], [], [], [], [], []
        self._A_views, self._X_views, self._YYB_views = {}, {}, {}

    def append_view(self, sig):
        if sig in self.sidx:
            return
        if not sig.is_view:
            raise ValueError("can only append views of known signals", sig)
        assert sig.size and sig.ndim <= 2
        idx = self.sidx[sig.base]
        shape0 = sig.shape[0] if sig.ndim > 0 else 1
        shape1 = sig.shape[1] if sig.ndim > 1 else 1
        self.starts.append(int(self.rarray.starts[idx]) + sig.elemoffset)
        self.shape0s.append(shape0)
        self.shape1s.append(shape1)
        self.stride0s.append(sig.elemstrides[0] if shape0 > 1 else 1)
        self.stride1s.append(sig.elemstrides[1] if shape1 > 1 else 1)
        self.names.append(getattr(sig, "name", ""))
        self.sidx[sig] = len(self.sidx)

    def add_views_to(self, rarray):
        rarray.add_views(self.starts, self.shape0s, self.shape1s, self.stride0s, self.stride1s, names=self.names)

    def setup_views(self, ops):
        views = [sig for op in ops for sig in op.all_signals]
        for op in ops:
            if isinstance(op, MultiDotInc):
                A_views, X_views, Y_view, Y_in_view, beta_view = op.get_views()
                views.extend(A_views + X_views + [Y_view, Y_in_view] + ([beta_view] if beta_view else []))
                self._A_views[op] = A_views
                self._X_views[op] = X_views
                self._YYB_views[op] = [Y_view, Y_in_view, beta_view]
        for view in views:
            if not getattr(view, "sparse", False):
                self.append_view(view)


class SimulationData(Mapping):
    """``sim.data[probe]`` -> array of recorded samples; also build parameters."""

    def __init__(self, raw):
        self.raw = raw
        self._cache = {}

    def __getitem__(self, key):
        rval = self.raw[key]
        if isinstance(rval, list):
            cached = self._cache.get(key)
            if cached is None or len(cached) != len(rval):
                cached = np.asarray(rval)
                cached.setflags(write=False)
                self._cache[key] = cached
            return cached
        return rval

    def __iter__(self):
        return iter(self.raw)

    def __len__(self):
        return len(self.raw)

    def reset(self, key=None):
        if key is None:
            self._cache.clear()
        else:
            self._cache.pop(key, None)


class Simulator:
    """Runs a model on a B200.

    Parameters
    ----------
    network : nengo.Network or None
        Built with nengo's builder when the nengo package is importable.
    dt, seed, model
        As in ``nengo.Simulator``; ``model`` may be a prebuilt
        ``nengo_ocl_b200.model.Model`` (then ``network`` is None).
    context : runtime.Context, optional
        Device to run on (default: ``LOCAL_RANK`` or device 0).
    n_prealloc_probes : int
        Steps buffered on the device between probe drains.
    profiling : bool, optional
        Time every plan with CUDA events (disables graph replay); defaults to
        the environment variable ``NENGO_OCL_PROFILING``.
    if_python_code : 'none' | 'warn' | 'error'
        Reaction when a Python function cannot be translated for the device.
    planner : callable
        Operator grouping function (see ``nengo_ocl_b200.planners``).
    fuse : bool
        Fuse ensemble-pattern operator groups into one kernel per step.
    graph_unroll : int
        Steps captured per CUDA graph (fewer graph launches per batch).
    exchange : (Signal, communicator), optional
        Multi-GPU run: the signal every rank replicates and of which this rank owns
        segment ``comm.rank`` (see ``nengo_ocl_b200.exchange``); other ranks' segments
        are refreshed before every step.
    stream_inputs : bool
        Keep input tables (WhiteSignal) in pinned host memory and upload only the
        rows of the next batch of steps before it runs.
    step_loop : bool, optional
        Run all steps of a ``run_steps`` batch as one launch of the persistent step-loop kernel
        instead of replaying a captured graph.  Default: only for models whose step is a handful
        of thread blocks (one CTA then runs the whole model out of its L1).  ``"single"`` forces
        that one-CTA form, ``True`` a grid as wide as the widest plan.
    """

    some_context = None
    #: large populations go through the streamed fused kernel (``nb2_ensemble_stream``); False keeps
    #: every fused population in the CTA- or warp-per-ensemble kernel
    stream_ensembles = True

    def Array(self, val, dtype=np.float32):
        return to_device(self.queue, np.asarray(val, dtype=dtype))

    def RaggedArray(self, listofarrays, **kwargs):
        return CUDARaggedArray.from_arrays(self.queue, listofarrays, **kwargs)

    def __init__(self, network, dt=0.001, seed=None, model=None, context=None, n_prealloc_probes=32,
                 profiling=None, if_python_code="none", planner=greedy_planner, progress_bar=True, fuse=True,
                 graph_unroll=8, stream_inputs=False, exchange=None, step_loop=None):
        self.closed = False
        self.model = None
        if context is None and Simulator.some_context is None:
            Simulator.some_context = create_some_context()
        if profiling is None:
            profiling = int(os.getenv("NENGO_OCL_PROFILING", "0"))
        self.context = Simulator.some_context if context is None else context
        self.profiling = profiling
        self.queue = CommandQueue(self.context, profiling=bool(profiling))
        if if_python_code not in ["none", "warn", "error"]:
            raise ValueError("%r not a valid value for `if_python_code`" % if_python_code)
        self.if_python_code = if_python_code
        self.n_prealloc_probes = n_prealloc_probes
        self.progress_bar = progress_bar
        self.fuse = fuse
        self._planner = planner
        self.stream_inputs = stream_inputs
        self._input_streams = []
        self.h2d_bytes_per_step = 0

        # --- model
        if model is None:
            model = self._build_with_nengo(network, dt)
        elif network is not None:
            model.build(network)
        self.model = model

        # --- operators: simplify, merge dot products, group
        all_operators = list(self.model.operators)
        operators = simplify_operators(all_operators)
        operators = list(map(MultiDotInc.convert_to, operators))
        operators = MultiDotInc.compress(operators)
        op_groups = planner(operators)
        assert len([typ for typ, _ in op_groups if typ.__name__ == "Reset"]) < 2, "All resets not planned together"
        self.operators = operators
        self.op_groups = op_groups

        # --- signals: every dense base in one ragged array, views appended
        all_signals = stable_unique(sig for op in all_operators for sig in op.all_signals)
        all_signals += [self.model.sig[p]["in"] for p in self.model.probes
                        if self.model.sig[p]["in"] not in set(all_signals)]
        # sparse signals stay on the host as matrices (reference simulator.py:281-329): each
        # sparse product uploads its own device form
        sparse_signals = [s for s in all_signals if getattr(s, "sparse", False)]
        if any(s.is_view for s in sparse_signals):
            raise NotImplementedError("Sparse signal views not yet supported")
        all_signals = [s for s in all_signals if not getattr(s, "sparse", False)]
        all_bases = stable_unique(sig.base for sig in all_signals)
        sigdict = {}
        for op in all_operators:
            op.init_signals(sigdict)
        for base in all_bases:
            if base not in sigdict:
                sigdict[base] = np.array(base.initial_value, dtype=np.float64)
        self.sparse_data = {}
        if sparse_signals:
            from nengo_ocl_b200.cura_spmv import HostSparseMatrix

            self.sparse_data = {s: HostSparseMatrix(s.initial_value) for s in stable_unique(sparse_signals)}
        self.base_reshapes = {}
        dense = []
        for base in all_bases:
            x = np.asarray(sigdict[base])
            if x.ndim > 2:
                self.base_reshapes[base] = x.shape
                x = x.reshape(-1, 1)
            dense.append(x)
        dense_data = RaggedArray(dense, names=[getattr(sb, "name", "") for sb in all_bases], dtype=np.float32,
                                 align=True)
        view_builder = ViewBuilder(all_bases, dense_data)
        view_builder.setup_views(operators)
        for probe in self.model.probes:
            view_builder.append_view(self.model.sig[probe]["in"])
        view_builder.add_views_to(dense_data)
        self.all_bases = all_bases
        self.sidx = {k: np.int32(v) for k, v in view_builder.sidx.items()}
        self._A_views = view_builder._A_views
        self._X_views = view_builder._X_views
        self._YYB_views = view_builder._YYB_views
        self._initial_buf = dense_data.buf.copy()
        self.all_data = CUDARaggedArray(self.queue, dense_data)
        self._probe_outputs = dict(getattr(self.model, "params", {}))
        self.data = SimulationData(self._probe_outputs)

        if seed is None:
            net_seed = getattr(network, "seed", None) if network is not None else getattr(self.model, "seed", None)
            seed = net_seed + 1 if net_seed is not None else np.random.randint(2 ** 31 - 1)
        self.seed = seed
        self.rng = np.random.RandomState(self.seed)

        # --- plans
        self._raggedarrays_to_reset = {}
        self._python_rngs = {}
        self._device_state_to_reset = []
        self.fused_groups = []
        # multi-GPU: the exchange buffers exist before planning, so that a compute kernel can take
        # the push of its own results
        self._exchange = None
        self._exchange_start = None
        if exchange is not None:
            from nengo_ocl_b200.exchange import Exchange

            sig, comm = exchange
            assert sig.size % comm.world == 0 and not sig.is_view
            self._exchange_start = int(self.all_data.starts[self.sidx[sig]])
            self._exchange = Exchange(self.queue, comm, self.all_data.cl_buf.data + 4 * self._exchange_start,
                                      sig.size // comm.world)
        plans = []
        groups = list(op_groups)
        if self.fuse:
            from nengo_ocl_b200.fusion import fuse_ensemble_groups

            groups = fuse_ensemble_groups(self, groups)
        for op_type, op_list in groups:
            group_plans = self._plan_op_group(op_type, op_list)
            use = self._signal_use(op_list)
            for plan in group_plans:  # (every plan of a group is charged with the whole group's signals)
                plan.signal_use = use
            plans.extend(group_plans)
        probe_plans = self._plan_probes()
        for plan in probe_plans:  # reads the probed signals; the rings and counters are its own
            plan.signal_use = ({self.model.sig[p]["in"].base for p in self.model.probes}, {plan})
        plans.extend(probe_plans)
        if self._exchange is not None:
            wait, push = self._exchange.plans()
            # What the exchange kernels touch, for the dependency edges of the captured graph: the
            # replica of the exchange signal and the exchange's control block (step counter, flags),
            # which the wait, the push and a compute kernel that pushes its own results all use.
            sig_base, control = exchange[0].base, self._exchange
            for p in wait:
                p.signal_use = ({control}, {sig_base, control})
            for p in push:
                p.signal_use = ({sig_base, control}, {control})
            for p in plans:
                if getattr(p, "fused_push", False):
                    p.signal_use = (set(p.signal_use[0]) | {control}, set(p.signal_use[1]) | {control})
            plans = wait + plans + push
        # A model whose whole step is a handful of blocks runs n steps as ONE launch of a single-CTA
        # persistent kernel (csrc/nb2_step_loop_single.cu); the others replay a captured graph.
        # step_loop: None = that rule, True = always use the loop where every plan has a phase form
        # ("single": on one CTA whatever the size), False = never.  NENGO_B200_STEP_LOOP=0 / 1 overrides the default.
        if step_loop is None:
            step_loop = {"0": False, "1": True}.get(os.environ.get("NENGO_B200_STEP_LOOP", ""), "auto")
        if self._exchange is not None or stream_inputs:
            step_loop = False
        self._plans = Plans(plans, self.profiling, unroll=graph_unroll, step_loop=step_loop,
                            group_tiny=os.environ.get("NENGO_B200_GROUP_TINY", "1") != "0",
                            parallel=os.environ.get("NENGO_B200_PARALLEL_GRAPH", "1") != "0",
                            max_ctas=1 if step_loop == "single" else int(os.environ.get("NENGO_B200_STEP_LOOP_CTAS", "0")))
        self._status_plans = [p for p in plans if getattr(p, "status", None) is not None]
        self.rng = None
        self._n_steps = 0
        self._time = 0.0
        self._reset_probes()
        if self._exchange is not None:
            # every rank has planned and uploaded before any rank starts to wait on a peer
            self.queue.finish()
            self._exchange.comm.barrier()

    @staticmethod
    def _build_with_nengo(network, dt):
        try:
            import nengo  # noqa: F401
            from nengo.builder import Model as NengoModel
        except ImportError as e:
            raise ImportError(
                "building from a nengo Network needs the nengo package; pass "
                "`model=` (a nengo_ocl_b200.model.Model) instead") from e
        model = NengoModel(dt=float(dt), label="%s, dt=%f" % (network, dt))
        if network is not None:
            model.build(network)
        return model

    def __del__(self):
        if not getattr(self, "closed", True):
            warnings.warn("Simulator with model=%s was deallocated while open. Please close simulators "
                          "manually to ensure resources are properly freed." % self.model, ResourceWarning)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()

    def __getitem__(self, item):
        """Internally shaped (always 2-D) value of a signal."""
        return self.all_data[self.sidx[item]]

    def __getstate__(self):
        raise NotImplementedError("this simulator does not support pickling")

    def __setstate__(self, state):
        raise NotImplementedError("this simulator does not support pickling")

    @property
    def dt(self):
        return self.model.dt

    @dt.setter
    def dt(self, dummy):
        raise ReadonlyError("dt is read-only")

    @property
    def n_steps(self):
        return self._n_steps

    @property
    def time(self):
        return self._time

    @property
    def signals(self):
        """Get/set properly shaped signal values (0-d, 1-d or 2-d)."""
        sim = self

        class Accessor(Mapping):
            def __iter__(_):
                return iter(sim.all_bases)

            def __len__(_):
                return len(sim.all_bases)

            def __getitem__(_, item):
                if getattr(item, "sparse", False):  # kept on the host, constant
                    return sim.sparse_data[item].matrix
                raw = sim.all_data[sim.sidx[item]]
                if item.ndim == 0:
                    return raw[0, 0]
                if item.ndim == 1:
                    return raw.ravel()
                if item.ndim == 2:
                    return raw
                raise NotImplementedError()

            def __setitem__(_, item, val):
                incoming = np.asarray(val)
                if item.ndim == 0:
                    assert incoming.size == 1
                    sim.all_data[sim.sidx[item]] = incoming
                elif item.ndim == 1:
                    assert (item.size,) == incoming.shape
                    sim.all_data[sim.sidx[item]] = incoming[:, None]
                elif item.ndim == 2:
                    assert item.shape == incoming.shape
                    sim.all_data[sim.sidx[item]] = incoming
                else:
                    raise NotImplementedError()

            def __str__(self_):
                sio = StringIO()
                for k in self_:
                    print(k, self_[k], file=sio)
                return sio.getvalue()

        return Accessor()

    # --- simulation control ---------------------------------------------------
    def clear_probes(self):
        for probe in self.model.probes:
            self._probe_outputs[probe] = []
        self.data.reset()

    def close(self):
        self.closed = True
        if getattr(self, "_exchange", None) is not None:
            self._exchange.close()
        for st in getattr(self, "_input_streams", []):
            _capi.lib().nb2_host_free(st["hptr"])
        self._input_streams = []
        if getattr(self, "_plans", None) is not None:
            self._plans.close()  # the step loop, grouped launches and side streams of the captured graph
        self.context = None
        self.queue = None
        self.all_data = None
        self._plans = None
        self._raggedarrays_to_reset = None
        self._cl_probe_plan = None

    def _probe(self, steps_run=None):
        """Drain the device-side probe ring buffers into ``data``.  ``steps_run``: the steps simulated
        since the last drain, when the caller knows them (``run_steps``): the step count and the time
        are then advanced on the host exactly as the clock kernel computes them (float32 step,
        ``float32(dt * step)``) instead of being read back."""
        if steps_run is None:
            self._probe_step_time()
        else:
            self._n_steps += int(steps_run)
            self._time = float(np.float32(float(self.model.dt) * float(np.float32(self._n_steps))))
        plan = self._cl_probe_plan
        if plan is None:
            return
        bufpositions = plan.cl_bufpositions.get()  # (a blocking copy on the stream: everything before it is done)
        for i, probe in enumerate(self.model.probes):
            n_buffered = int(bufpositions[i])
            if n_buffered:
                shape = self.model.sig[probe]["in"].shape
                width = int(plan.Y.shape1s[i])
                raw = plan.Y.cl_buf.read_region(int(plan.Y.starts[i]), n_buffered * width)
                self._probe_outputs[probe].extend(raw.reshape((n_buffered,) + tuple(shape)))
        # (a memset on the stream, ordered before the next step: no need to wait for it)
        _capi.call("nb2_memset", plan.cl_bufpositions.ptr, 0, plan.cl_bufpositions.nbytes, self.queue.stream)

    def _probe_step_time(self):
        self._n_steps = int(self.signals[self.model.step].item())
        self._time = float(self.signals[self.model.time].item())

    def _reset_probes(self):
        if self._cl_probe_plan is not None:
            self._cl_probe_plan.cl_bufpositions.fill(0)
            self._cl_probe_plan.cl_countdowns.set(self._cl_probe_plan.periods - 1)
        for probe in self.model.probes:
            self._probe_outputs[probe] = []
        self.data.reset()
        self._probe_step_time()

    def reset(self, seed=None):
        if self.closed:
            raise SimulatorClosed("Cannot reset closed Simulator.")
        if seed is not None:
            raise NotImplementedError("Seed changing not implemented")
        # one upload restores every signal (readonly ones are unchanged by construction)
        self.all_data.cl_buf.set(self._initial_buf)
        for clra, ra in self._raggedarrays_to_reset.items():
            clra.cl_buf.set(ra.buf)
        for darray, host in self._device_state_to_reset:
            darray.set(host)
        for rng, state in self._python_rngs.items():
            rng.set_state(state)
        if self._exchange is not None:
            self._exchange.reset()
        self._reset_probes()

    def run(self, time_in_seconds, progress_bar=None):
        if time_in_seconds < 0:
            raise ValidationError("Must be positive (got %g)" % (time_in_seconds,))
        steps = int(np.round(float(time_in_seconds) / self.dt))
        if steps == 0:
            warnings.warn("%g results in running for 0 timesteps. Simulator still at time %g."
                          % (time_in_seconds, self.time))
        else:
            self.run_steps(steps, progress_bar=progress_bar)

    def run_steps(self, steps, progress_bar=True):
        if self.closed:
            raise SimulatorClosed("Simulator cannot run because it is closed.")
        if self.n_steps + steps >= 2 ** 24:
            raise ValueError("Cannot handle more than 2**24 steps")  # step is a float32 signal
        if steps < 0:
            raise ValueError("Cannot run for negative steps (got %r)" % (steps,))
        while steps > 0:
            B = min(steps, self._max_steps_between_probes)
            self._upload_inputs(B)
            self._plans.call_n_times(B)
            self._probe(steps_run=B)
            self._plans.check_status()
            for plan in self._status_plans:  # bounded waits inside the pipelined kernels
                if int(plan.status.get()[0]) != 0:
                    raise RuntimeError("kernel %s gave up a bounded wait (NB2_ERR_TIMEOUT)" % plan.name)
            if self._exchange is not None and self._exchange.status() != 0:
                raise RuntimeError("multi-GPU exchange: a peer did not publish its step within %.1f s"
                                   % self._exchange.timeout_s)
            steps -= B
        if self.profiling > 1:
            self.print_profiling()

    def step(self):
        return self.run_steps(1, progress_bar=False)

    def trange(self, sample_every=None, dt=None):
        if dt is not None:
            if sample_every is not None:
                raise ValidationError("Cannot specify both `dt` and `sample_every`.")
            warnings.warn("`dt` is deprecated. Use `sample_every` instead.", DeprecationWarning)
            sample_every = dt
        period = 1 if sample_every is None else sample_every / self.dt
        steps = np.arange(1, self.n_steps + 1)
        return self.dt * steps[steps % period < 1]

    # --- planning ---------------------------------------------------------------
    def _plan_probes(self):
        """One plan that samples every probe into a device ring of ``n_prealloc_probes`` rows; the
        host drains the rings every ``_max_steps_between_probes`` steps (the slowest ring to fill
        decides; reference simulator.py:705-731)."""
        probes = self.model.probes
        self._cl_probe_plan = None
        self._max_steps_between_probes = self.n_prealloc_probes
        if not probes:
            return []
        targets = [self.model.sig[p]["in"] for p in probes]
        periods = [max(1 if p.sample_every is None else p.sample_every / self.dt, 1) for p in probes]
        rings = self.RaggedArray([np.zeros((self.n_prealloc_probes, sig.size)) for sig in targets], dtype=np.float32)
        self._cl_probe_plan = plan_probes(self.queue, periods, self._items(targets), rings)
        self._max_steps_between_probes = self.n_prealloc_probes * int(min(periods))
        assert self._max_steps_between_probes >= 1
        return [self._cl_probe_plan]

    @staticmethod
    def _signal_use(ops):
        """(base signals read, base signals written) by a group of operators."""
        reads, writes = set(), set()
        for op in ops:
            reads.update(s.base for s in list(op.reads) + list(op.incs) + list(op.updates))
            writes.update(s.base for s in list(op.sets) + list(op.incs) + list(op.updates))
            for s in getattr(op, "internal", ()):  # signals a fused kernel may still store
                writes.add(s.base)
        return reads, writes

    def _plan_op_group(self, op_type, ops):
        return getattr(self, "_plan_" + op_type.__name__)(ops)

    def _plan_SimProbe(self, ops):
        return []

    def _plan_FusedEnsembles(self, groups):
        from nengo_ocl_b200.fusion import plan_fused_ensembles

        return plan_fused_ensembles(self, groups)

    def _plan_GatherSum(self, ops):
        from nengo_ocl_b200.fusion import plan_gather_sums

        return plan_gather_sums(self, ops)

    def _plan_MultiDotInc(self, ops):
        constant_bs = [op for op in ops if op._float_beta is not None]
        vector_bs = [op for op in ops if op._signal_beta is not None and op._signal_beta.ndim == 1]
        if len(constant_bs) + len(vector_bs) != len(ops):
            raise NotImplementedError()
        if vector_bs:
            raise NotImplementedError("signal-valued beta")
        # one plan per (beta, gamma) pair, so that the kernels get scalar scales
        plans = []
        for scales in stable_unique((op._float_beta, op.gamma) for op in constant_bs):
            same = [op for op in constant_bs if (op._float_beta, op.gamma) == scales]
            plans += self._sig_gemv(
                same, lambda op: self._A_views[op], lambda op: self._X_views[op],
                lambda op: self._YYB_views[op][0], lambda op: self._YYB_views[op][1],
                beta=scales[0], gamma=scales[1], tag="c-beta-%d" % len(same))
        return plans

    def _sig_gemv(self, ops, A_js_fn, X_js_fn, Y_fn, Y_in_fn=None, alpha=1.0, beta=1.0, gamma=0.0, tag=None):
        if len(ops) == 0:
            return []
        all_data, sidx = self.all_data, self.sidx
        A_js = RaggedArray([[sidx[ss] for ss in A_js_fn(op)] for op in ops], dtype=np.int32)
        X_js = RaggedArray([[sidx[ss] for ss in X_js_fn(op)] for op in ops], dtype=np.int32)
        Y_sigs = [Y_fn(item) for item in ops]
        Y_in_sigs = [Y_in_fn(item) for item in ops] if Y_in_fn else Y_sigs
        Y = all_data[[sidx[sig] for sig in Y_sigs]]
        Y_in = all_data[[sidx[sig] for sig in Y_in_sigs]]
        rval = plan_block_gemv(self.queue, alpha, all_data, A_js, all_data, X_js, beta, Y, Y_in=Y_in, gamma=gamma,
                               tag=tag)
        return rval.plans

    def _plan_TimeUpdate(self, ops):
        assert len(ops) == 1, "a model has one clock"
        step, time = self._gather(ops, "step", "time")
        return [plan_timeupdate(self.queue, step, time, self.model.dt)]

    def _plan_Reset(self, ops):
        return [plan_reset(self.queue, self._gather(ops, "dst"), self.Array([op.value for op in ops]))]

    def _plan_Copy(self, ops):
        """Whole-signal copies go to ``plan_copy``; copies with a slice on either side to
        ``plan_slicedcopy`` with explicit element index lists (reference simulator.py:829-869)."""
        def element_indices(sig, sl):
            idx = np.arange(sig.size, dtype=np.int32)
            return idx if sl is None else idx[sl]

        whole = [op for op in ops if op.src_slice is None and op.dst_slice is None]
        sliced = [op for op in ops if op not in whole]
        plans = []
        for group, planner in ((whole, plan_copy), (sliced, plan_slicedcopy)):
            if not group:
                continue
            X, Y = self._gather(group, "src", "dst")
            incs = np.array([op.inc for op in group], dtype=np.int32)
            if planner is plan_copy:
                plans.append(plan_copy(self.queue, X, Y, incs))
                continue
            index_lists = [[element_indices(op.src, op.src_slice) for op in group],
                           [element_indices(op.dst, op.dst_slice) for op in group]]
            for idx in index_lists[0] + index_lists[1]:
                if len(np.unique(idx)) != len(idx):
                    raise NotImplementedError("Duplicates in indices")
            Xinds, Yinds = (self.RaggedArray(lists, dtype=np.int32) for lists in index_lists)
            plans.append(plan_slicedcopy(self.queue, X, Y, Xinds, Yinds, incs))
        return plans

    def _plan_SparseDotInc(self, ops):
        """One plan per sparse product (reference simulator.py:877-892); the algorithm is
        chosen by ``plan_sparse_dot_inc`` (environment variable ``NENGO_OCL_SPMV_ALGORITHM``
        or the footprint heuristic).  The product increments its target, as the operator
        says; the reference plans it in "set" mode, which gives the same values whenever the
        target was reset in the same step and this is the only product into it."""
        from nengo_ocl_b200.cura_spmv import plan_sparse_dot_inc

        plans = []
        for op in ops:
            A = self.sparse_data[op.A]
            X = self.all_data[[self.sidx[op.X]]]
            Y = self.all_data[[self.sidx[op.Y]]]
            plans += plan_sparse_dot_inc(self.queue, A, X, Y, inc=True, tag=op.tag).plans
        return plans

    def _plan_ElementwiseInc(self, ops):
        return [plan_elementwise_inc(self.queue, *self._gather(ops, "A", "X", "Y"))]

    # ---- python functions ---------------------------------------------------
    def _plan_SimPyFunc(self, ops):
        plans = []
        for fn, group in groupby(ops, lambda op: op.fn):
            plans.extend(self._plan_python_fn(fn, ts=[op.t for op in group], xs=[op.x for op in group],
                                              ys=[op.output for op in group]))
        return plans

    def _plan_python_fn(self, fn, ts, xs, ys):
        assert len(ts) == len(xs) == len(ys)
        assert all(t is None for t in ts) or all(t is not None for t in ts)
        assert all(x is None for x in xs) or all(x is not None for x in xs)
        assert all(y is None for y in ys) or all(y is not None for y in ys)
        if ts[0] is not None:
            assert all(t is self.model.time for t in ts)
        size = lambda sig: sig.size if sig is not None else None
        fn_name = getattr(fn, "__name__", type(fn).__name__)
        plans, unplanned = [], []
        for _, group in groupby(zip(ts, xs, ys), lambda s: size(s[1])):
            tt, xx, yy = zip(*group)
            if size(yy[0]) is None:
                self._found_python_code("Function %r could not be converted for the device since it has "
                                        "no outputs." % fn_name)
                unplanned.extend(zip(tt, xx, yy))
                continue
            if self.if_python_code == "error":
                plans.append(self._plan_fn_on_device(fn, tt, xx, yy, fn_name))
            else:
                try:
                    plans.append(self._plan_fn_on_device(fn, tt, xx, yy, fn_name))
                except Exception as e:  # pylint: disable=broad-except
                    self._found_python_code("Function %r could not be converted for the device due to %s%s"
                                            % (fn_name, type(e).__name__, e.args))
                    unplanned.extend(zip(tt, xx, yy))
        if unplanned:
            tt, xx, yy = zip(*unplanned)
            plans.append(self._plan_fn_in_python(fn, tt, xx, yy, fn_name))
        return plans

    def _found_python_code(self, message):
        if self.if_python_code == "error":
            raise RuntimeError(message)
        if self.if_python_code == "warn":
            warnings.warn(message, RuntimeWarning)

    def _plan_fn_on_device(self, fn, tt, xx, yy, fn_name):
        t_in = tt[0] is not None
        x_in = xx[0] is not None
        x_dim = xx[0].size if x_in else None
        y_dim = yy[0].size
        assert all(y.size == y_dim and y.ndim == 1 for y in yy)
        if x_in:
            assert all(x.size == x_dim and x.ndim == 1 for x in xx)
        in_dims = ([1] if t_in else []) + ([x_dim] if x_in else [])
        dev_fn = DeviceFunction(fn, in_dims=in_dims, out_dim=y_dim)
        inputs = []
        if t_in:
            inputs.append(self.all_data[[self.sidx[t] for t in tt]])
        if x_in:
            inputs.append(self.all_data[[self.sidx[x] for x in xx]])
        output = self.all_data[[self.sidx[y] for y in yy]]
        return plan_direct(self.queue, dev_fn.code, dev_fn.init, dev_fn.translator.arg_names[:len(inputs)], inputs,
                           output, tag=fn_name)

    def _plan_fn_in_python(self, fn, tt, xx, yy, fn_name):
        t_in = tt[0] is not None
        t_idx = self.sidx[self.model.time]
        ix_iy = [(self.sidx[x] if x is not None else None, self.sidx[y] if y is not None else None)
                 for x, y in zip(xx, yy)]
        m2v = lambda x: x[:, 0] if x.ndim == 2 and x.shape[1] == 1 else x
        v2m = lambda x: x[:, None] if x.ndim == 1 else x

        def step():
            t = float(self.all_data[t_idx][0, 0] if t_in else 0)
            for ix, iy in ix_iy:
                args = [t] if t_in else []
                args += [m2v(self.all_data[ix])] if ix is not None else []
                y = fn(*args)
                if iy is not None:
                    self.all_data[iy] = v2m(np.asarray(y, dtype=np.float32))

        return PythonPlan(step, name="python_fn", tag=fn_name)

    # ---- neurons ----------------------------------------------------------------
    def _plan_SimNeurons(self, all_ops):
        plans = []
        for neuron_class, ops in groupby(all_ops, lambda op: op.neurons.__class__):
            attr_name = "_plan_%s" % neuron_class.__name__
            if not hasattr(self, attr_name):
                raise ValueError("Unsupported neuron type '%s'" % neuron_class.__name__)
            plans.extend(getattr(self, attr_name)(ops))
        return plans

    def _items(self, signals):
        """Device view (sharing the packed buffer) of the ragged items of ``signals``."""
        return self.all_data[[self.sidx[sig] for sig in signals]]

    def _gather(self, ops, *names):
        """One device view per name: ``op.<name>`` over ``ops``.  A name with a dot is looked up in
        the operator's state dictionary (``"state.voltage"``)."""
        def pick(op, name):
            if name.startswith("state."):
                return op.state[name[6:]]
            return getattr(op, name)

        views = [self._items([pick(op, name) for op in ops]) for name in names]
        return views[0] if len(views) == 1 else views

    def _sigs(self, ops, fn):
        return self._items([fn(op) for op in ops])

    def _scaled_rates(self, ops):
        """learning_rate * dt of every operator, as a device vector."""
        return self.Array([op.learning_rate * self.model.dt for op in ops])

    def _param(self, ops, fn):
        """A python float when all ops agree, else a per-neuron ragged array
        (what the reference always builds, simulator.py:1054-1063)."""
        values = [float(fn(op)) for op in ops]
        if len(set(values)) == 1:
            return values[0]
        return self.RaggedArray([v * np.ones(op.J.size) for v, op in zip(values, ops)], dtype=np.float32)

    # neuron type -> (plan function, takes dt, signal arguments, parameter arguments, keyword signals,
    # keyword parameters); parameters become a python float when all operators agree, else a
    # per-neuron ragged array (what the reference always builds, simulator.py:1054-1063)
    _NEURON_PLANS = {
        "LIF": (plan_lif, True, ("J", "state.voltage", "state.refractory_time", "output"),
                ("tau_ref", "tau_rc", "amplitude"), {}, {}),
        "LIFRate": (plan_lif_rate, True, ("J", "output"), ("tau_ref", "tau_rc", "amplitude"), {}, {}),
        "AdaptiveLIF": (plan_lif, True, ("J", "state.voltage", "state.refractory_time", "output"),
                        ("tau_ref", "tau_rc", "amplitude"), {"N": "state.adaptation"},
                        {"tau_n": "tau_n", "inc_n": "inc_n"}),
        "AdaptiveLIFRate": (plan_lif_rate, True, ("J", "output"), ("tau_ref", "tau_rc", "amplitude"),
                            {"N": "state.adaptation"}, {"tau_n": "tau_n", "inc_n": "inc_n"}),
        "Sigmoid": (plan_sigmoid, False, ("J", "output"), ("tau_ref",), {}, {}),
    }

    def _plan_from_table(self, kind, ops):
        planner, with_dt, sig_names, param_names, kw_sigs, kw_params = self._NEURON_PLANS[kind]
        neuron_param = lambda name: self._param(ops, lambda op: getattr(op.neurons, name))
        views = self._gather(ops, *sig_names)
        args = ([self.model.dt] if with_dt else []) + list(views) + [neuron_param(n) for n in param_names]
        kwargs = {k: self._gather(ops, v) for k, v in kw_sigs.items()}
        kwargs.update({k: neuron_param(v) for k, v in kw_params.items()})
        return [planner(self.queue, *args, **kwargs)]

    def _plan_LIF(self, ops):
        if any(op.neurons.min_voltage != 0 for op in ops):
            raise NotImplementedError("LIF min voltage")
        return self._plan_from_table("LIF", ops)

    def _plan_LIFRate(self, ops):
        return self._plan_from_table("LIFRate", ops)

    def _plan_AdaptiveLIF(self, ops):
        return self._plan_from_table("AdaptiveLIF", ops)

    def _plan_AdaptiveLIFRate(self, ops):
        return self._plan_from_table("AdaptiveLIFRate", ops)

    def _plan_Sigmoid(self, ops):
        return self._plan_from_table("Sigmoid", ops)

    def _amplitudes(self, ops):
        return self.RaggedArray([op.neurons.amplitude * np.ones(op.J.size) for op in ops], dtype=np.float32)

    def _plan_RectifiedLinear(self, ops):
        J, out = self._gather(ops, "J", "output")
        return [plan_rectified_linear(self.queue, J, out, self._amplitudes(ops))]

    def _plan_SpikingRectifiedLinear(self, ops):
        J, V, out = self._gather(ops, "J", "state.voltage", "output")
        return [plan_spiking_rectified_linear(self.queue, self.model.dt, J, V, out, self._amplitudes(ops))]

    # ---- processes --------------------------------------------------------------
    def _plan_SimProcess(self, all_ops):
        plan_groups = defaultdict(list)
        python_ops = []
        for process_class, ops in groupby(all_ops, lambda op: type(op.process)):
            for cls in process_class.__mro__:
                attrname = "_plan_" + cls.__name__
                if hasattr(self, attrname):
                    plan_groups[attrname].extend(ops)
                    break
            else:
                python_ops.extend(ops)
        plans = [p for attr, ops in plan_groups.items() for p in getattr(self, attr)(ops)]
        plans += [p for op in python_ops for p in self._plan_python_process(op)]
        return plans

    def _plan_python_process(self, op):
        shape = lambda s: s.shape if s is not None else (0,)
        rng = op.process.get_rng(self.rng)
        state = op.process.make_state(shape(op.input), shape(op.output), self.model.dt, dtype=None)
        fn = op.process.make_step(shape(op.input), shape(op.output), self.model.dt, rng=rng, state=state)
        plans = self._plan_python_fn(fn, [op.t], [op.input], [op.output])
        self._python_rngs[rng] = rng.get_state()
        return plans

    def linear_filter_coefficients(self, op):
        """(num, den[1:]) of the discrete filter of a LinearFilter process op."""
        proc = op.process
        if hasattr(proc, "discrete_tf"):
            return proc.discrete_tf(self.model.dt)
        # a nengo LinearFilter: discretise through its own make_step (state space -> tf)
        from scipy.signal import ss2tf

        state = proc.make_state(op.input.shape, op.output.shape, self.model.dt, dtype=None)
        f = proc.make_step(op.input.shape, op.output.shape, self.model.dt, rng=None, state=state)
        if f.A.size == 0:
            num, den = np.asarray(f.D).flatten(), np.array([1.0])
        else:
            num, den = ss2tf(f.A, f.B, f.C, f.D)
            num = num.flatten()
        if den[0] != 1.0:
            raise ValidationError("First element of the denominator must be 1")
        return (num[1:] if num[0] == 0 else num), den[1:]

    def _plan_LinearFilter(self, ops):
        if any(op.mode != "update" and op.mode != "set" for op in ops):
            raise NotImplementedError("LinearFilter in 'inc' mode")
        nums, dens = zip(*(self.linear_filter_coefficients(op) for op in ops))
        A = self.RaggedArray(dens, dtype=np.float32)
        B = self.RaggedArray(nums, dtype=np.float32)
        X = self.all_data[[self.sidx[op.input] for op in ops]]
        Y = self.all_data[[self.sidx[op.output] for op in ops]]
        Xbuf0 = RaggedArray([np.zeros(shape) for shape in zip(B.sizes, X.sizes)], dtype=np.float32)
        Ybuf0 = RaggedArray([np.zeros(shape) for shape in zip(A.sizes, Y.sizes)], dtype=np.float32)
        Xbuf = CUDARaggedArray(self.queue, Xbuf0)
        Ybuf = CUDARaggedArray(self.queue, Ybuf0)
        self._raggedarrays_to_reset[Xbuf] = Xbuf0
        self._raggedarrays_to_reset[Ybuf] = Ybuf0
        plans = plan_linearfilter(self.queue, X, Y, A, B, Xbuf, Ybuf)
        for p in plans:
            if getattr(p, "Xbufpos", None) is not None and p.Xbufpos.size:
                self._device_state_to_reset.append((p.Xbufpos, np.zeros(p.Xbufpos.size, np.int32)))
                self._device_state_to_reset.append((p.Ybufpos, np.zeros(p.Ybufpos.size, np.int32)))
        return plans

    @staticmethod
    def _conv_geometry(conv):
        """(shape_in, shape_out, kernel_shape, strides) of a convolution as a 2-D one: a 1-D
        convolution gets a row dimension of one (reference simulator.py:1298-1313)."""
        assert conv.dimensions in (1, 2)
        shape_in, shape_out = tuple(conv.input_shape), tuple(conv.output_shape)
        kernel_shape, strides = tuple(conv.kernel_size), tuple(conv.strides)
        if conv.dimensions == 1:
            assert len(shape_in) == len(shape_out) == 2 and len(kernel_shape) == len(strides) == 1
            kernel_shape, strides = (1,) + kernel_shape, (1,) + strides
            if conv.channels_last:
                shape_in, shape_out = (1,) + shape_in, (1,) + shape_out
            else:
                shape_in, shape_out = (shape_in[0], 1, shape_in[1]), (shape_out[0], 1, shape_out[1])
        return shape_in, shape_out, kernel_shape, strides

    def _plan_ConvInc(self, ops):
        """One plan per operator (reference simulator.py:1290-1331); the result is added to Y."""
        from nengo_ocl_b200.cura_nonlinearities import plan_conv2d

        plans = []
        for op in ops:
            shape_in, shape_out, kernel_shape, strides = self._conv_geometry(op.conv)
            padding = op.conv.padding.lower() if isinstance(op.conv.padding, str) else op.conv.padding
            plans.append(plan_conv2d(
                self.queue, X=self.all_data.getitem_device(self.sidx[op.X]),
                Y=self.all_data.getitem_device(self.sidx[op.Y]), filters=self.all_data.getitem_device(self.sidx[op.W]),
                biases=None, shape_in=shape_in, shape_out=shape_out, kernel_shape=kernel_shape, padding=padding,
                strides=strides, channels_last=op.conv.channels_last, conv=True, inc=True))
        return plans

    def _plan_WhiteNoise(self, ops):
        """simulator.py:1245-1258; seeds not given are drawn from the simulator's generator."""
        from nengo_ocl_b200.cura_nonlinearities import create_rngs, get_dist_enums_params, init_rngs, plan_whitenoise

        assert all(op.input is None for op in ops)
        seeds = [op.process.seed if op.process.seed is not None else self.rng.randint(2 ** 31 - 1) for op in ops]
        rngs = create_rngs(self.queue, len(ops))
        init_rngs(self.queue, rngs, seeds)
        Y = self.all_data[[self.sidx[op.output] for op in ops]]
        t = self.all_data[[self.sidx[self.model.step] for _ in ops]]
        scale = to_device(self.queue, np.array([op.process.scale for op in ops], dtype=np.int32))
        inc = to_device(self.queue, np.array([op.mode == "inc" for op in ops], dtype=np.int32))
        enums, params = get_dist_enums_params([op.process.dist for op in ops])
        enums, params = CUDARaggedArray(self.queue, enums), CUDARaggedArray(self.queue, params)
        return [plan_whitenoise(self.queue, Y, enums, params, scale, inc, self.model.dt, rngs, t)]

    def _plan_WhiteSignal(self, ops):
        Y = self.all_data[[self.sidx[op.output] for op in ops]]
        t = self.all_data[[self.sidx[self.model.step] for _ in ops]]
        tables = [np.asarray(op.process.signal).reshape(len(op.process.signal), -1) for op in ops]
        if self.stream_inputs and len({len(tb) for tb in tables}) == 1:
            return [self._plan_streamed_tables(Y, t, tables)]
        signals = self.RaggedArray(tables, dtype=np.float32)
        return [plan_presentinput(self.queue, Y, t, signals, self.model.dt)]

    def _plan_streamed_tables(self, Y, t, tables):
        """Input tables kept in pinned host memory; the device holds a window of
        as many rows as there are steps between two probe drains, refilled from
        the host before every batch of steps (``_upload_inputs``).  All tables
        are column blocks of one (rows x total width) buffer, so a refill is at
        most three contiguous copies."""
        widths = np.array([tb.shape[1] for tb in tables], dtype=np.int64)
        total = int(widths.sum())
        n_table = len(tables[0])
        periods = [max(1 if p.sample_every is None else p.sample_every / self.dt, 1) for p in self.model.probes]
        window = int(self.n_prealloc_probes) * (int(min(periods)) if periods else 1)
        hptr = ctypes.c_void_p()
        _capi.call("nb2_host_alloc", ctypes.byref(hptr), n_table * total * 4)
        host = np.ctypeslib.as_array(ctypes.cast(hptr, ctypes.POINTER(ctypes.c_float)), shape=(n_table, total))
        host[...] = np.concatenate(tables, axis=1)
        dev = DeviceArray(self.queue, (window * total,), np.float32)
        cols = np.concatenate([[0], np.cumsum(widths)[:-1]])
        signals = CUDARaggedArray.from_buffer(self.queue, dev, cols, [window] * len(tables), widths,
                                              [total] * len(tables), [1] * len(tables))
        self._input_streams.append(dict(host=host, hptr=hptr, dev=dev, total=total, n_table=n_table, window=window))
        self.h2d_bytes_per_step += 4 * total
        return plan_presentinput(self.queue, Y, t, signals, self.model.dt)

    def _upload_inputs(self, n_steps):
        """Refill the device windows with the table rows of the next ``n_steps`` steps."""
        for st in self._input_streams:
            first = self._n_steps + 1  # the clock is incremented before the tables are read
            assert n_steps <= st["window"]
            done = 0
            while done < n_steps:
                step = first + done
                src, dst = step % st["n_table"], step % st["window"]
                run = min(n_steps - done, st["n_table"] - src, st["window"] - dst)
                _capi.call("nb2_memcpy_h2d", ctypes.c_void_p(st["dev"].data + dst * st["total"] * 4),
                           ctypes.c_void_p(st["host"].ctypes.data + src * st["total"] * 4), run * st["total"] * 4,
                           self.queue.stream, 0)
                done += run

    def _plan_PresentInput(self, ops):
        ps = [op.process for op in ops]
        Y = self.all_data[[self.sidx[op.output] for op in ops]]
        t = self.all_data[[self.sidx[self.model.step] for _ in ops]]
        inputs = self.RaggedArray([p.inputs.reshape(p.inputs.shape[0], -1) for p in ps], dtype=np.float32)
        pres_t = self.Array([p.presentation_time for p in ps])
        return [plan_presentinput(self.queue, Y, t, inputs, self.model.dt, pres_t=pres_t)]

    # ---- learning rules: every rule produces a delta; a separate Copy(inc) applies it ---------
    def _plan_SimPES(self, ops):
        """delta = alpha * outer(error, pre activities), alpha = -learning_rate * dt / n_pre
        (reference simulator.py:1334-1345)."""
        error, pre, delta = self._gather(ops, "error", "pre_filtered", "delta")
        alpha = np.array([-op.learning_rate * self.model.dt / op.pre_filtered.shape[0] for op in ops])
        return [plan_elementwise_inc(self.queue, error, pre, delta, alpha=alpha, outer=True, inc=False)]

    def _plan_SimBCM(self, ops):
        pre, post, theta, delta = self._gather(ops, "pre_filtered", "post_filtered", "theta", "delta")
        return [plan_bcm(self.queue, pre, post, theta, delta, self._scaled_rates(ops))]

    def _plan_SimOja(self, ops):
        pre, post, weights, delta = self._gather(ops, "pre_filtered", "post_filtered", "weights", "delta")
        return [plan_oja(self.queue, pre, post, weights, delta, self._scaled_rates(ops),
                         self.Array([op.beta for op in ops]))]

    def _plan_SimVoja(self, ops):
        pre, post, encoders, delta, learn = self._gather(ops, "pre_decoded", "post_filtered", "scaled_encoders",
                                                         "delta", "learning_signal")
        scale = self.RaggedArray([np.asarray(op.scale).reshape(-1, 1) for op in ops], dtype=np.float32)
        return [plan_voja(self.queue, pre, post, encoders, delta, learn, scale, self._scaled_rates(ops))]

    def _plan_SimRLS(self, ops):
        raise NotImplementedError("RLS learning rule not yet supported")  # (nor in the reference, :1372)

    # ---- reporting ---------------------------------------------------------------
    def print_plans(self):
        """Every plan of a step with its launch shape and what it works on."""
        print(" Plans ".center(80, "-"))
        for plan in self._plans:
            print(repr(plan))
            description = getattr(plan, "description", None)
            if description:
                print(indent(description, 4))

    def profiling_rows(self):
        """Per plan: calls, seconds on the device, GF/s and GB/s from the plan's own flop and byte
        counts (``flops_per_call`` / ``bw_per_call``, the figures the reference prints too)."""
        rows = []
        for plan in self._plans:
            if not isinstance(plan, BasePlan):
                continue
            seconds = float(sum(plan.ctimes))
            rate = plan.n_calls / seconds if seconds > 0 else float("nan")
            scale = lambda per_call: 1e-9 * per_call * rate if per_call is not None else float("nan")
            rows.append(dict(plan=str(plan), n_calls=plan.n_calls, seconds=seconds,
                             gflops=scale(plan.flops_per_call), gbs=scale(plan.bw_per_call)))
        return rows

    def print_profiling(self, sort=None):
        """Table of calls, device time, GF/s and GB/s per plan (needs ``profiling=True``).
        ``sort``: column to sort by (0 calls, 1 time, 2 GF/s, 3 GB/s; negative = ascending)."""
        if not self.profiling:
            print("Profiling not enabled!")
            return
        rows = self.profiling_rows()
        columns = ("n_calls", "seconds", "gflops", "gbs")
        if sort is not None:
            rows.sort(key=lambda r: r[columns[abs(sort)]], reverse=sort >= 0)
        print(" Profiling ".center(80, "-"))
        print("%8s|%10s|%10s|%10s|" % ("n_calls", "runtime", "GF/s", "GB/s"))
        for r in rows:
            print("%8d|%10.3f|%10.3f|%10.3f| %s" % (r["n_calls"], r["seconds"], r["gflops"], r["gbs"], r["plan"]))
        print("-" * 80)
        total = sum(r["seconds"] for r in rows)

        def time_weighted(col):
            pairs = [(r[col], r["seconds"]) for r in rows if r[col] == r[col]]  # (skip NaN)
            weight = sum(w for _, w in pairs)
            return sum(v * w for v, w in pairs) / weight if weight > 0 else float("nan")

        print("totals:\t%2.3f\t%2.3f\t%2.3f" % (total, time_weighted("gflops"), time_weighted("gbs")))
