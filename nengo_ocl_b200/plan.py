"""Plans: prepared kernel launches, and the step loop that replays them.

API of the reference's ``nengo_ocl/plan.py:12-149`` (``BasePlan``,
``PythonPlan``, ``Plan``, ``Plans`` with ``call_n_times`` /
``enqueue_n_times``), re-designed for CUDA:

* a ``Plan`` wraps a launch closure that issues one or more kernels on the
  queue's stream through the C ABI (the reference wraps a pyopencl kernel and
  ``enqueue_nd_range_kernel``, plan.py:85-91);
* ``Plans.call_n_times(n)`` captures one pass over all device plans into a
  CUDA graph once and replays it (optionally ``unroll`` steps per graph), so
  the per-step cost is one graph launch instead of one Python-issued launch
  per plan per step (plan.py:137-149).  A ``PythonPlan`` in the list splits
  the step into graph segments with a host callback in between;
* profiling brackets every plan with CUDA events on the launching stream and
  fills ``ctimes`` (kernel seconds); ``atimes``/``btimes`` (queue/submit
  latencies in OpenCL) are recorded as 0.
"""

import ctypes
import time

from nengo_ocl_b200 import _capi


class BasePlan:
    def __init__(self, name="", tag=None, flops_per_call=None, bw_per_call=None):
        self.name = name
        self.tag = tag
        self.atimes = []
        self.btimes = []
        self.ctimes = []
        self.n_calls = 0
        self.flops_per_call = flops_per_call
        self.bw_per_call = bw_per_call

    def _label(self):
        return "%s%s" % (self.name, ": %s" % self.tag if self.tag else "")

    def __str__(self):
        return "<%s>" % self._label()

    def __repr__(self):
        return "%s{%s}" % (self.__class__.__name__, self._label())

    def update_profiling(self):
        pass


class PythonPlan(BasePlan):
    """A host callback executed between device plans."""

    def __init__(self, function, **kwargs):
        super().__init__(**kwargs)
        self.function = function

    def __call__(self, profiling=False):
        t0 = time.time() if profiling else 0.0
        self.function()
        if profiling:
            self.atimes.append(0)
            self.btimes.append(0)
            self.ctimes.append(time.time() - t0)
            self.n_calls += 1


class _Event:
    """Completion handle returned by ``Plan.enqueue`` (``wait()`` like a cl.Event)."""

    def __init__(self, queue):
        self.queue = queue

    def wait(self):
        self.queue.finish()


class Plan(BasePlan):
    """A prepared device launch.

    Parameters
    ----------
    queue : CommandQueue
    kern : callable(stream)
        Issues the kernel(s) on ``stream`` via the C ABI.
    gsize, lsize : tuples
        Logical NDRange, kept for parity with the reference's plans.
    n_launches : int
        Kernels issued per call (for launch accounting).
    """

    def __init__(self, queue, kern, gsize, lsize=None, n_launches=1, **kwargs):
        super().__init__(**kwargs)
        self.queue = queue
        self.kern = kern
        self.gsize = self._format_size(gsize)
        self.lsize = self._format_size(lsize) if lsize is not None else None
        self.n_launches = n_launches
        self._events_to_profile = []

    @staticmethod
    def _format_size(size):
        assert size is not None
        size = tuple(int(s) for s in size)
        assert len(size) > 0
        assert all(s > 0 for s in size)
        return size

    def __call__(self, profiling=False):
        self.enqueue(profiling=profiling).wait()

    def enqueue(self, wait_for=None, profiling=False):
        stream = self.queue.stream
        if profiling:
            e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
            _capi.call("nb2_event_create", ctypes.byref(e0))
            _capi.call("nb2_event_create", ctypes.byref(e1))
            _capi.call("nb2_event_record", e0, stream)
            self.kern(stream)
            _capi.call("nb2_event_record", e1, stream)
            self._events_to_profile.append((e0, e1))
        else:
            self.kern(stream)
        return _Event(self.queue)

    def update_profiling(self):
        for e0, e1 in self._events_to_profile:
            _capi.call("nb2_event_sync", e1)
            ms = ctypes.c_float()
            _capi.call("nb2_event_elapsed_ms", e0, e1, ctypes.byref(ms))
            _capi.call("nb2_event_destroy", e0)
            _capi.call("nb2_event_destroy", e1)
            self.atimes.append(0.0)
            self.btimes.append(0.0)
            self.ctimes.append(1e-3 * ms.value)
            self.n_calls += 1
        self._events_to_profile[:] = []

    def __str__(self):
        return "<%s %s %s>" % (self._label(), self.gsize, self.lsize)

    def __repr__(self):
        return "%s{%s %s %s}" % (self.__class__.__name__, self._label(), self.gsize, self.lsize)


class _Graph:
    def __init__(self, handle):
        self.handle = handle

    def __del__(self):
        try:
            _capi.lib().nb2_graph_destroy(ctypes.c_void_p(self.handle))
        except Exception:
            pass


def phase_barriers(uses, ring=True):
    """Where a persistent step loop needs a grid-wide barrier.

    ``uses``: per phase ``(reads, writes)``, two sets of hashable signal keys, in
    step order; the list repeats every step.  Phase p needs a barrier before it
    when it reads or writes something that a phase since the last barrier wrote,
    or writes something one of them read (the phases of the previous step count:
    the list is a ring, unless ``ring=False``: one pass per launch).  Returns one
    bool per phase."""
    uses = [(set(r), set(w)) for r, w in uses]
    flags = [False] * len(uses)
    read_acc, write_acc = set(), set()
    quiet_laps = 0
    # Replay the list exactly as the kernel runs it (a flagged phase clears what has accumulated)
    # and flag every conflict met; for a ring, until two whole laps add nothing.
    while True:
        added = False
        for i, (reads, writes) in enumerate(uses):
            if not flags[i] and (write_acc & (reads | writes) or read_acc & writes):
                flags[i] = added = True
            if flags[i]:
                read_acc, write_acc = set(), set()
            read_acc |= reads
            write_acc |= writes
        quiet_laps = 0 if added else quiet_laps + 1
        if not ring or quiet_laps >= 2:
            break
    return flags


class StepLoop:
    """All plans of a step as phases of one persistent kernel (csrc/nb2_step_loop.cu):
    ``run(stream, n)`` simulates n steps with one launch.  No counterpart in the
    reference, which enqueues every kernel of every step (plan.py:137-149).

    ``max_ctas=1`` selects the single-CTA form (CTA barriers, signals resident in one
    multiprocessor's L1), which is what pays: measured on a B200, it takes the step of a
    two-ensemble model well below the launch-per-plan cost, while the multi-CTA form
    (grid-wide barriers, L2-only loads) is slower than replaying a captured graph for
    models of hundreds of blocks.  ``build(..., auto=True)`` therefore returns a loop only
    for models whose whole step is at most ``AUTO_MAX_BLOCKS`` blocks and whose widest plan is at
    most ``AUTO_MAX_WIDEST`` (a wider plan runs faster as a grid of its own)."""

    AUTO_MAX_BLOCKS = 16   # blocks of a whole step
    AUTO_MAX_WIDEST = 3    # blocks of its widest plan (one CTA walks them one after the other)

    @classmethod
    def build(cls, plans, barriers, max_ctas=0, auto=False):
        loop = cls(plans, barriers)
        if auto:
            widest = max(phase_blocks(p) or 0 for p in plans)
            if loop.total_blocks > cls.AUTO_MAX_BLOCKS or widest > cls.AUTO_MAX_WIDEST:
                loop.close()
                return None
            max_ctas = 1
        loop.finalize(max_ctas)
        return loop

    def __init__(self, plans, barriers):
        handle = ctypes.c_void_p()
        _capi.call("nb2_step_loop_create", ctypes.byref(handle))
        self.handle = handle
        self.grid = 0
        try:
            for plan, barrier in zip(plans, barriers):
                plan.phase(handle, barrier)
            self._info()
        except Exception:
            self.close()
            raise

    def _info(self):
        a, b, c, d = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _capi.call("nb2_step_loop_info", self.handle, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c),
                   ctypes.byref(d))
        self.n_phases, self.n_barriers, self.grid, self.total_blocks = a.value, b.value, c.value, d.value

    def finalize(self, max_ctas=0):
        try:
            _capi.call("nb2_step_loop_finalize", self.handle, int(max_ctas))
            self._info()
        except Exception:
            self.close()
            raise

    def run(self, stream, n):
        _capi.call("nb2_step_loop_run", self.handle, stream, int(n))

    def status(self, stream):
        st = ctypes.c_int()
        _capi.call("nb2_step_loop_status", self.handle, stream, ctypes.byref(st))
        return st.value

    def close(self):
        if self.handle is not None:
            try:
                _capi.lib().nb2_step_loop_destroy(self.handle)
            except Exception:
                pass
            self.handle = None

    def __del__(self):
        self.close()


class PhaseGroup(Plan):
    """Consecutive tiny plans (a clock update, a one-item node function, a few probes ...) as ONE
    launch: the single-CTA step-loop kernel runs them as phases of one pass, with a CTA barrier
    where one depends on another.  Each of them alone is a launch gap with almost no work."""

    def __init__(self, queue, plans):
        self.members = list(plans)
        self.loop = StepLoop(self.members, phase_barriers([p.signal_use for p in self.members], ring=False))
        self.loop.finalize(1)
        loop = self.loop
        Plan.__init__(self, queue, lambda stream: loop.run(stream, 1), (256,), n_launches=1, name="phase_group",
                      tag=" + ".join(p.name for p in self.members))
        self.signal_use = (set().union(*[set(p.signal_use[0]) for p in self.members]),
                           set().union(*[set(p.signal_use[1]) for p in self.members]))


def phase_blocks(plan):
    """Thread blocks of a plan's phase form (None: it has none)."""
    if getattr(plan, "phase", None) is None or getattr(plan, "signal_use", None) is None:
        return None
    if getattr(plan, "_phase_blocks", None) is None:
        probe = StepLoop([plan], [False])
        plan._phase_blocks = probe.total_blocks
        probe.close()
    return plan._phase_blocks


def group_tiny_plans(plans, max_blocks=4):
    """Replace every run of two or more consecutive device plans whose phase forms add up to at
    most ``max_blocks`` thread blocks by one ``PhaseGroup``."""
    out, run, blocks = [], [], 0

    def flush():
        nonlocal run, blocks
        out.extend([PhaseGroup(run[0].queue, run)] if len(run) >= 2 else run)
        run, blocks = [], 0

    for p in plans:
        b = phase_blocks(p) if hasattr(p, "enqueue") else None
        if b is None or b > max_blocks:
            flush()
            out.append(p)
            continue
        if blocks + b > max_blocks:
            flush()
        run.append(p)
        blocks += b
    flush()
    return out


class Plans:
    """Ordered plan list = one simulator step; replays it n times."""

    def __init__(self, planlist, profiling, use_graph=True, unroll=1, step_loop=False, max_ctas=0, group_tiny=False,
                 parallel=False):
        self.plans = list(planlist)
        self.profiling = profiling
        self.use_graph = use_graph
        self.unroll = max(1, int(unroll))
        self._segments = None  # list of ("graph", _Graph, _Graph_unrolled) / ("python", plan)
        self.kernel_launches = 0  # device kernels issued so far (graph nodes count)
        self.group_tiny = bool(group_tiny)
        self.parallel = bool(parallel)  # capture independent plans as parallel graph branches
        self._side_streams = None
        self._launch_plans = None  # what a captured step launches: self.plans with tiny runs grouped
        # persistent step loop (step_loop: False, True or "auto" = only where it pays): needs every
        # plan to have a phase form and to declare the signals it touches
        self.step_loop = None
        if (step_loop and use_graph and not profiling and self.plans
                and all(getattr(p, "phase", None) is not None and getattr(p, "signal_use", None) is not None
                        for p in self.plans)):
            self.step_loop = StepLoop.build(self.plans, phase_barriers([p.signal_use for p in self.plans]),
                                            max_ctas, auto=(step_loop == "auto"))

    def __call__(self):
        return self.call_n_times(1)

    def __len__(self):
        return len(self.plans)

    def __getitem__(self, i):
        return self.plans[i]

    def __iter__(self):
        return iter(self.plans)

    @property
    def queue(self):
        for p in self.plans:
            if hasattr(p, "queue"):
                return p.queue
        return None

    @property
    def launches_per_step(self):
        plans = self.plans if (self.profiling or not self.use_graph) else self.launch_plans()
        return sum(getattr(p, "n_launches", 0) for p in plans)

    def invalidate(self):
        """Drop captured graphs (call after changing the plan list)."""
        self._segments = None
        for p in self._launch_plans or []:
            if isinstance(p, PhaseGroup):
                p.loop.close()
        self._launch_plans = None
        if self.step_loop is not None:
            self.step_loop.close()
            self.step_loop = None

    def close(self):
        """Release the step loop and the side streams of the branch capture."""
        self.invalidate()
        for st in self._side_streams or []:
            try:
                _capi.lib().nb2_stream_destroy(st)
            except Exception:
                pass
        self._side_streams = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check_status(self):
        """Raise if the step loop gave up a bounded barrier wait (synchronises the stream)."""
        if self.step_loop is not None and self.step_loop.status(self.queue.stream) != 0:
            raise RuntimeError("the persistent step loop gave up waiting at a grid barrier (NB2_ERR_TIMEOUT)")

    def call_n_times(self, n):
        self.enqueue_n_times(n)
        q = self.queue
        if q is not None:
            q.finish()
        if self.profiling:
            for p in self.plans:
                p.update_profiling()

    # -- execution ----------------------------------------------------------
    MAX_BRANCH_PLANS = 32  # longer plan lists are captured as one chain
    N_SIDE_STREAMS = 3

    def _capture(self, plans, repeat):
        if (self.parallel and 1 < len(plans) <= self.MAX_BRANCH_PLANS
                and all(getattr(p, "signal_use", None) is not None for p in plans)):
            try:
                return self._capture_branches(plans, repeat)
            except _capi.NB2Error as err:
                # (the capture was aborted: the stream is usable) fall back to the plain in-order graph
                import warnings

                warnings.warn("graph capture along signal dependencies failed (%s); capturing the plans in "
                              "order instead" % err)
                self.parallel = False
        return self._capture_chain(plans, repeat)

    def _capture_branches(self, plans, repeat):
        """Capture ``repeat`` passes over ``plans`` as a graph whose edges are the signal
        dependencies (read-after-write, write-after-write, write-after-read on base signals)
        instead of the plan order: independent plans of a step, and of consecutive steps,
        become parallel branches.  The reference's plans run strictly in order on one queue
        (plan.py:85-91); the values are the same, only launch gaps overlap.  Built by stream
        capture on a few side streams joined with events."""
        q = self.queue
        s0 = q.stream
        if self._side_streams is None:
            self._side_streams = []
            for _ in range(self.N_SIDE_STREAMS):
                st = ctypes.c_void_p()
                _capi.call("nb2_stream_create", ctypes.byref(st))
                self._side_streams.append(st)
        streams = [s0] + self._side_streams
        events = []

        def new_event(stream):
            e = ctypes.c_void_p()
            _capi.call("nb2_event_create", ctypes.byref(e))
            events.append(e)
            _capi.call("nb2_event_record", e, stream)
            return e

        import gc

        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            _capi.call("nb2_graph_begin", s0)
            try:
                fork = new_event(s0)
                joined = {0}   # streams that are part of the capture
                tail = {}      # stream index -> node index of its last launch
                nodes = []     # (reads, writes, stream index, event, weight)
                for _ in range(repeat):
                    for p in plans:
                        reads, writes = set(p.signal_use[0]), set(p.signal_use[1])
                        touched = reads | writes
                        latest = {}  # stream index -> latest node on it that this plan must follow
                        for i, (r, w, si, _e, _w) in enumerate(nodes):
                            if w & touched or r & writes:
                                latest[si] = i
                        # continue a stream whose last launch is a dependency -- the heaviest one, which
                        # finishes last: only the edge inside a stream can be a programmatic one, whose
                        # launch latency overlaps the predecessor; else an unused stream; else the stream
                        # whose last launch is oldest (one needless edge)
                        cands = [si for si, i in latest.items() if tail.get(si) == i]
                        if cands:
                            si = max(cands, key=lambda c: (nodes[latest[c]][4], latest[c]))
                        else:
                            unused = [c for c in range(len(streams)) if c not in tail]
                            si = unused[0] if unused else min(tail, key=tail.get)
                        if si not in joined:
                            _capi.call("nb2_stream_wait_event", streams[si], fork)
                            joined.add(si)
                        for sj, i in latest.items():
                            if sj != si:
                                _capi.call("nb2_stream_wait_event", streams[si], nodes[i][3])
                        p.kern(streams[si])
                        nodes.append((reads, writes, si, new_event(streams[si]), self._weight(p)))
                        tail[si] = len(nodes) - 1
                for si, i in tail.items():  # every branch ends in the origin stream
                    if si != 0:
                        _capi.call("nb2_stream_wait_event", s0, nodes[i][3])
            except Exception:
                _capi.lib().nb2_graph_abort(s0)
                raise
            g = ctypes.c_void_p()
            _capi.call("nb2_graph_end", s0, ctypes.byref(g))
        finally:
            if gc_was_on:
                gc.enable()
            for e in events:
                _capi.lib().nb2_event_destroy(e)
        return _Graph(g.value)

    @staticmethod
    def _weight(plan):
        """Rough size of a plan (thread blocks), to tell the long branch from the short ones."""
        blocks = getattr(plan, "_phase_blocks", None)
        if blocks is None:
            blocks = 1
            for g in getattr(plan, "gsize", (1,)):
                blocks *= int(g)
            blocks = max(1, blocks // 256)
        return blocks

    def _capture_chain(self, plans, repeat):
        q = self.queue
        # No device array may be released while the stream is capturing (a free is not a
        # capturable call): keep the garbage collector out of the way until the capture ends.
        import gc

        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            _capi.call("nb2_graph_begin", q.stream)
            try:
                for _ in range(repeat):
                    for p in plans:
                        p.kern(q.stream)
            except Exception:
                _capi.lib().nb2_graph_abort(q.stream)
                raise
            g = ctypes.c_void_p()
            _capi.call("nb2_graph_end", q.stream, ctypes.byref(g))
        finally:
            if gc_was_on:
                gc.enable()
        return _Graph(g.value)

    def launch_plans(self):
        """The plans a captured step launches (runs of tiny plans grouped into one launch each)."""
        if self._launch_plans is None:
            self._launch_plans = group_tiny_plans(self.plans) if self.group_tiny else list(self.plans)
        return self._launch_plans

    def _build_segments(self):
        segments = []
        run = []
        for p in self.launch_plans():
            if hasattr(p, "enqueue"):
                run.append(p)
            else:
                if run:
                    segments.append(("graph", run))
                    run = []
                segments.append(("python", p))
        if run:
            segments.append(("graph", run))
        built = []
        only_device = len(segments) == 1 and segments[0][0] == "graph"
        for kind, payload in segments:
            if kind == "graph":
                g1 = self._capture(payload, 1)
                gu = self._capture(payload, self.unroll) if (only_device and self.unroll > 1) else None
                built.append(("graph", payload, g1, gu))
            else:
                built.append(("python", payload))
        self._segments = built

    def enqueue_n_times(self, n):
        if n <= 0 or not self.plans:
            return None
        q = self.queue
        if q is None:  # python-only plan list
            for _ in range(n):
                for p in self.plans:
                    p(profiling=self.profiling)
            return None
        if self.profiling or not self.use_graph:
            for _ in range(n):
                for p in self.plans:
                    if hasattr(p, "enqueue"):
                        p.enqueue(profiling=self.profiling)
                    else:
                        q.finish()
                        p(profiling=self.profiling)
            self.kernel_launches += n * self.launches_per_step
            return _Event(q)
        if self.step_loop is not None:
            self.step_loop.run(q.stream, n)
            self.kernel_launches += 1
            return _Event(q)
        if self._segments is None:
            self._build_segments()
        segs = self._segments
        if len(segs) == 1 and segs[0][0] == "graph":
            _, _, g1, gu = segs[0]
            left = n
            if gu is not None and left >= self.unroll:
                _capi.call("nb2_graph_launch", ctypes.c_void_p(gu.handle), q.stream, left // self.unroll)
                left %= self.unroll
            if left:
                _capi.call("nb2_graph_launch", ctypes.c_void_p(g1.handle), q.stream, left)
        else:
            for _ in range(n):
                for seg in segs:
                    if seg[0] == "graph":
                        _capi.call("nb2_graph_launch", ctypes.c_void_p(seg[2].handle), q.stream, 1)
                    else:
                        q.finish()
                        seg[1](profiling=False)
        self.kernel_launches += n * self.launches_per_step
        return _Event(q)
