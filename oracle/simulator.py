"""CPU oracle for whole-model parity: a direct interpreter of an operator list.

TEST INFRASTRUCTURE ONLY (checker for the CUDA simulator; never imported by
the product package).

It does not share the product's planning code: operators are topologically
sorted one by one with the rule sets -> incs -> reads -> updates and executed
with the float32 kernel restatements of ``oracle.kernels``, on plain numpy
arrays (one per base signal).  It therefore also checks the product's operator
merging, grouping and fusion, not only its kernels.  The per-operator
arithmetic follows what the reference launches for that operator type
(nengo_ocl/simulator.py:746-1345): e.g. all ``DotInc`` into one target are
summed first and added to the target once (``MultiDotInc``), a lowpass
``LinearFilter`` is ``y = b0*x - a0*y``, PES writes
``delta = alpha * outer(error, pre)``.  Dot products follow the kernel the
reference simulator plans for every ``MultiDotInc``, ``plan_block_gemv``
(nengo_ocl/simulator.py:803, clra_gemv.py:1018-1058,1137-1153): float32, four
column-strided partial sums per 128-column tile combined as
``(s0 + s2) + (s1 + s3)``, tiles added to the target in order.
"""

import numpy as np

from oracle import cport as C
from oracle import kernels as K

f32 = np.float32


def _toposort(operators):
    """Kahn's algorithm over the per-signal phase order (stable in list order)."""
    by_base = {}
    for i, op in enumerate(operators):
        for phase, kind in enumerate(("sets", "incs", "reads", "updates")):
            for sig in getattr(op, kind):
                by_base.setdefault(sig.base, [[], [], [], []])[phase].append((sig, i))
    succ = [set() for _ in operators]
    npred = [0] * len(operators)
    for phases in by_base.values():
        for pa in range(4):
            for pb in range(pa + 1, 4):
                for sa, ia in phases[pa]:
                    for sb, ib in phases[pb]:
                        if ia != ib and ib not in succ[ia] and sa.may_share_memory(sb):
                            succ[ia].add(ib)
                            npred[ib] += 1
    ready = [i for i, n in enumerate(npred) if n == 0]
    order = []
    import heapq

    heapq.heapify(ready)
    while ready:
        i = heapq.heappop(ready)
        order.append(i)
        for j in succ[i]:
            npred[j] -= 1
            if npred[j] == 0:
                heapq.heappush(ready, j)
    if len(order) != len(operators):
        raise ValueError("cycle in operator graph")
    return [operators[i] for i in order]


class OracleSimulator:
    """Runs ``model`` (nengo_ocl_b200.model.Model-like) step by step on the CPU."""

    def __init__(self, model, dt=None):
        self.model = model
        self.dt = float(model.dt if dt is None else dt)
        self.signals = {}
        for op in model.operators:
            for sig in op.all_signals:
                b = sig.base
                if b not in self.signals:
                    if getattr(b, "sparse", False):
                        self.signals[b] = b.initial_value.astype(np.float32).tocsr()
                    else:
                        self.signals[b] = np.array(b.initial_value, dtype=np.float32, order="C")
        for p in model.probes:
            b = model.sig[p]["in"].base
            if b not in self.signals:
                self.signals[b] = np.array(b.initial_value, dtype=np.float32, order="C")
        ops = list(model.operators)
        # all DotIncs into one target form one multi-term product (MultiDotInc.compress)
        self._dot_groups = {}
        merged = []
        for op in ops:
            if type(op).__name__ == "DotInc":
                key = id(op.Y)
                if key in self._dot_groups:
                    self._dot_groups[key].append(op)
                    continue
                self._dot_groups[key] = [op]
            merged.append(op)
        self._ops = _toposort(self._merge_view(merged))
        self._filter_state = {}
        self._views = {}  # signal -> strided view into its base array (the arrays never move)
        self._prepared = {}  # per-operator constants (2-D operand views, filter coefficients)
        self.probe_data = {p: [] for p in model.probes}
        self.n_steps = 0

    def _merge_view(self, merged):
        """Give a merged DotInc head the reads of its whole group for ordering."""
        out = []
        for op in merged:
            if type(op).__name__ == "DotInc" and len(self._dot_groups[id(op.Y)]) > 1:
                group = self._dot_groups[id(op.Y)]
                proxy = _DotGroup(group)
                out.append(proxy)
            else:
                out.append(op)
        return out

    # -- signal access ---------------------------------------------------------
    def view(self, sig):
        v = self._views.get(sig)
        if v is None:
            base = self.signals[sig.base].reshape(-1)
            isz = base.itemsize
            v = self._views[sig] = np.lib.stride_tricks.as_strided(
                base[sig.elemoffset:], shape=sig.shape, strides=tuple(s * isz for s in sig.elemstrides))
        return v

    def __getitem__(self, sig):
        return np.array(self.view(sig))

    # -- stepping --------------------------------------------------------------
    def run_steps(self, n):
        for _ in range(n):
            self.step()

    def step(self):
        for op in self._ops:
            getattr(self, "_do_" + type(op).__name__)(op)
        self.n_steps += 1
        for p in self.model.probes:
            period = 1 if p.sample_every is None else max(p.sample_every / self.dt, 1)
            # same float countdown rule as the probes kernel
            st = self._filter_state.setdefault(("probe", p), [f32(period - 1)])
            if st[0] <= 0:
                self.probe_data[p].append(self[self.model.sig[p]["in"]])
                st[0] = f32(f32(st[0] + f32(period)) - f32(1))
            else:
                st[0] = f32(st[0] - f32(1))

    # -- operators --------------------------------------------------------------
    def _do_TimeUpdate(self, op):
        s = f32(self.view(op.step)[()] + f32(1))
        self.view(op.step)[...] = s
        self.view(op.time)[...] = f32(self.dt * float(s))

    def _do_Reset(self, op):
        self.view(op.dst)[...] = f32(op.value)

    def _do_Copy(self, op):
        src, dst = self.view(op.src), self.view(op.dst)
        if op.src_slice is not None:
            src = src[op.src_slice]
        if op.dst_slice is not None:
            if op.inc:
                dst[op.dst_slice] = dst[op.dst_slice] + src
            else:
                dst[op.dst_slice] = src
        elif op.inc:
            dst[...] = dst + src
        else:
            dst[...] = src

    @staticmethod
    def _as2d(v):
        return v.reshape(1, 1) if v.ndim == 0 else v.reshape(v.shape[0], 1) if v.ndim == 1 else v

    def _block_inc(self, y_sig, ops):
        """``y += sum_i A_i . x_i`` as one multi-term block GEMV with alpha = beta = 1, gamma = 0
        (MultiDotInc.convert_to / get_views, nengo_ocl/operators.py:50-67,159-191: operands
        become 2-D, a (1, 1) matrix swaps roles with its vector)."""
        y = self.view(y_sig)
        terms = self._prepared.get(id(ops[0]))
        if terms is None:
            terms = []
            for op in ops:
                A, X = self.view(op.A), self.view(op.X)
                X2 = self._as2d(X)
                A2 = A.reshape(1, A.shape[0]) if (A.ndim == 1 and X.ndim == 1) else self._as2d(A)
                if A2.shape == (1, 1):
                    A2, X2 = X2, A2
                assert A2.shape == (y.size, X2.shape[0]) and X2.shape[1] == 1, (A.shape, X.shape, y.shape)
                # the running value is y itself (1.0 * y_in, + 0.0 at the end): accumulate in place
                terms.append(C.block_rows_args(y.reshape(-1) if y.ndim != 1 else y, A2, X2[:, 0]))
            self._prepared[id(ops[0])] = terms
        run = C.block_rows_run
        for args in terms:
            run(args)

    def _do_DotInc(self, op):
        self._block_inc(op.Y, [op])

    def _do__DotGroup(self, op):
        self._block_inc(op.Y, op.group)

    def _do_SparseDotInc(self, op):
        # the reference's CSR kernel in increment mode (clra_gemv.py:1591-1617)
        A = self.signals[op.A]
        y = self.view(op.Y)
        y[...] = K.spmv_csr(A.indices, A.indptr, A.data, self.view(op.X).reshape(-1), y.reshape(-1),
                            inc=True).reshape(y.shape)

    def _do_ElementwiseInc(self, op):
        A, X, Y = self.view(op.A), self.view(op.X), self.view(op.Y)
        Y[...] = Y + (A * X).astype(np.float32)

    def _do_SimNeurons(self, op):
        nt = op.neurons
        kind = type(nt).__name__
        J = self.view(op.J)
        out = self.view(op.output)
        if kind == "LIF" and J.flags.c_contiguous and out.flags.c_contiguous:
            # the compiled restatement of the same kernel (checked against kernels.lif in the tests)
            C.lif(self.dt, J, self.view(op.state["voltage"]), self.view(op.state["refractory_time"]), out,
                  f32(nt.tau_rc), f32(nt.tau_ref), f32(nt.amplitude))
        elif kind in ("LIF", "AdaptiveLIF"):
            V = self.view(op.state["voltage"])
            W = self.view(op.state["refractory_time"])
            n = J.size
            tau = np.full(n, nt.tau_rc, np.float32)
            ref = np.full(n, nt.tau_ref, np.float32)
            amp = np.full(n, nt.amplitude, np.float32)
            if kind == "AdaptiveLIF":
                Nn = self.view(op.state["adaptation"])
                v, w, s, nn = K.lif(self.dt, J, V, W, tau, ref, amp, N=Nn,
                                    tau_n=np.full(n, nt.tau_n, np.float32),
                                    inc_n=np.full(n, nt.inc_n, np.float32))
                Nn[...] = nn
            else:
                v, w, s = K.lif(self.dt, J, V, W, tau, ref, amp)
            V[...], W[...], out[...] = v, w, s
        elif kind == "LIFRate":
            out[...] = K.lif_rate(J, f32(nt.tau_rc), f32(nt.tau_ref), f32(nt.amplitude))
        elif kind == "RectifiedLinear":
            out[...] = K.relu(J, f32(nt.amplitude))
        elif kind == "SpikingRectifiedLinear":
            V = self.view(op.state["voltage"])
            v, s = K.spiking_relu(self.dt, J, V, f32(nt.amplitude))
            V[...], out[...] = v, s
        elif kind == "Sigmoid":
            out[...] = K.sigmoid(J, f32(nt.tau_ref))
        else:
            raise ValueError("Unsupported neuron type %r" % kind)

    def _do_SimProcess(self, op):
        proc = op.process
        names = self._prepared.get(type(proc))
        if names is None:
            names = self._prepared[type(proc)] = [c.__name__ for c in type(proc).__mro__]
        out = self.view(op.output)
        if "LinearFilter" in names:
            coef = self._prepared.get(id(op))
            if coef is None:
                num, den = proc.discrete_tf(self.dt)
                coef = self._prepared[id(op)] = (num.astype(np.float32), den.astype(np.float32))
            b, a = coef
            x = self.view(op.input)
            na, nb = len(a), len(b)
            if na == 0 and nb == 1:
                new = b[0] * x
            elif na == 1 and nb == 1:
                new = b[0] * x - a[0] * out
            else:
                st = self._filter_state.setdefault(
                    op, dict(xb=np.zeros((nb, x.size), np.float32), yb=np.zeros((na, x.size), np.float32),
                             ix=0, iy=0))
                ix, iy = st["ix"], st["iy"]
                iy1 = iy - 1 if iy > 0 else na - 1
                xf = x.reshape(-1)
                yi = b[0] * xf
                if nb > 1:
                    st["xb"][ix] = xf
                    for p in range(1, nb):
                        yi = yi + b[p] * st["xb"][(ix + p) % nb]
                if na > 0:
                    yi = yi - a[0] * out.reshape(-1)
                    if na > 1:
                        for p in range(1, na):
                            yi = yi - a[p] * st["yb"][(iy + p) % na]
                        st["yb"][iy1] = yi
                st["ix"] = ix - 1 if ix > 0 else nb - 1
                st["iy"] = iy - 1 if iy > 0 else na - 1
                new = yi.reshape(out.shape)
            new = new.astype(np.float32)
            out[...] = out + new if op.mode == "inc" else new
        elif "WhiteNoise" in names:
            if proc.seed is None:
                raise ValueError("the oracle needs an explicit seed for a WhiteNoise process")
            it = int(self.view(self.model.step)[()])
            dist = proc.dist
            enum = {"Uniform": 0, "Gaussian": 1}[type(dist).__name__]
            params = (dist.low, dist.high) if enum == 0 else (dist.mean, dist.std)
            s = K.whitenoise_samples(proc.seed, it, out.size, enum, params, proc.scale, self.dt).reshape(out.shape)
            out[...] = (out + s).astype(np.float32) if op.mode == "inc" else s
        elif "WhiteSignal" in names:
            it = int(self.view(self.model.step)[()])
            table = proc.signal.astype(np.float32)
            out[...] = table[it % table.shape[0]].reshape(out.shape)
        elif "PresentInput" in names:
            it = int(self.view(self.model.step)[()])
            table = proc.inputs.reshape(proc.inputs.shape[0], -1).astype(np.float32)
            v = f32(f32(f32(it) - f32(0.5)) * f32(f32(self.dt) / f32(proc.presentation_time)))
            ti = int(np.fmod(int(v), table.shape[0]))
            out[...] = table[ti].reshape(out.shape)
        else:
            raise NotImplementedError(type(proc).__name__)

    def _do_ConvInc(self, op):
        # nengo_ocl/simulator.py:1298-1313: a 1-D convolution is a 2-D one with a single row
        conv = op.conv
        shape_in, shape_out = tuple(conv.input_shape), tuple(conv.output_shape)
        kernel_shape, strides = tuple(conv.kernel_size), tuple(conv.strides)
        if conv.dimensions == 1:
            kernel_shape, strides = (1,) + kernel_shape, (1,) + strides
            if conv.channels_last:
                shape_in, shape_out = (1,) + shape_in, (1,) + shape_out
            else:
                shape_in, shape_out = (shape_in[0], 1, shape_in[1]), (shape_out[0], 1, shape_out[1])
        padding = op.conv.padding.lower() if isinstance(op.conv.padding, str) else op.conv.padding
        y = self.view(op.Y)
        out = K.conv2d(self.view(op.X), self.view(op.W), shape_in, shape_out, kernel_shape, True, padding, strides,
                       op.conv.channels_last)
        y[...] = (y + out.reshape(y.shape)).astype(np.float32)

    def _do_SimPES(self, op):
        pre = self.view(op.pre_filtered)
        err = self.view(op.error)
        delta = self.view(op.delta)
        alpha = f32(-op.learning_rate * self.dt / pre.shape[0])
        delta[...] = ((alpha * err)[:, None] * pre[None, :]).astype(np.float32)

    def _do_SimBCM(self, op):
        self.view(op.delta)[...] = K.bcm(self.view(op.pre_filtered), self.view(op.post_filtered),
                                         self.view(op.theta), op.learning_rate * self.dt)

    def _do_SimOja(self, op):
        self.view(op.delta)[...] = K.oja(self.view(op.pre_filtered), self.view(op.post_filtered),
                                         self.view(op.weights), op.learning_rate * self.dt, op.beta)

    def _do_SimVoja(self, op):
        self.view(op.delta)[...] = K.voja(self.view(op.pre_decoded), self.view(op.post_filtered),
                                          self.view(op.scaled_encoders), self.view(op.learning_signal).reshape(-1)[0],
                                          op.scale, op.learning_rate * self.dt)

    def _do_SimPyFunc(self, op):
        args = []
        if op.t is not None:
            args.append(float(self.view(op.t)[()]))
        if op.x is not None:
            args.append(np.array(self.view(op.x), dtype=np.float64))
        y = op.fn(*args)
        if op.output is not None:
            self.view(op.output)[...] = np.asarray(y, dtype=np.float32).reshape(op.output.shape)


class _DotGroup:
    """Several DotIncs into one target, executed as one multi-term product."""

    def __init__(self, group):
        self.group = group
        self.Y = group[0].Y
        self.sets, self.updates = [], []
        self.incs = [self.Y]
        self.reads = [s for op in group for s in (op.A, op.X)]

    @property
    def all_signals(self):
        return self.incs + self.reads
