"""A nengo-free operator-level model: signals, operators, neuron types, processes.

The reference consumes the output of nengo's builder: a ``Model`` holding a
list of ``Operator`` objects over ``Signal`` objects (nengo_ocl/simulator.py:
229-265).  nengo itself is a third-party dependency that is not part of the
reference tree, so this module defines the small operator-level interface the
simulator relies on, with the attribute names the reference reads:

* signals: ``base, is_view, sparse, ndim, shape, size, elemoffset,
  elemstrides, initial_value, readonly, name, may_share_memory()``
  (simulator.py:93-111,271-301,552-555; planners.py:52-62);
* operators: ``sets, incs, reads, updates, all_signals, init_signals(), tag``
  and the per-type fields each ``Simulator._plan_<Type>`` method reads
  (simulator.py:746-1345).

Models are written directly at this level (see ``nengo_ocl_b200.synth``); a
model built by real nengo exposes the same attributes and is accepted too.
Within one time step every signal goes through the phases
set -> inc -> read -> update, which is what orders operators.
"""

import numpy as np


class Signal:
    """An n-d float array (or a strided view of one) that operators act on."""

    sparse = False

    def __init__(self, initial_value=None, shape=None, name=None, base=None, readonly=False,
                 elemoffset=0, elemstrides=None):
        if base is None and hasattr(initial_value, "tocsr"):
            # a sparse matrix (scipy.sparse): kept as it is, outside the packed dense store
            self.sparse = True
            self._initial_value = initial_value.tocsr()
            self.shape = tuple(int(v) for v in initial_value.shape)
            self._base = None
            self.elemoffset = 0
            self.elemstrides = (self.shape[1], 1)
        elif base is None:
            if initial_value is None:
                initial_value = np.zeros(shape if shape is not None else ())
            initial_value = np.array(initial_value, dtype=np.float64)
            self._initial_value = initial_value
            self.shape = tuple(initial_value.shape)
            self._base = None
            self.elemoffset = 0
            strides, acc = [], 1
            for n in reversed(self.shape):  # C order
                strides.append(acc)
                acc *= n
            self.elemstrides = tuple(reversed(strides))
        else:
            assert base._base is None, "views must reference a base signal"
            self._initial_value = None
            self.shape = tuple(int(s) for s in shape)
            self._base = base
            self.elemoffset = int(elemoffset)
            self.elemstrides = tuple(int(s) for s in elemstrides)
        self.name = name if name is not None else "signal"
        self.readonly = bool(readonly)

    # -- structure ----------------------------------------------------------
    @property
    def base(self):
        return self if self._base is None else self._base

    @property
    def is_view(self):
        return self._base is not None

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def size(self):
        n = 1
        for v in self.shape:  # (a plain loop: this is called a million times while a large model is planned)
            n *= int(v)
        return n

    @property
    def initial_value(self):
        if self._base is None:
            return self._initial_value
        flat = self._base._initial_value.reshape(-1)
        isz = flat.itemsize
        return np.lib.stride_tricks.as_strided(
            flat[self.elemoffset:], shape=self.shape, strides=tuple(s * isz for s in self.elemstrides))

    def _view(self, shape, offset, strides, name=None):
        return Signal(shape=shape, base=self.base, elemoffset=offset, elemstrides=strides,
                      name=name or "%s.view" % self.name, readonly=self.readonly)

    def __getitem__(self, item):
        """Basic slicing (ints and slices) -> view signal."""
        if not isinstance(item, tuple):
            item = (item,)
        item = item + (slice(None),) * (self.ndim - len(item))
        shape, strides, offset = [], [], self.elemoffset
        for idx, n, st in zip(item, self.shape, self.elemstrides):
            if isinstance(idx, slice):
                start, stop, step = idx.indices(n)
                shape.append(max(0, -(-(stop - start) // step)))
                strides.append(st * step)
                offset += start * st
            else:
                idx = int(idx)
                offset += (idx % n) * st
        return self._view(tuple(shape), offset, tuple(strides), "%s[%s]" % (self.name, item))

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = tuple(int(s) for s in shape)
        assert int(np.prod(shape)) == self.size
        # only views whose elements are evenly spaced can be reshaped freely
        if self.ndim == 0 or self.size <= 1:
            step = 1
        elif self.ndim == 1:
            step = self.elemstrides[0]
        else:
            expect = 1
            for n, st in zip(reversed(self.shape), reversed(self.elemstrides)):
                if n > 1 and st != expect:
                    raise ValueError("cannot reshape a non-contiguous view")
                expect *= n
            step = 1
        strides = []
        acc = step
        for n in reversed(shape):
            strides.append(acc)
            acc *= n
        return self._view(shape, self.elemoffset, tuple(reversed(strides)), "%s.reshape%s" % (self.name, shape))

    def may_share_memory(self, other):
        if self.base is not other.base:
            return False

        def extent(s):
            lo = s.elemoffset
            hi = lo + sum((n - 1) * abs(st) for n, st in zip(s.shape, s.elemstrides)) + 1
            return lo, hi

        a0, a1 = extent(self)
        b0, b1 = extent(other)
        return a0 < b1 and b0 < a1

    def __repr__(self):
        return "Signal(%s, shape=%s)" % (self.name, self.shape)


class Operator:
    """Base class: declares which signals are set / incremented / read / updated."""

    def __init__(self, tag=None):
        self.tag = tag
        self.sets = []
        self.incs = []
        self.reads = []
        self.updates = []

    @property
    def all_signals(self):
        return list(self.sets) + list(self.incs) + list(self.reads) + list(self.updates)

    def init_signals(self, signals):
        """Enter the initial value of every base signal into ``signals``."""
        for sig in self.all_signals:
            base = sig.base
            if base not in signals:
                signals[base] = (base.initial_value if base.sparse
                                 else np.array(base.initial_value, dtype=np.float64))

    def __repr__(self):
        return "<%s%s at 0x%x>" % (type(self).__name__, " %s" % self.tag if self.tag else "", id(self))


class TimeUpdate(Operator):
    def __init__(self, step, time, tag=None):
        super().__init__(tag)
        self.step, self.time = step, time
        self.sets = [step, time]


class Reset(Operator):
    def __init__(self, dst, value=0.0, tag=None):
        super().__init__(tag)
        self.dst, self.value = dst, float(value)
        self.sets = [dst]


class Copy(Operator):
    def __init__(self, src, dst, inc=False, src_slice=None, dst_slice=None, tag=None):
        super().__init__(tag)
        self.src, self.dst, self.inc = src, dst, bool(inc)
        self.src_slice, self.dst_slice = src_slice, dst_slice
        self.reads = [src]
        if inc:
            self.incs = [dst]
        else:
            self.sets = [dst]


class DotInc(Operator):
    """``Y += A . X``"""

    def __init__(self, A, X, Y, tag=None):
        super().__init__(tag)
        self.A, self.X, self.Y = A, X, Y
        self.incs = [Y]
        self.reads = [A, X]


class SparseDotInc(Operator):
    """``Y += A . X`` with a sparse matrix signal ``A``"""

    def __init__(self, A, X, Y, tag=None):
        super().__init__(tag)
        assert A.sparse and not A.is_view
        self.A, self.X, self.Y = A, X, Y
        self.incs = [Y]
        self.reads = [A, X]


class ElementwiseInc(Operator):
    """``Y += A * X`` with broadcasting"""

    def __init__(self, A, X, Y, tag=None):
        super().__init__(tag)
        self.A, self.X, self.Y = A, X, Y
        self.incs = [Y]
        self.reads = [A, X]


class Convolution:
    """Geometry of a convolutional transform (what nengo's ``Convolution`` transform carries):
    ``input_shape`` / ``output_shape`` are (rows, cols, channels) when ``channels_last`` else
    (channels, rows, cols); 1-D convolutions give (cols, channels) / (channels, cols)."""

    def __init__(self, n_filters, input_shape, kernel_size=(3, 3), strides=(1, 1), padding="valid",
                 channels_last=True):
        self.n_filters, self.channels_last = int(n_filters), bool(channels_last)
        self.kernel_size = tuple(int(k) for k in kernel_size)
        self.strides = tuple(int(s) for s in strides)
        self.padding = padding
        self.input_shape = tuple(int(v) for v in input_shape)
        self.dimensions = len(self.kernel_size)
        spatial = self.input_shape[:-1] if channels_last else self.input_shape[1:]
        out = []
        for n, k, st in zip(spatial, self.kernel_size, self.strides):
            out.append(-(-n // st) if padding.lower() == "same" else (n - k) // st + 1)
        self.output_shape = tuple(out) + (self.n_filters,) if channels_last else (self.n_filters,) + tuple(out)
        self.n_channels = self.input_shape[-1] if channels_last else self.input_shape[0]
        self.kernel_shape = self.kernel_size + (self.n_channels, self.n_filters)


class ConvInc(Operator):
    """``Y += convolution(X, W)`` with W of shape kernel_size + (channels, filters)."""

    def __init__(self, W, X, Y, conv, tag=None):
        super().__init__(tag)
        self.W, self.X, self.Y, self.conv = W, X, Y, conv
        self.reads = [W, X]
        self.incs = [Y]


class SimNeurons(Operator):
    def __init__(self, neurons, J, output, state=None, tag=None):
        super().__init__(tag)
        self.neurons, self.J, self.output = neurons, J, output
        self.state = dict(state or {})
        self.sets = [output]
        self.reads = [J]
        self.updates = list(self.state.values())


class SimProcess(Operator):
    def __init__(self, process, input, output, t, mode="set", tag=None):
        super().__init__(tag)
        self.process, self.input, self.output, self.t, self.mode = process, input, output, t, mode
        self.reads = [t] + ([input] if input is not None else [])
        if output is not None:
            {"set": self.sets, "inc": self.incs, "update": self.updates}[mode].append(output)


class SimPES(Operator):
    """``delta = -learning_rate * dt / n * outer(error, pre_filtered)``"""

    def __init__(self, pre_filtered, error, delta, learning_rate, tag=None):
        super().__init__(tag)
        self.pre_filtered, self.error, self.delta = pre_filtered, error, delta
        self.learning_rate = float(learning_rate)
        self.reads = [pre_filtered, error]
        self.updates = [delta]


class SimBCM(Operator):
    """``delta = learning_rate * dt * post * (post - theta) * pre`` (outer product)"""

    def __init__(self, pre_filtered, post_filtered, theta, delta, learning_rate, tag=None):
        super().__init__(tag)
        self.pre_filtered, self.post_filtered, self.theta, self.delta = pre_filtered, post_filtered, theta, delta
        self.learning_rate = float(learning_rate)
        self.reads = [pre_filtered, post_filtered, theta]
        self.updates = [delta]


class SimOja(Operator):
    """``delta = learning_rate * dt * post * (pre - beta * weights * post)``"""

    def __init__(self, pre_filtered, post_filtered, weights, delta, learning_rate, beta, tag=None):
        super().__init__(tag)
        self.pre_filtered, self.post_filtered, self.weights, self.delta = pre_filtered, post_filtered, weights, delta
        self.learning_rate, self.beta = float(learning_rate), float(beta)
        self.reads = [pre_filtered, post_filtered, weights]
        self.updates = [delta]


class SimVoja(Operator):
    """``delta = learning_rate * dt * learning_signal * post * (scale * pre_decoded - scaled_encoders)``"""

    def __init__(self, pre_decoded, post_filtered, scaled_encoders, delta, scale, learning_signal, learning_rate,
                 tag=None):
        super().__init__(tag)
        self.pre_decoded, self.post_filtered, self.scaled_encoders = pre_decoded, post_filtered, scaled_encoders
        self.delta, self.learning_signal = delta, learning_signal
        self.scale = np.asarray(scale, dtype=np.float64)
        self.learning_rate = float(learning_rate)
        self.reads = [pre_decoded, post_filtered, scaled_encoders, learning_signal]
        self.updates = [delta]


class SimPyFunc(Operator):
    def __init__(self, output, fn, t, x, tag=None):
        super().__init__(tag)
        self.output, self.fn, self.t, self.x = output, fn, t, x
        self.sets = [output] if output is not None else []
        self.reads = ([t] if t is not None else []) + ([x] if x is not None else [])


# ---- neuron types (parameters only; the math lives in the kernels) ----------
class NeuronType:
    state_names = ()


class LIF(NeuronType):
    state_names = ("voltage", "refractory_time")

    def __init__(self, tau_rc=0.02, tau_ref=0.002, min_voltage=0.0, amplitude=1.0):
        self.tau_rc, self.tau_ref = float(tau_rc), float(tau_ref)
        self.min_voltage, self.amplitude = float(min_voltage), float(amplitude)

    def rates(self, J):
        """Steady-state firing rate for input current J (float64)."""
        J = np.asarray(J, dtype=np.float64)
        out = np.zeros_like(J)
        m = J > 1
        out[m] = self.amplitude / (self.tau_ref + self.tau_rc * np.log1p(1.0 / (J[m] - 1)))
        return out

    def gain_bias(self, max_rates, intercepts):
        """Gain and bias so a neuron fires ``max_rate`` at x=1 and starts at ``intercept``."""
        max_rates = np.asarray(max_rates, dtype=np.float64)
        intercepts = np.asarray(intercepts, dtype=np.float64)
        x = 1.0 / (1 - np.exp((self.tau_ref - 1.0 / max_rates) / self.tau_rc))
        gain = (1 - x) / (intercepts - 1.0)
        bias = 1 - gain * intercepts
        return gain, bias


class LIFRate(LIF):
    state_names = ()


class AdaptiveLIF(LIF):
    state_names = ("voltage", "refractory_time", "adaptation")

    def __init__(self, tau_n=1.0, inc_n=0.01, **kwargs):
        super().__init__(**kwargs)
        self.tau_n, self.inc_n = float(tau_n), float(inc_n)


class AdaptiveLIFRate(AdaptiveLIF):
    state_names = ("adaptation",)


class RectifiedLinear(NeuronType):
    def __init__(self, amplitude=1.0):
        self.amplitude = float(amplitude)


class SpikingRectifiedLinear(RectifiedLinear):
    state_names = ("voltage",)


class Sigmoid(NeuronType):
    def __init__(self, tau_ref=0.0025):
        self.tau_ref = float(tau_ref)


# ---- processes ---------------------------------------------------------------
class Process:
    pass


class LinearFilter(Process):
    """Continuous transfer function num(s)/den(s), discretised with a
    zero-order hold, or (``analog=False``) a discrete one used as given."""

    def __init__(self, num, den, analog=True):
        self.num = np.atleast_1d(np.asarray(num, dtype=np.float64))
        self.den = np.atleast_1d(np.asarray(den, dtype=np.float64))
        self.analog = analog

    def discrete_tf(self, dt):
        """(num, den) of the difference equation
        ``y[n+1] + a0 y[n] + ... = b0 x[n] + ...`` with the leading zero of num
        dropped and den[0] == 1 removed (simulator.py:1216-1227)."""
        num, den = self.num, self.den
        if self.analog:
            from scipy.signal import cont2discrete

            num, den, _ = cont2discrete((num, den), dt, method="zoh")
            num = np.asarray(num, dtype=np.float64).flatten()
            den = np.asarray(den, dtype=np.float64).flatten()
        num = num / den[0]
        den = den / den[0]
        if len(num) > 1 and num[0] == 0:
            num = num[1:]
        return num, den[1:]


class Lowpass(LinearFilter):
    def __init__(self, tau):
        self.tau = float(tau)
        super().__init__([1.0], [self.tau, 1.0])

    def discrete_tf(self, dt):
        if self.tau <= 0.03 * dt:  # pass-through
            return np.array([1.0]), np.array([])
        a = np.exp(-dt / self.tau)
        return np.array([1.0 - a]), np.array([-a])


class Alpha(LinearFilter):
    def __init__(self, tau):
        self.tau = float(tau)
        super().__init__([1.0], [self.tau ** 2, 2 * self.tau, 1.0])


class PresentInput(Process):
    """Plays the rows of ``inputs`` for ``presentation_time`` seconds each."""

    def __init__(self, inputs, presentation_time):
        self.inputs = np.asarray(inputs, dtype=np.float64)
        self.presentation_time = float(presentation_time)


class WhiteSignal(Process):
    """Band-limited white noise, synthesised once as a table of per-step values
    that is played back by step index (simulator.py:1263-1277)."""

    def __init__(self, period, high, rms=0.5, seed=None, dt=0.001, size_out=1):
        self.period, self.high, self.rms, self.seed = float(period), float(high), float(rms), seed
        n = int(np.round(self.period / dt))
        rng = np.random.RandomState(seed)
        freqs = np.fft.rfftfreq(n, d=dt)
        coefs = rng.normal(size=(len(freqs), size_out)) + 1j * rng.normal(size=(len(freqs), size_out))
        coefs[0] = 0
        coefs[freqs > self.high] = 0
        sig = np.fft.irfft(coefs, n=n, axis=0)
        power = np.sqrt(np.mean(sig ** 2, axis=0, keepdims=True))
        power[power == 0] = 1
        self.signal = (sig * (self.rms / power)).astype(np.float64)  # (n_steps, size_out)


class Uniform:
    def __init__(self, low, high):
        self.low, self.high = float(low), float(high)


class Gaussian:
    def __init__(self, mean, std):
        self.mean, self.std = float(mean), float(std)


class WhiteNoise(Process):
    """Independent samples of ``dist`` every step; ``scale`` multiplies them by
    1/sqrt(dt) so that the noise power does not depend on dt (simulator.py:1245-1258)."""

    def __init__(self, dist=None, scale=True, seed=None):
        self.dist = Gaussian(0.0, 1.0) if dist is None else dist
        self.scale, self.seed = bool(scale), seed


# ---- probes and the model container -----------------------------------------
class Probe:
    def __init__(self, target, sample_every=None, label=None):
        self.target = target  # the Signal whose value is recorded
        self.sample_every = sample_every
        self.label = label

    def __repr__(self):
        return "<Probe %s>" % (self.label or self.target.name)


class Model:
    """Operator-level model: what nengo's builder would hand to the simulator."""

    def __init__(self, dt=0.001, label=None, seed=None):
        self.dt = float(dt)
        self.label = label
        self.seed = seed
        self.operators = []
        self.probes = []
        self.params = {}
        self.sig = {}
        self.step = Signal(np.array(0.0), name="step")
        self.time = Signal(np.array(0.0), name="time")
        self.add_op(TimeUpdate(self.step, self.time))
        # ensemble-level annotations used by the fusion pass and the sharding
        self.n_neurons = 0

    def add_op(self, op):
        self.operators.append(op)
        return op

    def add_probe(self, signal, sample_every=None, label=None):
        probe = Probe(signal, sample_every=sample_every, label=label)
        self.probes.append(probe)
        self.sig[probe] = {"in": signal}
        return probe

    def build(self, network):
        raise NotImplementedError(
            "building from a nengo Network needs the nengo package; pass a prebuilt model instead")
