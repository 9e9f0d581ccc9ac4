"""Benchmark configuration 5 (the PES learning model) on the compiled CPU oracle.

TEST INFRASTRUCTURE ONLY (see ``oracle/kernels.py``).  ``PesBatch`` copies the
signals of a ``synth.pes_learning_model`` into batched arrays (all ensembles
have the same shape) and steps them with ``nb2o_pes_model_step`` of
``oracle/cport.c``: the reference's operators in the reference's order, one
loop nest per kernel launch, OpenMP over the ragged items.  It is checked
against the operator-list interpreter (``oracle/simulator.py``) in the tests
and is the timed CPU baseline of the benchmark.
"""

import ctypes

import numpy as np

from oracle import cport

_F = ctypes.POINTER(ctypes.c_float)
_I = ctypes.POINTER(ctypes.c_int)


class PesBatch:
    def __init__(self, model):
        info = model.info
        ens, conns = info["ensembles"], info["connections"]
        assert len(ens) == len(conns) and all(c["pre"] is e for c, e in zip(conns, ens))
        self.model = model
        self.E = E = len(ens)
        self.n, self.d = ens[0].n_neurons, ens[0].dimensions
        self.dc = conns[0]["weights"].shape[0]
        self.dt = float(model.dt)
        f32 = np.float32
        stack = lambda sigs: np.ascontiguousarray(np.stack([np.asarray(s.initial_value, dtype=f32) for s in sigs]))
        self.enc = stack([e.sig_enc for e in ens])
        self.bias = stack([e.sig_bias for e in ens])
        self.V = stack([e.state["voltage"] for e in ens])
        self.W = stack([e.state["refractory_time"] for e in ens])
        self.J = np.zeros((E, self.n), f32)
        self.S = np.zeros((E, self.n), f32)
        self.dec = stack([c["weights"] for c in conns])
        self.delta = np.zeros_like(self.dec)
        self.weighted = np.zeros((E, self.dc), f32)
        self.filtered = np.zeros((E, self.dc), f32)
        self.err = np.zeros((E, self.dc), f32)
        self.pf = np.zeros((E, self.n), f32)
        self.x = np.zeros((E, self.d), f32)
        self.targets = np.ascontiguousarray(info["targets"], dtype=np.int32)
        # error tables: the WhiteSignal process feeding each connection's error input
        procs = {}
        for op in model.operators:
            if type(op).__name__ == "SimProcess" and type(op.process).__name__ == "WhiteSignal":
                procs[op.output] = op.process
        copies = {op.dst: op.src for op in model.operators if type(op).__name__ == "Copy" and op.inc}
        self.tables = np.ascontiguousarray(
            np.stack([procs[copies[c["error"]]].signal.astype(f32) for c in conns]))
        self.nt = self.tables.shape[1]
        nt_ = ens[0].neuron_type
        self.neuron = (f32(nt_.tau_rc), f32(nt_.tau_ref), f32(nt_.amplitude))
        filt = {}
        for op in model.operators:
            if type(op).__name__ == "SimProcess" and type(op.process).__name__ == "Lowpass":
                num, den = op.process.discrete_tf(self.dt)
                filt[op.output] = (f32(num[0]), f32(den[0]))
        self.syn = filt[conns[0]["out"]]
        self.pre = filt[conns[0]["pre_filtered"]]
        pes = [op for op in model.operators if type(op).__name__ == "SimPES"][0]
        self.alpha = f32(-pes.learning_rate * self.dt / self.n)
        self.step_index = 0
        lib = cport.lib()
        lib.nb2o_pes_model_step.argtypes = ([ctypes.c_int] * 4 + [ctypes.c_double, ctypes.c_int, ctypes.c_int, _I]
                                            + [_F] * 14 + [ctypes.c_float] * 8)
        lib.nb2o_pes_model_step.restype = None
        self._fn = lib.nb2o_pes_model_step
        p = lambda a: a.ctypes.data_as(_F)
        self._arrays = [p(a) for a in (self.tables, self.x, self.enc, self.bias, self.J, self.V, self.W, self.S,
                                       self.dec, self.delta, self.weighted, self.filtered, self.err, self.pf)]

    def step(self):
        self.step_index += 1  # TimeUpdate comes first: tables are read at the new step number
        tau, ref, amp = self.neuron
        self._fn(self.E, self.n, self.d, self.dc, self.dt, self.step_index, self.nt,
                 self.targets.ctypes.data_as(_I), *self._arrays, tau, ref, amp, self.syn[0], self.syn[1],
                 self.pre[0], self.pre[1], self.alpha)

    def run_steps(self, k):
        for _ in range(k):
            self.step()

    @property
    def bytes_per_step(self):
        """Bytes the reference's kernels move per step, kernel by kernel (cport.c)."""
        E, n, d, dc = self.E, self.n, self.d, self.dc
        return 4 * E * (3 * dc * n + 2 * n + (n * d + d + 2 * n) + 7 * n + dc + (dc * n + n + 2 * dc)
                        + (dc + n + dc * n) + (3 * dc + 3 * n))
