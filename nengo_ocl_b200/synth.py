"""Seeded synthetic workloads with the shapes of the benchmark configurations.

nengo (which would build these networks from a high-level description) is
not a dependency, so every model here is written directly at the operator
level with ``nengo_ocl_b200.model``: the same signals and operators a nengo
build of the described network produces (ensemble = reset input, bias copy,
encoder DotInc, SimNeurons; decoded connection = reset, decoder DotInc,
synapse SimProcess, Copy into the target input; PES = pre-activity lowpass,
SimPES, Copy(inc) into the decoders).  Parameter distributions follow the
configuration text (max rates U(200,400) Hz, intercepts U(-1,1), unit-length
encoders, regularised least-squares decoders).  These are stand-ins for the
nengo-built networks, not reproductions of nengo's builder.
"""

import numpy as np

from nengo_ocl_b200 import model as m
from nengo_ocl_b200.raggedarray import RaggedArray


# ---- configuration 2: ragged gather-GEMV microbenchmark ------------------------
def gemv_workload(seed=1, n_outputs=4096, max_terms=4, max_rows=1024, max_cols=64, n_x=None, align=False):
    """``Y_k = beta*Y_k + alpha*sum_j A_kj X_idx(kj)``: ``n_outputs`` blocks with
    1..max_terms terms, rows ~ U[1,max_rows], columns ~ U[1,max_cols], float32
    N(0,1) data, uniform gather indices.  Returns host ragged arrays
    ``(A, A_js, X, X_js, Y)`` laid out like ``RaggedArray`` (row-major; starts
    unaligned unless ``align``)."""
    rng = np.random.RandomState(seed)
    n_x = n_outputs if n_x is None else n_x
    x_cols = rng.randint(1, max_cols + 1, size=n_x)
    X = [rng.normal(size=(n, 1)).astype(np.float32) for n in x_cols]
    rows = rng.randint(1, max_rows + 1, size=n_outputs)
    terms = rng.randint(1, max_terms + 1, size=n_outputs)
    A, A_js, X_js = [], [], []
    for k in range(n_outputs):
        xj = rng.randint(n_x, size=terms[k])
        aj = []
        for j in xj:
            aj.append(len(A))
            A.append(rng.standard_normal(size=(rows[k], x_cols[j])).astype(np.float32))
        A_js.append(np.asarray(aj, dtype=np.int32))
        X_js.append(np.asarray(xj, dtype=np.int32))
    Y = [rng.normal(size=(r, 1)).astype(np.float32) for r in rows]
    return (RaggedArray(A, dtype=np.float32, align=align), RaggedArray(A_js, dtype=np.int32),
            RaggedArray(X, dtype=np.float32, align=align), RaggedArray(X_js, dtype=np.int32),
            RaggedArray(Y, dtype=np.float32, align=align))


# ---- operator-level network construction ------------------------------------------
class Ensemble:
    """Signals and parameters of one population (what an ensemble build yields)."""

    def __init__(self, n, d, label):
        self.n_neurons, self.dimensions, self.label = n, d, label


class NetBuilder:
    """Emits the operators a nengo build of ensembles / nodes / decoded
    connections / PES rules produces, directly into a ``Model``."""

    def __init__(self, dt=0.001, seed=0, label=None):
        self.model = m.Model(dt=dt, label=label, seed=seed)
        self.rng = np.random.RandomState(seed)
        self.ensembles = []
        self.connections = []

    # -- populations ------------------------------------------------------------
    def ensemble(self, n, d, label=None, radius=1.0, max_rates=(200.0, 400.0), intercepts=(-1.0, 1.0),
                 neuron_type=None, encoders=None, params_from=None):
        """Reset input, copy bias into J, J += scaled_encoders . input, neuron update."""
        mdl = self.model
        label = label or "ens%d" % len(self.ensembles)
        nt = neuron_type or m.LIF()
        ens = Ensemble(n, d, label)
        ens.neuron_type, ens.radius = nt, radius
        if params_from is not None:  # share build parameters (not state) with a template ensemble
            enc, gain, bias = params_from.encoders, params_from.gain, params_from.bias
        else:
            rng = self.rng
            if encoders is None:
                encoders = rng.standard_normal(size=(n, d))
                encoders /= np.linalg.norm(encoders, axis=1, keepdims=True)
            enc = np.asarray(encoders, dtype=np.float64)
            rates = rng.uniform(max_rates[0], max_rates[1], size=n)
            icpt = rng.uniform(intercepts[0], intercepts[1], size=n)
            gain, bias = nt.gain_bias(rates, icpt)
        ens.encoders, ens.gain, ens.bias = enc, gain, bias
        ens.sig_in = m.Signal(np.zeros(d), name="%s.in" % label)
        ens.sig_J = m.Signal(np.zeros(n), name="%s.neurons.in" % label)
        ens.sig_out = m.Signal(np.zeros(n), name="%s.neurons.out" % label)
        ens.sig_enc = m.Signal(enc * (gain / radius)[:, None], name="%s.scaled_encoders" % label, readonly=True)
        ens.sig_bias = m.Signal(bias, name="%s.bias" % label, readonly=True)
        state = {}
        for name in nt.state_names:
            state[name] = m.Signal(np.zeros(n), name="%s.%s" % (label, name))
        ens.state = state
        mdl.add_op(m.Reset(ens.sig_in))
        mdl.add_op(m.Copy(ens.sig_bias, ens.sig_J))
        mdl.add_op(m.DotInc(ens.sig_enc, ens.sig_in, ens.sig_J, tag="%s.encode" % label))
        mdl.add_op(m.SimNeurons(nt, ens.sig_J, ens.sig_out, state=state))
        mdl.n_neurons += n
        self.ensembles.append(ens)
        return ens

    def solve_decoders(self, ens, function=None, n_eval=None, reg=0.1, rng=None):
        """Regularised least squares of the target function on random points in
        the ensemble's represented ball -> decoders of shape (d_out, n)."""
        rng = rng or self.rng
        d = ens.dimensions
        n_eval = n_eval or max(750, 2 * ens.n_neurons)
        pts = rng.standard_normal(size=(n_eval, d))
        pts *= (rng.uniform(size=(n_eval, 1)) ** (1.0 / d)) / np.linalg.norm(pts, axis=1, keepdims=True)
        pts *= ens.radius
        J = (pts / ens.radius) @ ens.encoders.T * ens.gain + ens.bias
        A = ens.neuron_type.rates(J)
        target = pts if function is None else np.array([np.atleast_1d(function(p)) for p in pts])
        sigma = reg * A.max()
        G = A.T @ A + n_eval * sigma ** 2 * np.eye(ens.n_neurons)
        return np.linalg.solve(G, A.T @ target).T

    # -- inputs -------------------------------------------------------------------
    def node_fn(self, fn, size_out, label="node"):
        out = m.Signal(np.zeros(size_out), name="<Node %s>.out" % label)
        self.model.add_op(m.SimPyFunc(out, fn, self.model.time, None))
        return out

    def node_process(self, process, size_out, label="node"):
        out = m.Signal(np.zeros(size_out), name="<Node %s>.out" % label)
        self.model.add_op(m.SimProcess(process, None, out, self.model.time, mode="set"))
        return out

    def node_const(self, value, label="node"):
        return m.Signal(np.asarray(value, dtype=np.float64), name="<Node %s>.out" % label, readonly=True)

    # -- connections ----------------------------------------------------------------
    def synapse(self, sig, tau, label="synapse", out=None):
        """Filtered copy of ``sig`` (updated at the end of the step), optionally
        written into a given signal (e.g. a slice of an exchange buffer)."""
        if tau is None:
            return sig
        if out is None:
            out = m.Signal(np.zeros(sig.shape), name="%s.filtered" % label)
        self.model.add_op(m.SimProcess(m.Lowpass(tau), sig, out, self.model.time, mode="update"))
        return out

    def connect_signal(self, src, dst, synapse=None, transform=None, label="conn"):
        """src -> [transform] -> [synapse] -> dst (increment)."""
        mdl = self.model
        sig = src
        if transform is not None:
            T = np.asarray(transform, dtype=np.float64)
            w = m.Signal(T, name="%s.weights" % label, readonly=True)
            weighted = m.Signal(np.zeros(T.shape[0] if T.ndim == 2 else src.shape), name="%s.weighted" % label)
            mdl.add_op(m.Reset(weighted))
            mdl.add_op(m.DotInc(w, src, weighted, tag="%s.transform" % label))
            sig = weighted
        sig = self.synapse(sig, synapse, label)
        mdl.add_op(m.Copy(sig, dst, inc=True))
        return sig

    def connect_decoded(self, pre, dst, decoders, synapse=0.005, label=None, pes=None, out_signal=None):
        """Decoded connection from ensemble ``pre`` into signal ``dst``.

        ``pes`` = dict(learning_rate, error (Signal), pre_synapse) adds the PES rule:
        a lowpass of the presynaptic activities, the delta operator and the
        increment of the decoders by the previous step's delta."""
        mdl = self.model
        label = label or "conn%d" % len(self.connections)
        dec = np.asarray(decoders, dtype=np.float64)
        w = m.Signal(dec, name="%s.weights" % label, readonly=pes is None)
        weighted = m.Signal(np.zeros(dec.shape[0]), name="%s.weighted" % label)
        mdl.add_op(m.Reset(weighted))
        mdl.add_op(m.DotInc(w, pre.sig_out, weighted, tag="%s.decode" % label))
        out = self.synapse(weighted, synapse, label, out=out_signal)
        if dst is not None:
            mdl.add_op(m.Copy(out, dst, inc=True))
        conn = dict(pre=pre, weights=w, weighted=weighted, out=out, label=label)
        if pes is not None:
            pre_f = m.Signal(np.zeros(pre.n_neurons), name="%s.pes.pre_filtered" % label)
            mdl.add_op(m.SimProcess(m.Lowpass(pes.get("pre_synapse", 0.005)), pre.sig_out, pre_f, mdl.time,
                                    mode="update"))
            delta = m.Signal(np.zeros(dec.shape), name="%s.pes.delta" % label)
            mdl.add_op(m.SimPES(pre_f, pes["error"], delta, pes["learning_rate"]))
            mdl.add_op(m.Copy(delta, w, inc=True, tag="%s.pes.apply" % label))
            conn.update(pre_filtered=pre_f, delta=delta, error=pes["error"])
        self.connections.append(conn)
        return conn

    def probe(self, sig, synapse=None, sample_every=None, label=None):
        filtered = self.synapse(sig, synapse, label or "probe")
        return self.model.add_probe(filtered, sample_every=sample_every, label=label)

    def probe_decoded(self, ens, synapse=0.01, function=None, label=None):
        dec = self.solve_decoders(ens, function=function)
        conn = self.connect_decoded(ens, None, dec, synapse=synapse, label=label or "%s.probe" % ens.label)
        return self.model.add_probe(conn["out"], label=label or "%s.probe" % ens.label)


# ---- configuration 1: two-ensemble communication channel ------------------------
def two_ensemble_model(seed=0, n_neurons=100, dt=0.001):
    """Node(sin t) -> A (100 LIF, 1-d) -> x**2 -> B (100 LIF, 1-d); both decoded
    outputs probed through a 0.01 s lowpass."""
    nb = NetBuilder(dt=dt, seed=seed, label="two ensembles")
    stim = nb.node_fn(lambda t: np.sin(t), 1, label="stim")
    A = nb.ensemble(n_neurons, 1, label="A")
    B = nb.ensemble(n_neurons, 1, label="B")
    nb.connect_signal(stim, A.sig_in, synapse=None, label="stim->A")
    nb.connect_decoded(A, B.sig_in, nb.solve_decoders(A, function=lambda x: x ** 2), synapse=0.005, label="A->B")
    pA = nb.probe_decoded(A, synapse=0.01, label="A.probe")
    pB = nb.probe_decoded(B, synapse=0.01, label="B.probe")
    nb.model.info = dict(probes=dict(A=pA, B=pB), ensembles=nb.ensembles, connections=nb.connections)
    return nb.model


# ---- configuration 4: Watts-Strogatz ring of ensembles --------------------------
def watts_strogatz_edges(n, k, p, rng):
    """Ring lattice with k neighbours per side; each edge's source is rewired
    with probability p (no self loops, no duplicate edges per target)."""
    edges = []
    for i in range(n):
        sources = [(i + o) % n for o in range(-k, k + 1) if o != 0]
        for j, s in enumerate(sources):
            if rng.uniform() < p:
                s = int(rng.randint(n))
                while s == i or s in sources:
                    s = int(rng.randint(n))
                sources[j] = s
        edges.extend((s, i) for s in sources)
    return edges


def watts_strogatz_model(seed=2, n_ensembles=4096, n_neurons=50, k=4, p=0.1, synapse=0.01, dt=0.001,
                         n_templates=16, n_probes=4):
    """Every edge is a decoded connection (identity decoders scaled by a U(-1,1)
    weight) with its own lowpass state; sin(t) drives ensemble 0.  Ensemble
    parameters are drawn for ``n_templates`` distinct ensembles and reused
    round-robin to bound the build time (each ensemble still owns its arrays)."""
    nb = NetBuilder(dt=dt, seed=seed, label="watts-strogatz")
    rng = nb.rng
    templates, decoders, ens = [], [], []
    for i in range(n_ensembles):
        t = templates[i % n_templates] if i >= n_templates else None
        e = nb.ensemble(n_neurons, 1, label="e%d" % i, params_from=t)
        if t is None:
            templates.append(e)
            decoders.append(nb.solve_decoders(e))
        ens.append(e)
    edges = watts_strogatz_edges(n_ensembles, k, p, rng)
    weights = rng.uniform(-1, 1, size=len(edges))
    for (s, d), wgt in zip(edges, weights):
        nb.connect_decoded(ens[s], ens[d].sig_in, wgt * decoders[s % n_templates], synapse=synapse,
                           label="e%d->e%d" % (s, d))
    stim = nb.node_fn(lambda t: np.sin(t), 1, label="stim")
    nb.connect_signal(stim, ens[0].sig_in, synapse=None, label="stim->e0")
    probes = [nb.model.add_probe(ens[i].sig_in, label="e%d.in" % i)
              for i in np.linspace(0, n_ensembles - 1, n_probes).astype(int)]
    nb.model.info = dict(probes=probes, ensembles=nb.ensembles, connections=nb.connections, edges=edges)
    return nb.model


def watts_strogatz_shard(seed=2, n_ensembles=4096, rank=0, world=1, n_neurons=50, k=4, p=0.1, synapse=0.01,
                         dt=0.001, n_templates=16, n_probes=4, max_out=16):
    """Shard ``rank`` of ``world`` of the Watts-Strogatz network (``n_ensembles`` a multiple of
    ``world``), in the same way as ``pes_learning_shard``: the whole network is described by
    seeded draws that do not depend on the rank; a shard instantiates its contiguous block of
    ensembles, their OUTGOING edges (decoders live with the source ensemble) and the increments
    of its own ensembles' inputs.  The filtered value of the j-th outgoing edge of ensemble ``s``
    lives in slot ``s * max_out + j`` of one ``exchange`` signal (identical layout on every rank;
    unused slots stay zero), so a rank's slots are one contiguous segment and the only cross-rank
    data per step are the other ranks' segments.  With ``world == 1`` this is the complete model
    (the unsharded reference of the sharded runs)."""
    assert n_ensembles % world == 0
    n_local = n_ensembles // world
    lo = rank * n_local
    nb = NetBuilder(dt=dt, seed=seed, label="watts-strogatz shard %d/%d" % (rank, world))
    trng = np.random.RandomState(seed)
    scratch = NetBuilder(dt=dt, seed=seed)  # template ensembles are solved outside the shard's model
    scratch.rng = trng
    templates = [scratch.ensemble(n_neurons, 1, label="template%d" % t) for t in range(n_templates)]
    decoders = [scratch.solve_decoders(t) for t in templates]
    grng = np.random.RandomState(seed + 1)
    edges = watts_strogatz_edges(n_ensembles, k, p, grng)
    weights = grng.uniform(-1, 1, size=len(edges))
    out_index, out_count = [], np.zeros(n_ensembles, dtype=np.int64)
    for s_, _ in edges:
        out_index.append(int(out_count[s_]))
        out_count[s_] += 1
    assert out_count.max() <= max_out, "an ensemble has more than max_out outgoing edges"

    exchange = m.Signal(np.zeros(n_ensembles * max_out), name="exchange")
    slot = lambda s_, j: exchange[s_ * max_out + j:s_ * max_out + j + 1]
    ens = {}
    for g in range(lo, lo + n_local):
        ens[g] = nb.ensemble(n_neurons, 1, label="e%d" % g, params_from=templates[g % n_templates])
    # inputs of local ensembles: every edge (from any rank) that targets them, in edge order
    for e_i, (s_, d_) in enumerate(edges):
        if lo <= d_ < lo + n_local:
            nb.model.add_op(m.Copy(slot(s_, out_index[e_i]), ens[d_].sig_in, inc=True))
    # outgoing edges of local ensembles
    for e_i, (s_, d_) in enumerate(edges):
        if lo <= s_ < lo + n_local:
            nb.connect_decoded(ens[s_], None, weights[e_i] * decoders[s_ % n_templates], synapse=synapse,
                               label="e%d->e%d" % (s_, d_), out_signal=slot(s_, out_index[e_i]))
    if lo == 0:
        stim = nb.node_fn(lambda t: np.sin(t), 1, label="stim")
        nb.connect_signal(stim, ens[0].sig_in, synapse=None, label="stim->e0")
    probe_ids = [lo + int(i) for i in np.linspace(0, n_local - 1, n_probes).astype(int)]
    probes = [nb.model.add_probe(ens[g].sig_in, label="e%d.in" % g) for g in probe_ids]
    nb.model.info = dict(probes=probes, probe_ids=probe_ids, ensembles=nb.ensembles, connections=nb.connections,
                         edges=edges, exchange=exchange, segment=(lo * max_out, n_local * max_out), rank=rank,
                         world=world)
    return nb.model


# ---- sparse recurrent population (the reference's own Watts-Strogatz benchmark) ------
def watts_strogatz_adjacency(n, fan_out, rewire, rng, scale=None):
    """Sparse (n, n) float32 weights: column j feeds the rows j +- 1 .. fan_out / 2 of
    a ring; every edge is moved to a random row with probability ``rewire``
    (duplicates are summed); weights U(-1, 1) * scale."""
    import scipy.sparse as sp

    half = max(fan_out // 2, 1)
    offs = np.concatenate([np.arange(-half, 0), np.arange(1, half + 1)])
    cols = np.repeat(np.arange(n), len(offs))
    rows = (cols + np.tile(offs, n)) % n
    moved = rng.uniform(size=rows.size) < rewire
    rows = np.where(moved, rng.randint(n, size=rows.size), rows)
    scale = 1.0 / len(offs) if scale is None else scale
    vals = (rng.uniform(-1, 1, size=rows.size) * scale).astype(np.float32)
    mat = sp.coo_matrix((vals, (rows, cols)), shape=(n, n)).tocsr()
    mat.sum_duplicates()
    return mat


def sparse_recurrent_model(seed=9, n_neurons=2000, fan_out=50, rewire=0.1, synapse=0.1, probe_synapse=0.03,
                           dt=0.001, tau_ref=0.001):
    """One population with a sparse neuron-to-neuron recurrent connection (the
    shape of examples/benchmark_wattsstrogatz.py:69-87 of the reference): the
    spikes go through a sparse matrix, a lowpass synapse and back into the input
    currents; the filtered spikes are probed."""
    nb = NetBuilder(dt=dt, seed=seed, label="sparse recurrent")
    ens = nb.ensemble(n_neurons, 1, label="ens", neuron_type=m.LIF(tau_ref=tau_ref))
    W = m.Signal(watts_strogatz_adjacency(n_neurons, fan_out, rewire, nb.rng), name="recurrent.weights",
                 readonly=True)
    weighted = m.Signal(np.zeros(n_neurons), name="recurrent.weighted")
    nb.model.add_op(m.Reset(weighted))
    nb.model.add_op(m.SparseDotInc(W, ens.sig_out, weighted, tag="recurrent.sparse"))
    filtered = nb.synapse(weighted, synapse, "recurrent")
    nb.model.add_op(m.Copy(filtered, ens.sig_J, inc=True))
    probe = nb.probe(ens.sig_out, synapse=probe_synapse, label="ens.neurons")
    nb.model.info = dict(probes=[probe], ensembles=nb.ensembles, connections=[], weights=W)
    return nb.model


# ---- configuration 3: circular convolution through product ensembles ------------
def circular_convolution_model(seed=4, dimensions=256, n_neurons=200, synapse=0.005, dt=0.001, n_templates=8):
    """c = a (*) b computed in the Fourier domain by 2-d product ensembles.

    Both inputs are seeded unit vectors held constant.  A real DFT of each
    input (``dimensions // 2 + 1`` complex bins) is formed by dense transforms;
    every complex product (ar + i ai)(br + i bi) takes four real products, each
    computed by one ensemble of ``n_neurons`` LIF neurons representing the pair
    of factors (4 * (D/2 + 1) ensembles, 516 for D = 256); a third dense
    transform combines the products and applies the inverse real DFT.  All
    three connections carry a lowpass synapse.  (A construction of the same
    shapes as a nengo circular-convolution network; the ensemble count of the
    library network is not reproduced from it.)"""
    nb = NetBuilder(dt=dt, seed=seed, label="circular convolution")
    rng = nb.rng
    D = int(dimensions)
    nbins = D // 2 + 1
    a = rng.standard_normal(D)
    b = rng.standard_normal(D)
    a /= np.linalg.norm(a)
    b /= np.linalg.norm(b)
    # real DFT as a matrix: rows (re_0 .. re_{nb-1}, im_0 .. im_{nb-1}); unit vectors give O(1) bins
    k = np.arange(nbins)[:, None] * np.arange(D)[None, :]
    F = np.concatenate([np.cos(2 * np.pi * k / D), -np.sin(2 * np.pi * k / D)], axis=0)  # (2 nbins, D)
    re, im = np.arange(nbins), nbins + np.arange(nbins)
    # product p = 4 * bin + {0: ar*br, 1: ai*bi, 2: ar*bi, 3: ai*br}
    rows_a = np.stack([re, im, re, im], axis=1).reshape(-1)
    rows_b = np.stack([re, im, im, re], axis=1).reshape(-1)
    n_prod = 4 * nbins
    Ta, Tb = F[rows_a], F[rows_b]
    sa = nb.node_const(a, label="a")
    sb = nb.node_const(b, label="b")
    fa = m.Signal(np.zeros(n_prod), name="A.factors")
    fb = m.Signal(np.zeros(n_prod), name="B.factors")
    for src, T, dst, label in ((sa, Ta, fa, "a->factors"), (sb, Tb, fb, "b->factors")):
        w = m.Signal(T, name="%s.weights" % label, readonly=True)
        weighted = m.Signal(np.zeros(n_prod), name="%s.weighted" % label)
        nb.model.add_op(m.Reset(weighted))
        nb.model.add_op(m.DotInc(w, src, weighted, tag="%s.transform" % label))
        nb.synapse(weighted, synapse, label, out=dst)
    templates, decoders, ens = [], [], []
    products = m.Signal(np.zeros(n_prod), name="products")
    for p_i in range(n_prod):
        t = templates[p_i % n_templates] if p_i >= n_templates else None
        e = nb.ensemble(n_neurons, 2, label="prod%d" % p_i, radius=np.sqrt(2.0), params_from=t)
        if t is None:
            templates.append(e)
            decoders.append(nb.solve_decoders(e, function=lambda x: x[0] * x[1]))
        ens.append(e)
        nb.model.add_op(m.Copy(fa[p_i:p_i + 1], e.sig_in[0:1], inc=True))
        nb.model.add_op(m.Copy(fb[p_i:p_i + 1], e.sig_in[1:2], inc=True))
        nb.connect_decoded(e, None, decoders[p_i % n_templates], synapse=synapse, label="prod%d.out" % p_i,
                           out_signal=products[p_i:p_i + 1])
    # combine: Re = ar br - ai bi, Im = ar bi + ai br; inverse real DFT
    C = np.zeros((2 * nbins, n_prod))
    for bin_ in range(nbins):
        C[bin_, 4 * bin_ + 0], C[bin_, 4 * bin_ + 1] = 1.0, -1.0
        C[nbins + bin_, 4 * bin_ + 2], C[nbins + bin_, 4 * bin_ + 3] = 1.0, 1.0
    wgt = np.full(nbins, 2.0)
    wgt[0] = 1.0
    if D % 2 == 0:
        wgt[-1] = 1.0
    kk = np.arange(D)[:, None] * np.arange(nbins)[None, :]
    Finv = np.concatenate([wgt * np.cos(2 * np.pi * kk / D), -wgt * np.sin(2 * np.pi * kk / D)], axis=1) / D
    out = m.Signal(np.zeros(D), name="c.in")
    nb.model.add_op(m.Reset(out))
    w = m.Signal(Finv @ C, name="products->c.weights", readonly=True)
    nb.model.add_op(m.DotInc(w, products, out, tag="products->c.transform"))
    probe = nb.probe(out, synapse=0.01, label="c")
    exact = np.fft.irfft(np.fft.rfft(a) * np.fft.rfft(b), n=D)
    nb.model.info = dict(probes=[probe], ensembles=nb.ensembles, connections=nb.connections, a=a, b=b,
                         exact=exact, n_products=n_prod)
    return nb.model


# ---- configuration 5: large PES learning model -----------------------------------
def pes_learning_model(seed=3, n_ensembles=4096, n_neurons=1024, dimensions=16, learning_rate=1e-4,
                       synapse=0.01, pre_synapse=0.005, dt=0.001, sim_time=0.5, n_templates=8, n_probes=4,
                       error_cutoff=5.0):
    """Each ensemble has one decoded connection to a random other ensemble with
    a PES rule; the error of every rule is band-limited white noise (5 Hz)
    played back from a table.  Parameters/decoders come from ``n_templates``
    solved ensembles reused round-robin (every ensemble owns its own arrays)."""
    nb = NetBuilder(dt=dt, seed=seed, label="pes learning")
    rng = nb.rng
    templates, decoders, ens = [], [], []
    for i in range(n_ensembles):
        t = templates[i % n_templates] if i >= n_templates else None
        e = nb.ensemble(n_neurons, dimensions, label="e%d" % i, params_from=t)
        if t is None:
            templates.append(e)
            decoders.append(nb.solve_decoders(e, n_eval=2 * n_neurons))
        ens.append(e)
    n_table = int(round(sim_time / dt))
    targets = rng.randint(n_ensembles - 1, size=n_ensembles)
    targets = np.where(targets >= np.arange(n_ensembles), targets + 1, targets)  # never itself
    for i, e in enumerate(ens):
        err_proc = m.WhiteSignal(sim_time, error_cutoff, rms=0.3, seed=int(rng.randint(2 ** 31 - 1)), dt=dt,
                                 size_out=dimensions)
        assert err_proc.signal.shape == (n_table, dimensions)
        err_node = nb.node_process(err_proc, dimensions, label="err%d" % i)
        err_in = m.Signal(np.zeros(dimensions), name="c%d.pes.in" % i)
        nb.model.add_op(m.Reset(err_in))
        nb.model.add_op(m.Copy(err_node, err_in, inc=True))
        nb.connect_decoded(e, ens[int(targets[i])].sig_in, decoders[i % n_templates], synapse=synapse,
                           label="c%d" % i, pes=dict(learning_rate=learning_rate, error=err_in,
                                                     pre_synapse=pre_synapse))
    probes = [nb.model.add_probe(nb.connections[i]["out"], label="c%d.out" % i)
              for i in np.linspace(0, n_ensembles - 1, n_probes).astype(int)]
    nb.model.info = dict(probes=probes, ensembles=nb.ensembles, connections=nb.connections, targets=targets)
    return nb.model


# ---- sharded form of the PES model (one shard per GPU) ---------------------------
def pes_learning_shard(seed=3, n_ensembles=4096, rank=0, world=1, n_neurons=1024, dimensions=16,
                       learning_rate=1e-4, synapse=0.01, pre_synapse=0.005, dt=0.001, sim_time=0.5,
                       n_templates=8, n_probes=4, error_cutoff=5.0):
    """Shard ``rank`` of ``world`` of the PES learning model with ``n_ensembles``
    ensembles in total (``n_ensembles`` must be a multiple of ``world``).

    The whole network is described by seeded draws that do not depend on the
    rank (template parameters, connection targets, error seeds); a shard then
    instantiates only its contiguous block of ensembles, their outgoing
    connections and the increments of its own ensembles' inputs.  The filtered
    output of connection ``g`` lives in slot ``g`` of one ``exchange`` signal
    (``n_ensembles * dimensions`` floats, identical layout on every rank): a
    rank writes the slots of its own connections and reads any slot, so the only
    cross-rank data per step are the other ranks' segments of that signal.
    With ``world == 1`` this is the complete model."""
    assert n_ensembles % world == 0
    n_local = n_ensembles // world
    lo = rank * n_local
    nb = NetBuilder(dt=dt, seed=seed, label="pes learning shard %d/%d" % (rank, world))
    # rank-independent description of the network
    trng = np.random.RandomState(seed)
    nb.rng = trng
    scratch = NetBuilder(dt=dt, seed=seed)  # template ensembles are solved outside the shard's model
    scratch.rng = trng
    templates = [scratch.ensemble(n_neurons, dimensions, label="template%d" % k) for k in range(n_templates)]
    decoders = [scratch.solve_decoders(t, n_eval=2 * n_neurons) for t in templates]
    grng = np.random.RandomState(seed + 1)
    targets = grng.randint(n_ensembles - 1, size=n_ensembles)
    targets = np.where(targets >= np.arange(n_ensembles), targets + 1, targets)
    err_seeds = np.random.RandomState(seed + 2).randint(2 ** 31 - 1, size=n_ensembles)

    exchange = m.Signal(np.zeros(n_ensembles * dimensions), name="exchange")
    slot = lambda g: exchange[g * dimensions:(g + 1) * dimensions]
    ens = {}
    for g in range(lo, lo + n_local):
        ens[g] = nb.ensemble(n_neurons, dimensions, label="e%d" % g, params_from=templates[g % n_templates])
    # inputs of local ensembles: every connection (from any rank) that targets them
    for g in np.flatnonzero((targets >= lo) & (targets < lo + n_local)):
        nb.model.add_op(m.Copy(slot(int(g)), ens[int(targets[g])].sig_in, inc=True))
    for g in range(lo, lo + n_local):
        err_proc = m.WhiteSignal(sim_time, error_cutoff, rms=0.3, seed=int(err_seeds[g]), dt=dt, size_out=dimensions)
        err_node = nb.node_process(err_proc, dimensions, label="err%d" % g)
        err_in = m.Signal(np.zeros(dimensions), name="c%d.pes.in" % g)
        nb.model.add_op(m.Reset(err_in))
        nb.model.add_op(m.Copy(err_node, err_in, inc=True))
        nb.connect_decoded(ens[g], None, decoders[g % n_templates], synapse=synapse, label="c%d" % g,
                           pes=dict(learning_rate=learning_rate, error=err_in, pre_synapse=pre_synapse),
                           out_signal=slot(g))
    probe_ids = [lo + int(i) for i in np.linspace(0, n_local - 1, n_probes).astype(int)]
    probes = [nb.model.add_probe(slot(g), label="c%d.out" % g) for g in probe_ids]
    nb.model.info = dict(probes=probes, probe_ids=probe_ids, ensembles=nb.ensembles, connections=nb.connections,
                         targets=targets, exchange=exchange, segment=(lo * dimensions, n_local * dimensions),
                         rank=rank, world=world)
    return nb.model


def white_noise_model(seed=21, n=300):
    """Two white-noise processes: a scaled Gaussian set into a signal with a lowpass behind it, and an
    unscaled uniform one incremented into a signal (a random walk).  Seeds are explicit, so the CPU
    oracle draws the same Philox stream."""
    mdl = m.Model(dt=0.001)
    a = m.Signal(np.zeros(n), name="noise")
    b = m.Signal(np.ones(7), name="walk")
    fa = m.Signal(np.zeros(n), name="noise.filtered")
    gauss = m.WhiteNoise(m.Gaussian(0.1, 0.5), scale=True, seed=seed)
    unif = m.WhiteNoise(m.Uniform(-1, 1), scale=False, seed=(seed + 1) | (7 << 32))
    mdl.add_op(m.SimProcess(gauss, None, a, mdl.step, mode="set"))
    mdl.add_op(m.SimProcess(unif, None, b, mdl.step, mode="inc"))
    mdl.add_op(m.SimProcess(m.Lowpass(0.01), a, fa, mdl.step, mode="update"))
    probes = [mdl.add_probe(fa, label="noise.filtered"), mdl.add_probe(b, label="walk")]
    mdl.info = dict(probes=probes, noise=a, walk=b, seeds=(gauss.seed, unif.seed))
    return mdl


def convolution_model(seed=31, channels_last=True, one_d=False):
    """An image signal (a sine pattern that moves with time, from a node function) through a strided
    "same" convolution into a rate layer, then a "valid" convolution of that layer's output: the
    operators a nengo Convolution transform builds (Reset, ConvInc, SimNeurons)."""
    rng = np.random.RandomState(seed)
    mdl = m.Model(dt=0.001)
    if one_d:
        shape_in, k1, st1, k2 = ((16, 2) if channels_last else (2, 16)), (3,), (2,), (2,)
    else:
        shape_in, k1, st1, k2 = ((9, 8, 2) if channels_last else (2, 9, 8)), (3, 3), (2, 1), (2, 3)
    conv1 = m.Convolution(5, shape_in, kernel_size=k1, strides=st1, padding="same", channels_last=channels_last)
    conv2 = m.Convolution(3, conv1.output_shape, kernel_size=k2, strides=(1,) * len(k2), padding="valid",
                          channels_last=channels_last)
    n_in, n_mid, n_out = (int(np.prod(s)) for s in (shape_in, conv1.output_shape, conv2.output_shape))
    image = m.Signal(rng.uniform(-1, 1, size=n_in), name="image")
    w1 = m.Signal(rng.normal(scale=0.5, size=conv1.kernel_shape), name="w1", readonly=True)
    w2 = m.Signal(rng.normal(scale=0.5, size=conv2.kernel_shape), name="w2", readonly=True)
    j1 = m.Signal(np.zeros(n_mid), name="j1")
    r1 = m.Signal(np.zeros(n_mid), name="r1")
    y2 = m.Signal(np.zeros(n_out), name="y2")
    noise = m.WhiteNoise(m.Uniform(-0.1, 0.1), scale=False, seed=seed)
    mdl.add_op(m.SimProcess(noise, None, image, mdl.step, mode="inc"))  # the image drifts
    mdl.add_op(m.Reset(j1))
    mdl.add_op(m.ConvInc(w1, image, j1, conv1))
    mdl.add_op(m.SimNeurons(m.RectifiedLinear(), j1, r1))
    mdl.add_op(m.Reset(y2))
    mdl.add_op(m.ConvInc(w2, r1, y2, conv2))
    probes = [mdl.add_probe(y2, label="y2"), mdl.add_probe(j1, label="j1")]
    mdl.info = dict(probes=probes, signals=[image, j1, r1, y2], convs=(conv1, conv2))
    return mdl
