"""Elementwise / neuron / filter / probe plans on the GPU through the C ABI,
against the CPU oracle and the outputs of the reference's own kernels
(tests/golden/kernels.npz).  Structure follows the reference's
nengo_ocl/tests/test_clra_nonlinearities.py:35-406.

Tolerances: copy / reset / sliced copy / elementwise / relu / spiking relu /
linear filter are mul-add only and compiled without FMA contraction: bit-exact.
Kernels calling expm1/log1p/exp differ from the oracle by the math library:
rtol 1e-5, atol 1e-6."""

import numpy as np
import pytest

from nengo_ocl_b200 import cura_nonlinearities as nl
from nengo_ocl_b200.curaggedarray import CUDARaggedArray as CLRA
from nengo_ocl_b200.raggedarray import RaggedArray
from nengo_ocl_b200.runtime import to_device
from oracle import kernels as K

pytestmark = pytest.mark.gpu
RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)


def ragged_like(buf, shapes):
    out = RA([np.zeros(s) for s in shapes])
    out.buf[...] = buf
    return out


def test_lif_step_matches_reference_kernel(queue, golden_kernels, golden_tables):
    g = golden_kernels
    sizes = [int(s) for s in g["lif/sizes"]]
    split = lambda buf: RA(np.split(buf, np.cumsum(sizes)[:-1]))
    for up in (1, 4):
        key = "lif_up%d/" % up
        clJ, clV, clW = (CLRA(queue, split(g[key + k])) for k in ("J", "V0", "W0"))
        clS = CLRA(queue, RA([np.zeros(n) for n in sizes]))
        clT = CLRA(queue, split(g[key + "tau"]))
        plan = nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0, upsample=up)
        # block tables equal the reference's
        t = golden_tables
        assert plan.gsize == tuple(t["lif_up%d/gsize" % up])
        assert np.array_equal(plan.tables["sizes"], t["lif_up%d/sizes" % up])
        assert np.array_equal(plan.tables["J_starts"], t["lif_up%d/J_starts" % up])
        assert plan.bw_per_call == int(t["lif_up%d/bw" % up])
        plan()
        assert np.allclose(clV.cl_buf.get(), g[key + "V1"], rtol=1e-5, atol=1e-6)
        assert np.allclose(clW.cl_buf.get(), g[key + "W1"], rtol=1e-5, atol=1e-6)
        assert np.array_equal(clS.cl_buf.get(), g[key + "S1"])


def test_lif_large_populations_vs_oracle(queue):
    """reference test_lif_step sizes (12k-35k neurons), float parameters"""
    rng = np.random.RandomState(5)
    dt = 1e-3
    n_neurons = [12345, 23456, 34567]
    J = RA([rng.normal(scale=1.2, size=n) for n in n_neurons])
    V = RA([rng.uniform(low=0, high=1, size=n) for n in n_neurons])
    W = RA([rng.uniform(low=-5 * dt, high=5 * dt, size=n) for n in n_neurons])
    OS = RA([np.zeros(n) for n in n_neurons])
    taus = rng.uniform(low=15e-3, high=80e-3, size=len(n_neurons))
    T = RA([t * np.ones(n) for t, n in zip(taus, n_neurons)])
    clJ, clV, clW, clOS, clT = (CLRA(queue, r) for r in (J, V, W, OS, T))
    plan = nl.plan_lif(queue, dt, clJ, clV, clW, clOS, 2e-3, clT, 1.0)
    v, w, s = K.lif(dt, J.buf, V.buf, W.buf, T.buf, np.float32(2e-3), np.float32(1.0))
    plan()
    assert (s > 0).sum() > 50
    # expm1 / log1p are correctly rounded on both sides: voltages, refractory times and spikes are
    # bit-identical (one element in a million is allowed for the double-rounding corner)
    gs, gv, gw = clOS.cl_buf.get(), clV.cl_buf.get(), clW.cl_buf.get()
    assert np.count_nonzero(gs != s) + np.count_nonzero(gv != v) + np.count_nonzero(gw != w) <= 3 * s.size // 1000000
    assert np.array_equal(clJ.cl_buf.get(), J.buf)


def test_lif_fifty_steps(queue, golden_kernels):
    g = golden_kernels
    n = g["lif50/J"].size
    clJ = CLRA(queue, RA([g["lif50/J"]]))
    clV, clW, clS = (CLRA(queue, RA([np.zeros(n)])) for _ in range(3))
    plan = nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, 0.02, 1.0)
    counts = np.zeros(n, dtype=np.int32)
    for _ in range(50):
        plan()
        counts += clS.cl_buf.get() > 0
    moved = np.abs(counts - g["lif50/spike_counts"])
    assert moved.max() <= 1 and (moved > 0).mean() < 2e-3
    same = moved == 0
    assert np.allclose(clV.cl_buf.get()[same], g["lif50/V"][same], rtol=1e-4, atol=1e-5)


def test_rate_and_static_neurons(queue, golden_kernels):
    g = golden_kernels
    sizes = [int(s) for s in g["lif/sizes"]]
    split = lambda buf: RA(np.split(np.asarray(buf, dtype=np.float32), np.cumsum(sizes)[:-1]))
    clJ = CLRA(queue, split(g["lif_up1/J"]))
    clT = CLRA(queue, split(g["lif_up1/tau"]))
    clR = CLRA(queue, RA([np.zeros(n) for n in sizes]))
    nl.plan_lif_rate(queue, 1e-3, clJ, clR, 2e-3, clT, 1.0)()
    assert np.allclose(clR.cl_buf.get(), g["lif_rate/R"], rtol=1e-5, atol=1e-6)
    amp = CLRA(queue, RA([1.5 * np.ones(n) for n in sizes]))
    nl.plan_rectified_linear(queue, clJ, clR, amp)()
    assert np.array_equal(clR.cl_buf.get(), g["relu/R"])
    clJ2 = CLRA(queue, split(g["spikingrelu/J"]))
    clV = CLRA(queue, split(g["lif_up1/V0"]))
    nl.plan_spiking_rectified_linear(queue, 1e-3, clJ2, clV, clR, amp)()
    assert np.array_equal(clV.cl_buf.get(), g["spikingrelu/V1"])
    assert np.array_equal(clR.cl_buf.get(), g["spikingrelu/S"])
    clJ3 = CLRA(queue, split(g["sigmoid/J"]))
    nl.plan_sigmoid(queue, clJ3, clR, 0.0025)()
    assert np.allclose(clR.cl_buf.get(), g["sigmoid/R"], rtol=1e-5, atol=1e-6)


def test_copy_and_elementwise_and_reset_and_slicedcopy(queue, golden_kernels, golden_tables):
    g, t = golden_kernels, golden_tables
    shapes = [(3, 5), (1, 1), (700, 1), (40, 13)]
    clX = CLRA(queue, ragged_like(g["copy/X"], shapes))
    clY = CLRA(queue, ragged_like(g["copy/Y0"], shapes))
    plan = nl.plan_copy(queue, clX, clY, np.array([0, 1, 1, 0], dtype=np.int32))
    assert np.array_equal(plan.tables["offsets"], t["copy/offsets"])
    plan()
    assert np.array_equal(clY.cl_buf.get(), g["copy/Y1"])

    clA = CLRA(queue, ragged_like(g["ewinc/A"], [(3, 5), (1, 1), (700, 1), (1, 13)]))
    clXe = CLRA(queue, ragged_like(g["ewinc/X"], [(3, 1), (1, 1), (1, 1), (40, 13)]))
    clY = CLRA(queue, ragged_like(g["copy/Y0"], shapes))
    nl.plan_elementwise_inc(queue, clA, clXe, clY)()
    assert np.array_equal(clY.cl_buf.get(), g["ewinc/Y1"])

    dims = ((4, 50), (1, 300), (16, 1024))
    clE = CLRA(queue, ragged_like(g["outer/E"], [(d, 1) for d, _ in dims]))
    clP = CLRA(queue, ragged_like(g["outer/P"], [(n, 1) for _, n in dims]))
    clD = CLRA(queue, RA([np.ones(s) for s in dims]))
    nl.plan_elementwise_inc(queue, clE, clP, clD, alpha=g["outer/alpha"], outer=True, inc=False)()
    assert np.array_equal(clD.cl_buf.get(), g["outer/D"])

    clYr = CLRA(queue, RA([np.ones(s) for s in [(3, 5), (1, 1), (70, 1), (4, 13)]]))
    vals = to_device(queue, np.array([0.0, 1.5, -2.0, 7.0], dtype=np.float32))
    plan = nl.plan_reset(queue, clYr, vals)
    assert plan.gsize == tuple(t["reset/gsize"]) and plan.lsize == tuple(t["reset/lsize"])
    plan()
    assert np.array_equal(clYr.cl_buf.get(), g["reset/Y1"])

    clXs = CLRA(queue, ragged_like(g["slicedcopy/X"], [(10, 1), (50, 1), (33, 1)]))
    clYs = CLRA(queue, ragged_like(g["slicedcopy/Y0"], [(20, 1), (50, 1), (40, 1)]))
    xi = [np.arange(10)[::2], np.arange(50)[::-1].copy(), np.arange(33)[5:25]]
    yi = [np.arange(20)[3:8], np.arange(50), np.arange(40)[::2]]
    plan = nl.plan_slicedcopy(queue, clXs, clYs, CLRA(queue, RA(xi, np.int32)), CLRA(queue, RA(yi, np.int32)),
                              np.array([1, 0, 1], dtype=np.int32))
    plan()
    assert np.array_equal(clYs.cl_buf.get(), g["slicedcopy/Y1"])


def test_elementwise_inc_broadcasting_vs_numpy(queue, rng):
    """reference test_elementwise_inc (:194-251): scalar / row / column operands"""
    Yshapes = [(1, 1), (2, 1), (1, 5), (3, 4), (300, 1)]
    Ashapes = [(1, 1), (1, 1), (1, 5), (3, 1), (1, 1)]
    Xshapes = [(1, 1), (2, 1), (1, 1), (3, 4), (300, 1)]
    A = RA([rng.normal(size=s) for s in Ashapes])
    X = RA([rng.normal(size=s) for s in Xshapes])
    Y = RA([rng.normal(size=s) for s in Yshapes])
    clA, clX, clY = CLRA(queue, A), CLRA(queue, X), CLRA(queue, Y)
    nl.plan_elementwise_inc(queue, clA, clX, clY)()
    K.elementwise_inc(A, X, Y)
    assert np.array_equal(clY.cl_buf.get(), Y.buf)


def test_linearfilter_sequence(queue, golden_kernels):
    g = golden_kernels
    dens = [[-0.9], [], [-1.6, 0.64]]
    nums = [[0.1], [0.5], [0.02, 0.02]]
    shapes = [(300, 1), (5, 1), (64, 1)]
    cl = [CLRA(queue, RA([np.zeros(s) for s in shapes])) for _ in range(2)]
    cl += [CLRA(queue, RA(dens)), CLRA(queue, RA(nums))]
    cl += [CLRA(queue, RA([np.zeros((len(b), s[0])) for b, s in zip(nums, shapes)])),
           CLRA(queue, RA([np.zeros((len(a), s[0])) for a, s in zip(dens, shapes)]))]
    plans = nl.plan_linearfilter(queue, *cl)
    for step in range(6):
        cl[0].cl_buf.set(g["linearfilter/xs"][step])
        for p in plans:
            p()
        assert np.array_equal(cl[1].cl_buf.get(), g["linearfilter/ys"][step]), step


def test_lowpass_many_items(queue, rng):
    n_items = 3000
    X = RA([rng.normal(size=(rng.randint(1, 20), 1)) for _ in range(n_items)])
    Y = RA([rng.normal(size=X[i].shape) for i in range(n_items)])
    a = rng.uniform(-0.99, -0.5, size=n_items)
    A = RA([[v] for v in a])
    B = RA([[1 + v] for v in a])
    Xb = RA([np.zeros((1, X[i].shape[0])) for i in range(n_items)])
    Yb = RA([np.zeros((1, X[i].shape[0])) for i in range(n_items)])
    cl = [CLRA(queue, r) for r in (X, Y, A, B, Xb, Yb)]
    (plan,) = nl.plan_linearfilter(queue, *cl)
    xp, yp = np.zeros(n_items, np.int32), np.zeros(n_items, np.int32)
    for _ in range(3):
        plan()
        K.linearfilter(X, Y, A, B, Xb, Yb, xp, yp)
    assert np.array_equal(cl[1].cl_buf.get(), Y.buf)


def test_probes_timeupdate_presentinput(queue, rng):
    step = CLRA(queue, RA([[0.0]]))
    time = CLRA(queue, RA([[0.0]]))
    tplan = nl.plan_timeupdate(queue, step, time, 0.001)
    sig = RA([rng.normal(size=(4, 3)), rng.normal(size=(7, 1)), rng.normal(size=(1, 1))])
    sig.add_views([sig.starts[0] + 1], [4], [1], [3], [1])  # a column view of item 0
    X = CLRA(queue, sig)
    n_pre = 8
    periods = [1, 2, 1, 3]
    Y = CLRA(queue, RA([np.zeros((n_pre, int(s))) for s in sig.sizes]))
    pplan = nl.plan_probes(queue, periods, X, Y)
    table = RA([rng.normal(size=(5, 2)), rng.normal(size=(3, 4))])
    S = CLRA(queue, table)
    out = CLRA(queue, RA([np.zeros(2), np.zeros(4)]))
    tt = step[[0, 0]]
    iplan = nl.plan_presentinput(queue, out, tt, S, 0.001)
    cd = np.asarray(periods, np.float32) - 1
    pos = np.zeros(4, np.int32)
    Yh = RA([np.zeros((n_pre, int(s))) for s in sig.sizes])
    for i in range(6):
        tplan()
        iplan()
        pplan()
        K.probes(cd, pos, np.asarray(periods, np.float32), sig, Yh)
        assert step[0][0, 0] == i + 1
        assert time[0][0, 0] == np.float32(0.001 * (i + 1))
        assert np.array_equal(out[0][:, 0], table[0][(i + 1) % 5])
        assert np.array_equal(out[1][:, 0], table[1][(i + 1) % 3])
    assert np.array_equal(pplan.cl_bufpositions.get(), pos)
    assert pos.tolist() == [6, 3, 6, 2]
    assert np.array_equal(Y.cl_buf.get(), Yh.buf)


def test_probes_of_large_signals(queue, rng):
    """Probes larger than one CTA's share go through the several-CTAs-per-probe kernel; a
    small probe, a strided view and different periods ride along."""
    big = nl.PROBE_WIDE_ELEMENTS * 3 + 17
    sig = RA([rng.normal(size=(big, 1)), rng.normal(size=(5, 1)), rng.normal(size=(300, 40))])
    sig.add_views([sig.starts[2] + 3], [300], [1], [40], [1])  # a column of the matrix
    X = CLRA(queue, sig)
    n_pre = 5
    periods = [1, 2, 3, 1]
    Y = CLRA(queue, RA([np.zeros((n_pre, int(s))) for s in sig.sizes]))
    pplan = nl.plan_probes(queue, periods, X, Y)
    assert pplan.full_args[-1] is not None  # the arrival counters of the wide kernel
    cd = np.asarray(periods, np.float32) - 1
    pos = np.zeros(4, np.int32)
    Yh = RA([np.zeros((n_pre, int(s))) for s in sig.sizes])
    for i in range(5):
        X[1] = np.full((5, 1), float(i))  # the probed signal changes between samples
        sig[1] = np.full((5, 1), float(i))
        pplan()
        K.probes(cd, pos, np.asarray(periods, np.float32), sig, Yh)
    assert np.array_equal(pplan.cl_bufpositions.get(), pos) and pos.tolist() == [5, 2, 1, 5]
    assert np.array_equal(pplan.cl_countdowns.get(), cd)
    assert np.array_equal(pplan.full_args[-1].get(), np.zeros(4, np.int32))  # counters are left clear
    assert np.array_equal(Y.cl_buf.get(), Yh.buf)


def test_learning_rule_deltas(queue, rng):
    """plan_bcm / plan_oja / plan_voja against the oracle: bit-exact (multiply-add only), with a
    strided delta view among the items."""
    shapes = [(5, 3), (1, 7), (40, 33), (300, 17)]  # (post, pre)
    pre = RA([rng.normal(size=(n, 1)) for _, n in shapes])
    post = RA([rng.normal(size=(m, 1)) for m, _ in shapes])
    theta = RA([rng.normal(size=(m, 1)) for m, _ in shapes])
    mat = RA([rng.normal(size=sh) for sh in shapes])
    scale = RA([rng.uniform(0.5, 2, size=(m, 1)) for m, _ in shapes])
    learn = RA([rng.normal(size=(1, 1)) for _ in shapes])
    alpha = rng.uniform(-1, 1, size=len(shapes)).astype(np.float32)
    beta = rng.uniform(0, 2, size=len(shapes)).astype(np.float32)
    d_alpha, d_beta = to_device(queue, alpha), to_device(queue, beta)
    cl = lambda a: CLRA(queue, a)
    for rule in ("bcm", "oja", "voja"):
        delta = cl(RA([np.full(sh, 9.0) for sh in shapes]))
        if rule == "bcm":
            plan = nl.plan_bcm(queue, cl(pre), cl(post), cl(theta), delta, d_alpha)
        elif rule == "oja":
            plan = nl.plan_oja(queue, cl(pre), cl(post), cl(mat), delta, d_alpha, d_beta)
        else:
            plan = nl.plan_voja(queue, cl(pre), cl(post), cl(mat), delta, cl(learn), cl(scale), d_alpha)
        plan()
        assert plan.bw_per_call > 0 and plan.flops_per_call > 0
        for k, (m, n) in enumerate(shapes):
            if rule == "bcm":
                want = K.bcm(pre[k], post[k], theta[k], alpha[k])
            elif rule == "oja":
                want = K.oja(pre[k], post[k], mat[k], alpha[k], beta[k])
            else:
                want = K.voja(pre[k], post[k], mat[k], learn[k][0, 0], scale[k], alpha[k])
            assert np.array_equal(delta[k], want), (rule, k)


def test_adaptive_lif_matches_reference_kernel(queue, golden_kernels):
    """cl_alif (clra_nonlinearities.py:1028-1146 with N): three consecutive steps with the
    adaptation state carried, against outputs of the reference's own rendered kernel and, bit for
    bit, against the oracle."""
    g = golden_kernels
    sizes = [int(s) for s in g["lif/sizes"]]
    split = lambda buf: RA(np.split(buf, np.cumsum(sizes)[:-1]))
    key = "lif_up1/"
    clJ, clV, clW = (CLRA(queue, split(g[key + k])) for k in ("J", "V0", "W0"))
    clS = CLRA(queue, RA([np.zeros(n) for n in sizes]))
    clT = CLRA(queue, split(g[key + "tau"]))
    clN = CLRA(queue, split(g["alif/N0"]))
    plan = nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0, N=clN, tau_n=0.1, inc_n=0.05)
    n = sum(sizes)
    V, W, N = g[key + "V0"], g[key + "W0"], g["alif/N0"]
    for step in range(1, 4):
        plan()
        V, W, S, N = K.lif(1e-3, g[key + "J"], V, W, g[key + "tau"], np.full(n, 2e-3, np.float32),
                           np.full(n, 1.0, np.float32), N=N, tau_n=np.full(n, 0.1, np.float32),
                           inc_n=np.full(n, 0.05, np.float32))
        for got, ref in ((clV, V), (clW, W), (clS, S), (clN, N)):
            assert np.array_equal(got.cl_buf.get(), ref)
        assert np.allclose(clV.cl_buf.get(), g["alif/V%d" % step], rtol=1e-4, atol=1e-5)
        assert np.allclose(clN.cl_buf.get(), g["alif/N%d" % step], rtol=1e-4, atol=1e-6)
        assert (clS.cl_buf.get() > 0).sum() == (g["alif/S%d" % step] > 0).sum()


def test_timeupdate_and_presentinput_match_reference_kernels(queue, golden_kernels):
    g = golden_kernels
    step = CLRA(queue, RA([np.zeros((1, 1))]))
    time = CLRA(queue, RA([np.zeros((1, 1))]))
    tplan = nl.plan_timeupdate(queue, step, time, 0.001)
    for want in g["timeupdate/step_time"]:
        tplan()
        assert step[0][0, 0] == want[0] and time[0][0, 0] == want[1]
    tabs = RA([np.zeros((7, 3)), np.zeros((4, 1))])
    tabs.buf[...] = g["presentinput/tables"]
    for mode, pres in (("index", None), ("time", np.array([0.003, 0.002], np.float32))):
        S = CLRA(queue, tabs)
        Y = CLRA(queue, RA([np.zeros((3, 1)), np.zeros((1, 1))]))
        t = CLRA(queue, RA([np.zeros((1, 1)), np.zeros((1, 1))]))
        from nengo_ocl_b200.runtime import to_device

        plan = nl.plan_presentinput(queue, Y, t, S, 0.001, pres_t=None if pres is None else to_device(queue, pres))
        for i, s_ in enumerate(range(1, 13)):
            t[0] = np.full((1, 1), float(s_))
            t[1] = np.full((1, 1), float(s_))
            plan()
            assert np.array_equal(Y.cl_buf.get(), g["presentinput/%s" % mode][i]), (mode, s_)


def test_whitenoise_matches_oracle(queue):
    """plan_whitenoise (clra_nonlinearities.py:1577-1675) with the Philox generator: uniform samples are
    exact; the gaussian ones go through log / sqrt / sincos in double on both sides and are rounded
    once, so at most one in a million may differ (a double that lands on a float32 rounding boundary)."""
    from nengo_ocl_b200 import model as m

    sizes = [1, 3, 4, 5, 1023, 4097, 20000]
    dists = [m.Uniform(-1, 1), m.Gaussian(0, 1), m.Gaussian(0.5, 2), m.Uniform(0, 3), m.Gaussian(-1, 0.1),
             m.Uniform(-2, -1), m.Gaussian(0, 1)]
    seeds = [3, 3, 2 ** 40 + 17, 11, 0, 2 ** 63 - 1, 99]
    scales = np.array([0, 1, 1, 0, 1, 0, 0], np.int32)
    incs = np.array([0, 0, 1, 1, 0, 0, 1], np.int32)
    dt = 0.001
    Yh = RA([np.full(n, 0.25) for n in sizes])
    Y = CLRA(queue, Yh)
    step = CLRA(queue, RA([np.zeros((1, 1))]))
    t = step[[0] * len(sizes)]
    enums, params = nl.get_dist_enums_params(dists)
    rngs = nl.create_rngs(queue, len(sizes))
    nl.init_rngs(queue, rngs, seeds)
    plan = nl.plan_whitenoise(queue, Y, CLRA(queue, enums), CLRA(queue, params), to_device(queue, scales),
                              to_device(queue, incs), dt, rngs, t)
    total = differ = 0
    for s_ in (1, 2, 77, 4000):
        step[0] = np.full((1, 1), float(s_))
        plan()
        th = RA([np.full((1, 1), float(s_))] * len(sizes))
        K.whitenoise(Yh, th, enums, params, scales, incs, dt, seeds)
        for k, d in enumerate(dists):
            got, want = Y[k][:, 0], Yh[k][:, 0]
            if type(d).__name__ == "Uniform":
                assert np.array_equal(got, want), (k, s_)
            total += got.size
            differ += int(np.count_nonzero(got != want))
            assert np.allclose(got, want, rtol=1e-6, atol=1e-7)
    assert differ <= max(1, total // 1000000), (differ, total)


def test_whitenoise_model_matches_oracle_and_repeats_after_reset():
    from nengo_ocl_b200 import synth
    from nengo_ocl_b200.simulator import Simulator
    from oracle.simulator import OracleSimulator

    mdl = synth.white_noise_model(seed=21, n=300)
    ora = OracleSimulator(mdl)
    with Simulator(None, model=mdl) as sim:
        for _ in range(40):
            sim.step()
            ora.step()
            assert np.allclose(np.asarray(sim.signals[mdl.info["noise"]]), ora[mdl.info["noise"]], rtol=1e-6, atol=1e-7)
            assert np.array_equal(np.asarray(sim.signals[mdl.info["walk"]]), ora[mdl.info["walk"]])
        first = [sim.data[p].copy() for p in mdl.probes]
        assert np.allclose(first[0], np.array(ora.probe_data[mdl.probes[0]]), rtol=1e-5, atol=1e-6)
        assert np.array_equal(first[1], np.array(ora.probe_data[mdl.probes[1]], dtype=first[1].dtype))
        sim.reset()
        sim.run_steps(40)
        for a, p in zip(first, mdl.probes):
            assert np.array_equal(a, sim.data[p])  # the stream is a function of (seed, step, element)


@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("conv", [True, False], ids=["shared_filters", "local_filters"])
def test_conv2d_matches_oracle(queue, rng, conv, channels_last):
    """plan_conv2d (clra_nonlinearities.py:1762-1969): mul-add only, same loop order as the oracle,
    no FMA contraction: bit-exact.  Geometries: valid / same / explicit padding, strides, 1 x n kernels."""
    cases = [  # nxi, nxj, nc, nf, (si, sj), padding, strides
        (7, 9, 3, 4, (3, 2), "valid", (1, 1)),
        (12, 10, 2, 5, (3, 3), "same", (2, 1)),
        (8, 8, 1, 1, (1, 1), (0, 0), (1, 1)),
        (1, 33, 4, 6, (1, 5), "same", (1, 3)),
        (28, 28, 1, 32, (7, 7), (1, 0), (3, 2)),
    ]
    for nxi, nxj, nc, nf, (si, sj), padding, (sti, stj) in cases:
        pi, pj = (0, 0) if padding == "valid" else ((si - 1) // 2, (sj - 1) // 2) if padding == "same" else padding
        nyi, nyj = (nxi + 2 * pi - si) // sti + 1, (nxj + 2 * pj - sj) // stj + 1
        shape_in = (nxi, nxj, nc) if channels_last else (nc, nxi, nxj)
        shape_out = (nyi, nyj, nf) if channels_last else (nf, nyi, nyj)
        fshape = (si, sj, nc, nf) if conv else (nf, nc, si, sj, nyi, nyj)
        x, f = rng.normal(size=shape_in), rng.normal(size=fshape)
        y0 = rng.normal(size=shape_out)
        data = CLRA(queue, RA([np.zeros(3), x.reshape(-1), f.reshape(-1), y0.reshape(-1)]))  # unaligned starts
        want = K.conv2d(data[1], data[2], shape_in, shape_out, (si, sj), conv, padding, (sti, stj), channels_last)
        for inc in (False, True):
            data[3] = y0.reshape(-1, 1)
            plan = nl.plan_conv2d(queue, data.getitem_device(1), data.getitem_device(3), data.getitem_device(2),
                                  shape_in, shape_out, (si, sj), conv=conv, padding=padding, strides=(sti, stj),
                                  channels_last=channels_last, inc=inc)
            plan()
            ref = (data.dtype.type(0) + want) if not inc else (y0.reshape(-1).astype(np.float32) + want)
            assert np.array_equal(data[3][:, 0], ref.astype(np.float32)), (nxi, nxj, padding, inc)
        assert plan.flops_per_call == 2 * nyi * nyj * nf * nc * si * sj


def test_pool2d_matches_oracle(queue, rng):
    """plan_pool2d (:1972-2079): windows that overhang the image average what lies inside."""
    for nc, nxi, nxj, (si, sj), (sti, stj) in [(3, 8, 8, (2, 2), (2, 2)), (2, 7, 9, (3, 2), (2, 2)),
                                                 (1, 5, 5, (3, 3), (1, 1)), (4, 30, 31, (4, 4), (3, 4))]:
        nyi, nyj = -(-nxi // sti), -(-nxj // stj)
        x = rng.normal(size=(nc, nxi, nxj))
        data = CLRA(queue, RA([np.zeros(1), x.reshape(-1), np.zeros(nc * nyi * nyj)]))
        plan = nl.plan_pool2d(queue, data.getitem_device(1), data.getitem_device(2), (nc, nyi, nyj, nxi, nxj),
                              (si, sj), (sti, stj))
        plan()
        want = K.pool2d(data[1], (nc, nyi, nyj, nxi, nxj), (si, sj), (sti, stj))
        assert np.array_equal(data[2][:, 0], want)


@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("one_d", [False, True], ids=["2d", "1d"])
def test_convolution_model_matches_oracle(channels_last, one_d):
    """Reset + ConvInc + rate neurons + a second ConvInc (simulator.py:1290-1331), with a drifting
    input image: every signal bit for bit, every step."""
    from nengo_ocl_b200 import synth
    from nengo_ocl_b200.simulator import Simulator
    from oracle.simulator import OracleSimulator

    mdl = synth.convolution_model(channels_last=channels_last, one_d=one_d)
    ora = OracleSimulator(mdl)
    with Simulator(None, model=mdl) as sim:
        assert [p.name for p in sim._plans].count("cl_conv2d") == 2
        for _ in range(30):
            sim.step()
            ora.step()
            for sig in mdl.info["signals"]:
                assert np.array_equal(np.asarray(sim.signals[sig]).reshape(-1), ora[sig].reshape(-1)), sig
        for p in mdl.probes:
            assert np.array_equal(sim.data[p], np.array(ora.probe_data[p], dtype=sim.data[p].dtype))


def test_fastlif_matches_oracle_and_reference_kernel(queue, golden_kernels):
    """plan_lif(fastlif=True): bit-exact against the oracle; spikes and refractory times equal to the
    reference's kernel text, voltages within one ulp of it."""
    g = golden_kernels
    sizes = [int(s) for s in g["lif/sizes"]]
    split = lambda buf: RA(np.split(buf, np.cumsum(sizes)[:-1]))
    for up in (1, 2):
        clJ, clV, clW = (CLRA(queue, split(g["lif_up1/" + k])) for k in ("J", "V0", "W0"))
        clS = CLRA(queue, RA([np.zeros(n) for n in sizes]))
        clT = CLRA(queue, split(g["lif_up1/tau"]))
        plan = nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0, upsample=up, fastlif=True)
        V, W = g["lif_up1/V0"].copy(), g["lif_up1/W0"].copy()
        for step in range(1, 4):
            plan()
            V, W, S = K.lif(1e-3, g["lif_up1/J"], V, W, g["lif_up1/tau"], 2e-3, 1.0, upsample=up, fastlif=True)
            assert np.array_equal(clV.cl_buf.get(), V)
            assert np.array_equal(clW.cl_buf.get(), W)
            assert np.array_equal(clS.cl_buf.get(), S)
        key = "fastlif_up%d/" % up
        assert np.allclose(clV.cl_buf.get(), g[key + "V3"], rtol=1e-5, atol=1e-6)
