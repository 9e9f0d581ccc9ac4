"""Pin the CPU oracle: known answers from the reference's own tests, and
outputs of the reference's own kernel source executed on the CPU
(tests/golden/kernels.npz, made by tests/golden/make_golden.py)."""

import numpy as np
import pytest

from nengo_ocl_b200.raggedarray import RaggedArray
from oracle import kernels as K

RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)


def ragged_like(buf, shapes):
    """Ragged array with the given item shapes and flat contents."""
    out = RA([np.zeros(s) for s in shapes])
    out.buf[...] = buf
    return out


# ---- GEMV known answers (reference tests/test_clra_gemv.py:60-93) --------------
@pytest.mark.parametrize("fn", [K.gemv_ref, K.gemv_many_dots, K.gemv_block])
def test_gemv_basic_known_answer(fn):
    A = RA([[[0.1, 0.2], [0.3, 0.4]], [[0.5, 0.6]]])
    X = RA([[3, 5]])
    Y = RA([[0.0], [2, 3]])
    A_js = RA([[1], [0]], dtype=np.int32)
    X_js = RA([[0], [0]], dtype=np.int32)
    fn(1.0, A, A_js, X, X_js, 1.0, Y)
    assert np.allclose(Y[0].ravel(), [4.5])
    assert np.allclose(Y[1].ravel(), [3.3, 5.9])


def _check_from_shapes(fn, A_shapes, X_shapes, A_js, X_js, alpha=0.5, beta=0.6, gamma=0.7):
    """reference tests/test_clra_gemv.py:165-215 (RandomState(1234))"""
    rng = np.random.RandomState(1234)
    A = RA([0.1 + rng.rand(*shp) for shp in A_shapes])
    X = RA([0.1 + rng.rand(*shp) for shp in X_shapes])
    Y = RA([0.1 + rng.rand(A_shapes[A_js[ii][0]][0], X_shapes[X_js[ii][0]][1]) for ii in range(len(A_js))])
    Y0 = [np.array(Y[i]) for i in range(len(Y))]
    A_js = RA(A_js, dtype=np.int32)
    X_js = RA(X_js, dtype=np.int32)
    fn(alpha, A, A_js, X, X_js, beta, Y, gamma=gamma)
    for i in range(len(A_js)):
        ref = gamma + beta * Y0[i] + alpha * sum(
            np.dot(A[aj], X[xj]) for aj, xj in zip(A_js[i].ravel(), X_js[i].ravel()))
        assert np.allclose(ref, Y[i], atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("fn", [K.gemv_ref, K.gemv_many_dots, K.gemv_block])
def test_gemv_shapes_family(fn):
    _check_from_shapes(fn, [(1, 1)], [(1, 1)], [[0]], [[0]])
    _check_from_shapes(fn, [(10, 1)], [(1, 1)], [[0]], [[0]])
    _check_from_shapes(fn, [(2001, 1)], [(1, 1)], [[0]], [[0]])
    for ND in (2, 20, 100):
        _check_from_shapes(fn, [(10, 1 + ii % 2) for ii in range(ND)], [(1 + ii % 2, 1) for ii in range(ND)],
                           [range(ND)], [range(ND)])
    _check_from_shapes(fn, [(200, ii + 1) for ii in range(20)], [(ii + 1, 1) for ii in range(20)],
                       [range(20)], [range(20)])
    _check_from_shapes(fn, [(40, 300)], [(300, 1)], [[0]], [[0]])


def test_gemv_variants_agree_with_exact_value(rng):
    from nengo_ocl_b200.synth import gemv_workload

    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=24, max_rows=64)
    outs = []
    for fn in (K.gemv_ref, K.gemv_many_dots, K.gemv_block):
        Yc = RaggedArray.from_buffer(Y.buf.copy(), Y.starts, Y.shape0s, Y.shape1s, Y.stride0s, Y.stride1s)
        fn(0.5, A, A_js, X, X_js, 0.1, Yc)
        outs.append(Yc)
    vals, mags = K.gemv_exact(0.5, A, A_js, X, X_js, 0.1, Y)
    for Yc in outs:
        for i in range(len(Y)):
            # float32 evaluation error is bounded relative to the sum of |terms|
            assert np.all(np.abs(Yc[i][:, 0] - vals[i]) <= 1e-5 * mags[i] + 1e-7)


# ---- kernels executed from the reference's own source --------------------------
def test_lif_matches_reference_kernel(golden_kernels):
    g = golden_kernels
    for up in (1, 4):
        key = "lif_up%d/" % up
        V, W, S = K.lif(1e-3, g[key + "J"], g[key + "V0"], g[key + "W0"], g[key + "tau"],
                        np.float32(2e-3), np.float32(1.0), upsample=up)
        # same formula, libm vs correctly-rounded expm1/log1p: a few ulp at most
        assert np.allclose(V, g[key + "V1"], rtol=1e-5, atol=1e-6)
        assert np.allclose(W, g[key + "W1"], rtol=1e-5, atol=1e-6)
        assert np.array_equal(S > 0, g[key + "S1"] > 0)
        assert np.array_equal(S, g[key + "S1"])
        assert (S > 0).sum() >= 1  # the spiking branch is exercised (more so in the 50-step test)


def test_lif_fifty_steps_matches_reference_kernel(golden_kernels):
    g = golden_kernels
    J = g["lif50/J"]
    V = np.zeros_like(J)
    W = np.zeros_like(J)
    counts = np.zeros(J.shape, dtype=np.int32)
    for _ in range(50):
        V, W, S = K.lif(1e-3, J, V, W, np.float32(0.02), np.float32(2e-3), np.float32(1.0))
        counts += S > 0
    assert counts.sum() > 1000
    # a 1-ulp difference in V next to the threshold can move a spike by one step
    moved = np.abs(counts - g["lif50/spike_counts"])
    assert moved.max() <= 1 and (moved > 0).mean() < 2e-3
    same = moved == 0
    assert np.allclose(V[same], g["lif50/V"][same], rtol=1e-4, atol=1e-5)


def test_rate_neurons_match_reference_kernels(golden_kernels):
    g = golden_kernels
    J = g["lif_up1/J"]
    tau = g["lif_up1/tau"]
    assert np.allclose(K.lif_rate(J, tau, np.float32(2e-3), np.float32(1.0)), g["lif_rate/R"], rtol=1e-5,
                       atol=1e-6)
    assert np.array_equal(K.relu(J, np.float32(1.5)), g["relu/R"])
    V1, S = K.spiking_relu(1e-3, g["spikingrelu/J"], g["lif_up1/V0"], np.float32(1.5))
    assert np.array_equal(V1, g["spikingrelu/V1"]) and np.array_equal(S, g["spikingrelu/S"])
    assert np.allclose(K.sigmoid(g["sigmoid/J"], np.float32(0.0025)), g["sigmoid/R"], rtol=1e-5, atol=1e-6)


def test_copy_elementwise_reset_slicedcopy_match_reference_kernels(golden_kernels):
    g = golden_kernels
    shapes = [(3, 5), (1, 1), (700, 1), (40, 13)]
    X = ragged_like(g["copy/X"], shapes)
    Y = ragged_like(g["copy/Y0"], shapes)
    K.copy(X, Y, [0, 1, 1, 0])
    assert np.array_equal(Y.buf, g["copy/Y1"])

    A = ragged_like(g["ewinc/A"], [(3, 5), (1, 1), (700, 1), (1, 13)])
    Xe = ragged_like(g["ewinc/X"], [(3, 1), (1, 1), (1, 1), (40, 13)])
    Y = ragged_like(g["copy/Y0"], shapes)
    K.elementwise_inc(A, Xe, Y)
    assert np.array_equal(Y.buf, g["ewinc/Y1"])

    dims = ((4, 50), (1, 300), (16, 1024))
    E = ragged_like(g["outer/E"], [(d, 1) for d, _ in dims])
    P = ragged_like(g["outer/P"], [(n, 1) for _, n in dims])
    D = RA([np.zeros(s) for s in dims])
    K.elementwise_inc(E, P, D, alpha=g["outer/alpha"], outer=True, inc=False)
    assert np.array_equal(D.buf, g["outer/D"])

    Yr = RA([np.ones(s) for s in [(3, 5), (1, 1), (70, 1), (4, 13)]])
    K.reset(Yr, [0.0, 1.5, -2.0, 7.0])
    assert np.array_equal(Yr.buf, g["reset/Y1"])

    Xs = ragged_like(g["slicedcopy/X"], [(10, 1), (50, 1), (33, 1)])
    Ys = ragged_like(g["slicedcopy/Y0"], [(20, 1), (50, 1), (40, 1)])
    xi = [np.arange(10)[::2], np.arange(50)[::-1].copy(), np.arange(33)[5:25]]
    yi = [np.arange(20)[3:8], np.arange(50), np.arange(40)[::2]]
    K.slicedcopy(Xs, Ys, RA(xi, np.int32), RA(yi, np.int32), [1, 0, 1])
    assert np.array_equal(Ys.buf, g["slicedcopy/Y1"])


def test_linearfilter_matches_reference_kernel(golden_kernels):
    g = golden_kernels
    dens = [[-0.9], [], [-1.6, 0.64]]
    nums = [[0.1], [0.5], [0.02, 0.02]]
    shapes = [(300, 1), (5, 1), (64, 1)]
    X = RA([np.zeros(s) for s in shapes])
    Y = RA([np.zeros(s) for s in shapes])
    A, B = RA(dens), RA(nums)
    Xb = RA([np.zeros((len(b), s[0])) for b, s in zip(nums, shapes)])
    Yb = RA([np.zeros((len(a), s[0])) for a, s in zip(dens, shapes)])
    xpos = np.zeros(3, dtype=np.int32)
    ypos = np.zeros(3, dtype=np.int32)
    for step in range(6):
        X.buf[...] = g["linearfilter/xs"][step]
        K.linearfilter(X, Y, A, B, Xb, Yb, xpos, ypos)
        assert np.array_equal(Y.buf, g["linearfilter/ys"][step]), step


def _learning_items(gk):
    """Per item (pre, post, theta, matrix, scale, learn) of the learning-rule fixture."""
    shapes = [tuple(int(v) for v in sh) for sh in gk["learning/shapes"]]
    def split(name, sizes):
        buf, out, pos = gk["learning/%s_buf" % name], [], 0
        for n in sizes:
            out.append(buf[pos:pos + n])
            pos += n
        return out
    pre = split("pre", [n for _, n in shapes])
    post = split("post", [m for m, _ in shapes])
    theta = split("theta", [m for m, _ in shapes])
    mat = [a.reshape(sh) for a, sh in zip(split("mat", [m * n for m, n in shapes]), shapes)]
    scale = split("scale", [m for m, _ in shapes])
    learn = split("learn", [1 for _ in shapes])
    return shapes, pre, post, theta, mat, scale, learn


def test_learning_rule_deltas_match_reference_kernels(golden_kernels):
    """bcm / oja / voja restatements against the reference's kernels (multiply-add only: bit-exact)."""
    gk = golden_kernels
    shapes, pre, post, theta, mat, scale, learn = _learning_items(gk)
    alpha, beta = gk["learning/alpha"], gk["learning/beta"]
    for rule in ("bcm", "oja", "voja"):
        want, pos = gk["learning/%s_delta" % rule], 0
        for k, (m, n) in enumerate(shapes):
            if rule == "bcm":
                got = K.bcm(pre[k], post[k], theta[k], alpha[k])
            elif rule == "oja":
                got = K.oja(pre[k], post[k], mat[k], alpha[k], beta[k])
            else:
                got = K.voja(pre[k], post[k], mat[k], learn[k][0], scale[k], alpha[k])
            assert got.shape == (m, n)
            assert np.array_equal(got.reshape(-1), want[pos:pos + m * n]), (rule, k)
            pos += m * n


def test_compiled_oracle_matches_numpy_oracle():
    """oracle/cport.c (the compiled restatement used for large models and as the timed CPU
    baseline) against oracle/kernels.py on random data: block GEMV and LIF, bit for bit."""
    from oracle import cport as C
    from nengo_ocl_b200.raggedarray import RaggedArray

    rng = np.random.RandomState(5)
    for M, N in [(1, 1), (7, 3), (16, 1024), (100, 16), (33, 300), (5, 129)]:
        A = rng.randn(M, N).astype(np.float32)
        x = rng.randn(N).astype(np.float32)
        y = rng.randn(M).astype(np.float32)
        total = y.copy()
        C.block_rows(total, A, x)
        RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)
        Y = RA([y.reshape(-1, 1)])
        K.gemv_block(1.0, RA([A]), RA([[0]], np.int32), RA([x.reshape(-1, 1)]), RA([[0]], np.int32), 1.0, Y)
        assert np.array_equal(total, Y[0][:, 0])
        # strided operands (views of larger signals)
        big = rng.randn(M, 2 * N + 3).astype(np.float32)
        total = y.copy()
        C.block_rows(total, big[:, 1:2 * N + 1:2], x)
        Y2 = RA([y.reshape(-1, 1)])
        K.gemv_block(1.0, RA([np.ascontiguousarray(big[:, 1:2 * N + 1:2])]), RA([[0]], np.int32),
                     RA([x.reshape(-1, 1)]), RA([[0]], np.int32), 1.0, Y2)
        assert np.array_equal(total, Y2[0][:, 0])
    n = 5000
    J = rng.uniform(-1, 8, n).astype(np.float32)
    V = rng.uniform(0, 1, n).astype(np.float32)
    W = rng.uniform(-0.001, 0.003, n).astype(np.float32)
    for _ in range(5):
        v, w, s = K.lif(0.001, J, V, W, np.full(n, 0.02, np.float32), np.full(n, 0.002, np.float32),
                        np.full(n, 1.0, np.float32))
        Vc, Wc, Sc = V.copy(), W.copy(), np.zeros(n, np.float32)
        C.lif(0.001, J, Vc, Wc, Sc, 0.02, 0.002, 1.0)
        assert np.array_equal(v, Vc) and np.array_equal(w, Wc) and np.array_equal(s, Sc)
        V, W = v, w


def test_compiled_pes_model_step_matches_interpreter():
    """The compiled whole-step restatement of benchmark configuration 5 (oracle/pes_batch.py:
    the timed CPU baseline) against the operator-list interpreter, every array, 30 steps."""
    from nengo_ocl_b200 import synth
    from oracle.pes_batch import PesBatch
    from oracle.simulator import OracleSimulator

    mdl = synth.pes_learning_model(seed=3, n_ensembles=12, n_neurons=128, dimensions=4, n_templates=3, n_probes=2,
                                   sim_time=0.05)
    ora, batch = OracleSimulator(mdl), PesBatch(mdl)
    for _ in range(30):
        ora.step()
        batch.step()
    assert np.abs(batch.filtered).max() > 0
    for i, (c, e) in enumerate(zip(mdl.info["connections"], mdl.info["ensembles"])):
        for arr, sig in [(batch.filtered[i], c["out"]), (batch.V[i], e.state["voltage"]),
                         (batch.W[i], e.state["refractory_time"]), (batch.dec[i], c["weights"]),
                         (batch.delta[i], c["delta"]), (batch.pf[i], c["pre_filtered"]), (batch.x[i], e.sig_in),
                         (batch.S[i], e.sig_out)]:
            assert np.array_equal(arr, ora[sig].reshape(arr.shape)), (i, sig.name)


def _block_case(g, tag):
    shapes = {"three_terms": ([(40, 300), (40, 129), (40, 7)], [(40, 1)], [[0, 1, 2]]),
              "scaled": ([(70, 260), (5, 16)], [(70, 1), (5, 1)], [[0], [1]])}[tag]
    A_shapes, Y_shapes, js = shapes
    A = RaggedArray([np.zeros(s) for s in A_shapes], dtype=np.float32)
    X = RaggedArray([np.zeros((s[1], 1)) for s in A_shapes], dtype=np.float32)
    Y = RaggedArray([np.zeros(s) for s in Y_shapes], dtype=np.float32)
    A.buf[...], X.buf[...], Y.buf[...] = g["gemv_block/%s/A" % tag], g["gemv_block/%s/X" % tag], g["gemv_block/%s/Y0" % tag]
    J = RaggedArray(js, dtype=np.int32)
    alpha, beta, gamma = (float(v) for v in g["gemv_block/%s/scales" % tag])
    return A, X, Y, J, alpha, beta, gamma


@pytest.mark.parametrize("tag", ["three_terms", "scaled"])
def test_block_gemv_oracle_matches_reference_kernel_text(golden_kernels, tag):
    """oracle.kernels.gemv_block against the reference's own block kernels (tile kernel +
    reduce kernel, rendered and executed on the CPU): several column tiles per term, several
    terms, alpha/beta/gamma other than the simulator's; bit for bit."""
    A, X, Y, J, alpha, beta, gamma = _block_case(golden_kernels, tag)
    K.gemv_block(alpha, A, J, X, J, beta, Y, gamma=gamma)
    assert np.array_equal(Y.buf, golden_kernels["gemv_block/%s/Y1" % tag])


def test_adaptive_lif_oracle_matches_reference_kernel(golden_kernels):
    g = golden_kernels
    V, W, N = g["lif_up1/V0"], g["lif_up1/W0"], g["alif/N0"]
    J, tau = g["lif_up1/J"], g["lif_up1/tau"]
    n = J.size
    for step in range(1, 4):
        V, W, S, N = K.lif(1e-3, J, V, W, tau, np.full(n, 2e-3, np.float32), np.full(n, 1.0, np.float32), N=N,
                           tau_n=np.full(n, 0.1, np.float32), inc_n=np.full(n, 0.05, np.float32))
        # the reference kernel ran with glibc's float expm1 / log1p, the oracle rounds correctly
        assert np.allclose(V, g["alif/V%d" % step], rtol=1e-5, atol=1e-6)
        assert np.allclose(W, g["alif/W%d" % step], rtol=1e-5, atol=1e-6)
        assert np.array_equal(S > 0, g["alif/S%d" % step] > 0)
        assert np.allclose(N, g["alif/N%d" % step], rtol=1e-6, atol=1e-7)
        V, W, N = g["alif/V%d" % step], g["alif/W%d" % step], g["alif/N%d" % step]


def test_timeupdate_and_presentinput_oracle_match_reference_kernels(golden_kernels):
    g = golden_kernels
    RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)
    step, time = RA([np.zeros((1, 1))]), RA([np.zeros((1, 1))])
    for want in g["timeupdate/step_time"]:
        K.timeupdate(step, time, 0.001)
        assert step[0][0, 0] == want[0] and time[0][0, 0] == want[1]
    tabs = RA([np.zeros((7, 3)), np.zeros((4, 1))])
    tabs.buf[...] = g["presentinput/tables"]
    for mode, pres in (("index", None), ("time", np.array([0.003, 0.002], np.float32))):
        Y = RA([np.zeros((3, 1)), np.zeros((1, 1))])
        for i, s_ in enumerate(range(1, 13)):
            t = RA([np.full((1, 1), s_), np.full((1, 1), s_)])
            K.presentinput(Y, t, tabs, 0.001, pres_t=pres)
            assert np.array_equal(Y.buf, g["presentinput/%s" % mode][i]), (mode, s_)


def test_fastlif_oracle_matches_reference_kernel(golden_kernels):
    """The `fastlif` variant of cl_lif (clra_nonlinearities.py:1079-1114), three consecutive steps of
    the reference's kernel text at upsample 1 and 2: refractory times and spikes exactly, voltages to
    one ulp (the reference text calls the float expm1 of the C library it is compiled with)."""
    g = golden_kernels
    J, tau = g["lif_up1/J"], g["lif_up1/tau"]
    for up in (1, 2):
        V, W = g["lif_up1/V0"].copy(), g["lif_up1/W0"].copy()
        for step in range(1, 4):
            V, W, S = K.lif(1e-3, J, V, W, tau, 2e-3, 1.0, upsample=up, fastlif=True)
            key = "fastlif_up%d/" % up
            assert np.array_equal(S, g[key + "S%d" % step])
            assert np.allclose(W, g[key + "W%d" % step], rtol=1e-6, atol=1e-9)
            assert np.allclose(V, g[key + "V%d" % step], rtol=2e-7, atol=1e-7)
            V, W = g[key + "V%d" % step].copy(), g[key + "W%d" % step].copy()  # follow the reference's state
        assert g[key + "S3"].sum() > 0
