"""Ragged gather-GEMV on the GPU through the C ABI, checked against the CPU
oracle.  Cases follow the reference's nengo_ocl/tests/test_clra_gemv.py:60-289
(same seeds, shapes, alpha/beta/gamma); tolerances: the reference's own
atol=rtol=1e-3 against numpy, and a tighter float32 bound against the exact
value: |y - exact| <= 1e-5 * sum|terms| + 1e-7."""

import numpy as np
import pytest

from nengo_ocl_b200 import _capi, cura_gemv
from nengo_ocl_b200.curaggedarray import CUDARaggedArray as CLRA
from nengo_ocl_b200.raggedarray import RaggedArray
from nengo_ocl_b200.synth import gemv_workload
from oracle import kernels as K

pytestmark = pytest.mark.gpu

RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)
PLANNERS = [cura_gemv.plan_reduce_gemv, cura_gemv.plan_many_dots_gemv, cura_gemv.plan_block_gemv,
            cura_gemv.plan_ragged_gather_gemv, cura_gemv.plan_ref_gemv, cura_gemv.plan_fused_gemv]
KINDS = [_capi.GEMV_CTA, _capi.GEMV_CTA_BULK, _capi.GEMV_PIPE, 4]


def clone(r):
    return RaggedArray.from_buffer(r.buf.copy(), r.starts, r.shape0s, r.shape1s, r.stride0s, r.stride1s)


def run(queue, planner, alpha, A, A_js, X, X_js, beta, Y, gamma=0.0, kind=None):
    clA, clX, clY = CLRA(queue, A), CLRA(queue, X), CLRA(queue, Y)
    prog = planner(queue, alpha, clA, A_js, clX, X_js, beta, clY, gamma=gamma, cta_kind=kind)
    for plan in prog.plans:
        plan()
        if getattr(plan, "status", None) is not None:  # (kernels with bounded waits report them here)
            assert int(plan.status.get()[0]) == 0
    return clY, prog


def check_exact(alpha, A, A_js, X, X_js, beta, Y0, clY, gamma=0.0):
    vals, mags = K.gemv_exact(alpha, A, A_js, X, X_js, beta, Y0, gamma=gamma)
    for i in range(len(Y0)):
        got = clY[i][:, 0]
        assert np.all(np.abs(got - vals[i]) <= 1e-5 * mags[i] + 1e-7), i


@pytest.mark.parametrize("planner", PLANNERS)
@pytest.mark.parametrize("kind", KINDS)
def test_basic(queue, planner, kind):
    A = RA([[[0.1, 0.2], [0.3, 0.4]], [[0.5, 0.6]]])
    X = RA([[3, 5]])
    Y = RA([[0.0], [2, 3]])
    A_js = RA([[1], [0]], dtype=np.int32)
    X_js = RA([[0], [0]], dtype=np.int32)
    clY, _ = run(queue, planner, 1.0, A, A_js, X, X_js, 1.0, Y, kind=kind)
    assert np.allclose(clY[0].ravel(), [4.5])
    assert np.allclose(clY[1].ravel(), [3.3, 5.9])


def check_from_shapes(queue, planner, alpha, beta, gamma, A_shapes, X_shapes, A_js, X_js, kind=None):
    rng = np.random.RandomState(1234)
    A = RA([0.1 + rng.rand(*shp) for shp in A_shapes])
    X = RA([0.1 + rng.rand(*shp) for shp in X_shapes])
    Y = RA([0.1 + rng.rand(A_shapes[A_js[ii][0]][0], X_shapes[X_js[ii][0]][1]) for ii in range(len(A_js))])
    A_js = RA(A_js, dtype=np.int32)
    X_js = RA(X_js, dtype=np.int32)
    clY, _ = run(queue, planner, alpha, A, A_js, X, X_js, beta, Y, gamma=gamma, kind=kind)
    for i in range(len(A_js)):
        ref = gamma + beta * Y[i] + alpha * sum(
            np.dot(A[aj], X[xj]) for aj, xj in zip(A_js[i].ravel(), X_js[i].ravel()))
        assert np.allclose(ref, clY[i], atol=1e-3, rtol=1e-3)
    check_exact(alpha, A, A_js, X, X_js, beta, Y, clY, gamma=gamma)


@pytest.mark.parametrize("planner", PLANNERS)
def test_shape_family(queue, planner):
    args = (queue, planner, 0.5, 0.6, 0.7)
    check_from_shapes(*args, A_shapes=[(1, 1)], X_shapes=[(1, 1)], A_js=[[0]], X_js=[[0]])
    check_from_shapes(*args, A_shapes=[(10, 1)], X_shapes=[(1, 1)], A_js=[[0]], X_js=[[0]])
    check_from_shapes(*args, A_shapes=[(2001, 1)], X_shapes=[(1, 1)], A_js=[[0]], X_js=[[0]])
    for ND in (2, 20, 100):
        check_from_shapes(*args, A_shapes=[(10, 1 + ii % 2) for ii in range(ND)],
                          X_shapes=[(1 + ii % 2, 1) for ii in range(ND)], A_js=[range(ND)], X_js=[range(ND)])
    for ND in (2, 20, 100):
        check_from_shapes(*args, A_shapes=[(2000, ii + 1) for ii in range(ND)],
                          X_shapes=[(ii + 1, 1) for ii in range(ND)], A_js=[range(ND)], X_js=[range(ND)])


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("k,p,m,n", [(4, 1, 10, 10), (10, 1, 550, 550), (4, 4, 10, 10), (4, 4, 2000, 1000)])
def test_random(queue, kind, k, p, m, n):
    """reference _test_random (RandomState(3294), alpha=.5, beta=.1)"""
    rng = np.random.RandomState(3294)
    A = RA([rng.normal(size=(m, n)) for i in range(k)])
    X = RA([rng.normal(size=n) for i in range(k)])
    Y = RA([rng.normal(size=m) for i in range(k)])
    A_js = RA([rng.randint(k, size=p) for i in range(k)], dtype=np.int32)
    X_js = RA([rng.randint(k, size=p) for i in range(k)], dtype=np.int32)
    clY, _ = run(queue, cura_gemv.plan_ragged_gather_gemv, 0.5, A, A_js, X, X_js, 0.1, Y, kind=kind)
    for i in range(k):
        ref = 0.1 * Y[i]
        for aj, xj in zip(A_js[i].ravel(), X_js[i].ravel()):
            ref = ref + 0.5 * np.dot(A[aj], X[xj])
        assert np.allclose(ref, clY[i], atol=1e-3, rtol=1e-3)
    check_exact(0.5, A, A_js, X, X_js, 0.1, Y, clY)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("align", [False, True])
def test_config2_scaled_matches_oracle(queue, kind, align):
    """Benchmark configuration 2 generator at 256 outputs against the oracle's
    serial float32 restatement and the exact value."""
    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=256, align=align)
    Yo = clone(Y)
    K.gemv_ref(0.5, A, A_js, X, X_js, 0.1, Yo)
    clY, prog = run(queue, cura_gemv.plan_fused_gemv, 0.5, A, A_js, X, X_js, 0.1, Y, kind=kind)
    got = clY.to_host()
    # two float32 summation orders of the same terms
    assert np.allclose(got.buf, Yo.buf, rtol=1e-4, atol=1e-4)
    check_exact(0.5, A, A_js, X, X_js, 0.1, Y, clY)
    cta, warp = prog.plans[0].worklist
    if kind == cura_gemv.GEMV_PIPE:  # one launch: tiny items are records of the pipelined kernel too
        assert len(prog.plans[0].records) > 0 and len(cta) == 0 and len(warp) == 0
    else:
        assert len(cta) > 0 and len(warp) > 0  # both kernels ran


def test_per_item_scales_strided_x_and_inplace(queue, rng):
    A = RA([rng.normal(size=(7, 5)), rng.normal(size=(3, 5)), rng.normal(size=(7, 2))])
    Xbig = RA([rng.normal(size=(10, 1)), rng.normal(size=(2, 1))])
    # a strided view of X[0]: every second element
    Xbig.add_views([Xbig.starts[0]], [5], [1], [2], [1])
    Y = RA([rng.normal(size=7), rng.normal(size=3)])
    A_js = RA([[0, 2], [1]], dtype=np.int32)
    X_js = RA([[2, 1], [2]], dtype=np.int32)
    alpha, beta, gamma = [0.5, -1.5], [0.25, 2.0], [1.0, -3.0]
    clY, _ = run(queue, cura_gemv.plan_ref_gemv, alpha, A, A_js, Xbig, X_js, beta, Y, gamma=gamma)
    for i in range(2):
        ref = gamma[i] + beta[i] * Y[i]
        for aj, xj in zip(A_js[i].ravel(), X_js[i].ravel()):
            ref = ref + alpha[i] * np.dot(A[aj], Xbig[xj])
        assert np.allclose(ref, clY[i], rtol=1e-5, atol=1e-5)
    # specialised variants refuse per-item alpha/gamma, as the reference does
    with pytest.raises(NotImplementedError):
        run(queue, cura_gemv.plan_block_gemv, alpha, A, A_js, Xbig, X_js, beta, Y, gamma=gamma)


def test_idempotent_replay_and_linearity(queue):
    """Size-independent properties on the full configuration-2 workload:
    beta=0 makes the call idempotent, and the result is linear in alpha."""
    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=4096)
    clA, clX = CLRA(queue, A), CLRA(queue, X)
    clY1, clY2 = CLRA(queue, Y), CLRA(queue, Y)
    p1 = cura_gemv.plan_fused_gemv(queue, 1.0, clA, A_js, clX, X_js, 0.0, clY1)
    p2 = cura_gemv.plan_fused_gemv(queue, 2.0, clA, A_js, clX, X_js, 0.0, clY2)
    p1.plans[0]()
    first = clY1.cl_buf.get()
    p1.plans[0]()
    assert np.array_equal(first, clY1.cl_buf.get())
    p2.plans[0]()
    assert np.array_equal(2 * first, clY2.cl_buf.get())  # scaling by 2 is exact in float32
    assert p1.plans[0].bw_per_call == cura_gemv.bw_from_geometry(p1.geometry, range(len(Y)))
    # spot-check 32 outputs against the exact value
    idx = list(range(0, 4096, 128))
    vals, mags = K.gemv_exact(1.0, A, A_js[idx], X, X_js[idx], 0.0, Y[idx])
    for j, i in enumerate(idx):
        assert np.all(np.abs(clY1[i][:, 0] - vals[j]) <= 1e-5 * mags[j] + 1e-7)


def test_config2_full_size_properties(queue):
    """Benchmark configuration 2 at its full size (4096 outputs, 688 MB of matrices), checked by
    properties that do not need the oracle on every element: the pipelined kernel agrees with the
    independent row-group kernel on every output, with the float64 value on a sample of items, and
    is linear in alpha (Y(2a) - Y(0) = 2 (Y(a) - Y(0)))."""
    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=4096)
    clA, clX = CLRA(queue, A), CLRA(queue, X)

    def product(alpha, kind):
        clY = CLRA(queue, Y)
        prog = cura_gemv.plan_fused_gemv(queue, alpha, clA, A_js, clX, X_js, 0.1, clY, cta_kind=kind)
        for plan in prog.plans:
            plan()
            assert int(plan.status.get()[0]) == 0
        return clY.cl_buf.get()

    y_pipe = product(0.5, cura_gemv.GEMV_PIPE)
    y_rows = product(0.5, cura_gemv.GEMV_ROWS)
    scale = np.abs(y_pipe).max()
    assert np.allclose(y_pipe, y_rows, rtol=1e-4, atol=1e-5 * scale)
    # float64 value of 64 sampled items
    rng = np.random.RandomState(0)
    for i in rng.choice(len(Y), size=64, replace=False):
        exact = 0.1 * Y[i].astype(np.float64)
        mag = np.abs(exact)
        for a_j, x_j in zip(A_js[i].ravel(), X_js[i].ravel()):
            a, x = A[int(a_j)].astype(np.float64), X[int(x_j)].astype(np.float64)
            exact = exact + 0.5 * (a @ x)
            mag = mag + 0.5 * (np.abs(a) @ np.abs(x))
        lo = int(Y.starts[i])
        got = y_pipe[lo:lo + exact.size]
        assert np.all(np.abs(got - exact.ravel()) <= 1e-5 * mag.ravel() + 1e-7), i
    y0 = product(0.0, cura_gemv.GEMV_PIPE)
    y2 = product(1.0, cura_gemv.GEMV_PIPE)
    assert np.allclose(y2 - y0, 2 * (y_pipe - y0), rtol=1e-4, atol=1e-5 * scale)


def check_block_exact(queue, alpha, A, A_js, X, X_js, beta, Y, gamma=0.0):
    """plan_block_gemv against the oracle's restatement of the reference's block kernels
    (clra_gemv.py:1018-1058,1137-1153): every output bit for bit."""
    ref = clone(Y)
    K.gemv_block(alpha, A, A_js, X, X_js, beta, ref, gamma=gamma)
    clY, prog = run(queue, cura_gemv.plan_block_gemv, alpha, A, A_js, X, X_js, beta, Y, gamma=gamma)
    for i in range(len(Y)):
        assert np.array_equal(clY[i], ref[i]), i
    return prog


def test_block_gemv_is_bit_exact(queue):
    """The planner the simulator uses for every MultiDotInc reproduces the float32 summation
    order of the reference's block kernels: 128-column tiles, four column-strided partial sums
    per tile, (s0 + s2) + (s1 + s3), tiles added in order to beta * y_in, gamma last."""
    # the reference's known-answer case
    A = RA([[[0.1, 0.2], [0.3, 0.4]], [[0.5, 0.6]]])
    X = RA([[3, 5]])
    Y = RA([[0.0], [2, 3]])
    check_block_exact(queue, 1.0, A, RA([[1], [0]], dtype=np.int32), X, RA([[0], [0]], dtype=np.int32), 1.0, Y)
    # shape family of the reference tests, alpha = .5, beta = .6, gamma = .7
    rng = np.random.RandomState(1234)
    for A_shapes in ([(1, 1)], [(10, 1)], [(2001, 1)], [(10, 1 + ii % 2) for ii in range(20)],
                     [(2000, ii + 1) for ii in range(100)], [(33, 129), (33, 517), (33, 128)],
                     [(5, 1030)], [(300, 260)]):
        A = RA([0.1 + rng.rand(*shp) for shp in A_shapes])
        X = RA([0.1 + rng.rand(shp[1], 1) for shp in A_shapes])
        Y = RA([0.1 + rng.rand(A_shapes[0][0], 1)])
        js = RA([range(len(A_shapes))], dtype=np.int32)
        check_block_exact(queue, 0.5, A, js, X, js, 0.6, Y, gamma=0.7)
        check_block_exact(queue, 1.0, A, js, X, js, 1.0, Y)  # the simulator's scales
        check_block_exact(queue, 1.0, A, js, X, js, 0.0, Y)  # a folded reset
    # the reference's random test and the scaled benchmark configuration 2
    rng = np.random.RandomState(3294)
    k, p_, m_, n_ = 4, 4, 2000, 1000
    A = RA([rng.normal(size=(m_, n_)) for i in range(k)])
    X = RA([rng.normal(size=n_) for i in range(k)])
    Y = RA([rng.normal(size=m_) for i in range(k)])
    A_js = RA([rng.randint(k, size=p_) for i in range(k)], dtype=np.int32)
    X_js = RA([rng.randint(k, size=p_) for i in range(k)], dtype=np.int32)
    check_block_exact(queue, 0.5, A, A_js, X, X_js, 0.1, Y)
    for align in (False, True):
        A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=256, align=align)
        prog = check_block_exact(queue, 0.5, A, A_js, X, X_js, 0.1, Y)
        cta, warp = prog.plans[0].worklist
        assert len(cta) and len(warp)  # both kernels ran


@pytest.mark.parametrize("tag", ["three_terms", "scaled"])
def test_block_gemv_matches_reference_kernel_text(queue, golden_kernels, tag):
    """plan_block_gemv on the GPU against outputs of the reference's own block kernels (tile +
    reduce, rendered and executed on the CPU; tests/golden/make_golden.py): bit for bit."""
    import sys, os

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_oracle_golden import _block_case

    A, X, Y, J, alpha, beta, gamma = _block_case(golden_kernels, tag)
    clY, _ = run(queue, cura_gemv.plan_block_gemv, alpha, A, J, X, J, beta, Y, gamma=gamma)
    assert np.array_equal(clY.cl_buf.get()[:Y.buf.size], golden_kernels["gemv_block/%s/Y1" % tag])
