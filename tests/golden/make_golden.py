"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference source tree is mounted:

    python tests/golden/make_golden.py /path/to/nengo-ocl

It imports the reference's planning modules under the stand-ins of
``refstubs.py``, calls its own ``plan_*`` functions on seeded inputs and stores

* ``tables.npz``  -- the exact int32 index tables, launch sizes and bw/flops
  figures those planners upload (bit-exact targets for the planning code), and
* ``kernels.npz`` -- inputs and outputs of the reference's own kernel source
  executed on the CPU (``oracle/refkernels.py``) for the neuron models, the
  linear filter and the small elementwise kernels (pins for ``oracle/kernels.py``).

The fixtures are small; the tests read only the ``.npz`` files.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import refstubs  # noqa: E402


def main(reference_root, write_fixtures=True):
    mods = refstubs.install(reference_root)
    from oracle import refkernels  # noqa: E402

    RA = mods["raggedarray"].RaggedArray
    CLRA = mods["clraggedarray"].CLRaggedArray
    gemv = mods["clra_gemv"]
    nl = mods["clra_nonlinearities"]
    queue = refstubs.Queue()
    ra = lambda arrays, dtype=np.float32: RA(arrays, dtype=dtype)
    tables = {}
    kernels = {}

    def capture(fn):
        n0, p0 = len(refstubs.CAPTURE), len(refstubs.PROGRAMS)
        out = fn()
        return out, refstubs.CAPTURE[n0:], refstubs.PROGRAMS[p0:]

    # ---------------- GEMV index plans ----------------
    def gemv_case(tag, A, X, Y, A_js, X_js, alpha, beta, gamma):
        clA, clX, clY = CLRA(queue, A), CLRA(queue, X), CLRA(queue, Y)
        for pname in ("plan_many_dots_gemv", "plan_reduce_gemv", "plan_block_gemv", "plan_ragged_gather_gemv"):
            try:
                prog, cap, _ = capture(lambda: getattr(gemv, pname)(
                    queue, alpha, clA, A_js, clX, X_js, beta, clY, gamma=gamma))
            except Exception as e:  # the dispatcher's ref_impl fallback is broken upstream
                tables["%s/%s/error" % (tag, pname)] = np.array(type(e).__name__)
                continue
            key = "%s/%s" % (tag, pname)
            tables[key + "/n_plans"] = np.array(len(prog.plans))
            for i, plan in enumerate(prog.plans):
                tables["%s/plan%d/gsize" % (key, i)] = np.array(plan.gsize)
                tables["%s/plan%d/lsize" % (key, i)] = np.array(plan.lsize if plan.lsize else ())
                tables["%s/plan%d/bw" % (key, i)] = np.array(plan.bw_per_call or 0)
                tables["%s/plan%d/flops" % (key, i)] = np.array(plan.flops_per_call or 0)
                tables["%s/plan%d/name" % (key, i)] = np.array(plan.name)
            if pname == "plan_block_gemv":
                tables[key + "/gstructure"] = cap[0]
                tables[key + "/Ybuf_size"] = np.array(cap[1].size)
                for j, nm in enumerate(["Yshape0s", "Yinstride0s", "Yinstarts", "Ystride0s", "Ystarts"]):
                    tables[key + "/reduce_" + nm] = cap[2 + j]
                tables[key + "/reduce_inds_starts"] = cap[7]
                tables[key + "/reduce_inds_shape0s"] = cap[8]
                tables[key + "/reduce_inds_buf"] = cap[12]
            elif pname in ("plan_many_dots_gemv", "plan_reduce_gemv"):
                tables[key + "/gstructure"] = cap[0]
            else:
                for j, arr in enumerate(cap):
                    tables["%s/gstructure%d" % (key, j)] = arr

    A = ra([[[0.1, 0.2], [0.3, 0.4]], [[0.5, 0.6]]])
    X = ra([[3, 5]])
    Y = ra([[0.0], [2, 3]])
    gemv_case("basic", A, X, Y, ra([[1], [0]], np.int32), ra([[0], [0]], np.int32), 1.0, 1.0, 0.0)

    rng = np.random.RandomState(1234)
    ND = 20
    A_shapes = [(10, 1 + ii % 2) for ii in range(ND)]
    X_shapes = [(1 + ii % 2, 1) for ii in range(ND)]
    A = ra([0.1 + rng.rand(*s) for s in A_shapes])
    X = ra([0.1 + rng.rand(*s) for s in X_shapes])
    Y = ra([0.1 + rng.rand(10, 1)])
    gemv_case("manydots20", A, X, Y, ra([range(ND)], np.int32), ra([range(ND)], np.int32), 0.5, 0.6, 0.7)

    # scaled-down configuration-2 workload (same generator as the benchmark)
    from nengo_ocl_b200.synth import gemv_workload

    hA, hA_js, hX, hX_js, hY = gemv_workload(seed=1, n_outputs=64)
    toref = lambda r: RA.from_buffer(r.buf.copy(), r.starts, r.shape0s, r.shape1s, r.stride0s, r.stride1s)
    gemv_case("config2_k64", toref(hA), toref(hX), toref(hY), toref(hA_js), toref(hX_js), 0.5, 0.1, 0.0)

    # ---------------- the block GEMV executed from the reference's kernel text ----------------
    # plan_block_gemv (what the reference simulator plans for every MultiDotInc): the tile
    # kernel has barriers that only separate "fill local memory" from "use it" and a two-level
    # tree: with work-items run one after the other, every sweep over a work-group completes one more
    # stage (structure, x, partial sums, tree, output), so five sweeps reproduce it; the reduce
    # kernel has no barrier.
    def block_case(tag, A, X, Y, A_js, X_js, alpha, beta, gamma):
        clA, clX, clY = CLRA(queue, A), CLRA(queue, X), CLRA(queue, Y)
        kernels["gemv_block/%s/A" % tag] = A.buf.copy()
        kernels["gemv_block/%s/X" % tag] = X.buf.copy()
        kernels["gemv_block/%s/Y0" % tag] = Y.buf.copy()
        prog, _, progs = capture(lambda: gemv.plan_block_gemv(queue, alpha, clA, A_js, clX, X_js, beta, clY,
                                                              gamma=gamma))
        texts = [t for t in progs if "__kernel void fn" in t] + [t for t in progs if "__kernel void reduce" in t]
        refkernels.run_plan_grouped(prog.plans[0], texts[0], "fn", passes=5, group_axis=2)
        refkernels.run_plan(prog.plans[1], texts[1], "reduce")
        kernels["gemv_block/%s/Y1" % tag] = clY.cl_buf._arr.copy()
        kernels["gemv_block/%s/scales" % tag] = np.array([alpha, beta, gamma])

    brng = np.random.RandomState(99)
    shapes_b = [(40, 300), (40, 129), (40, 7)]  # three terms: 3, 2 and 1 column tiles
    block_case("three_terms", ra([brng.normal(size=s_) for s_ in shapes_b]),
               ra([brng.normal(size=(s_[1], 1)) for s_ in shapes_b]), ra([brng.normal(size=(40, 1))]),
               ra([[0, 1, 2]], np.int32), ra([[0, 1, 2]], np.int32), 1.0, 1.0, 0.0)
    block_case("scaled", ra([brng.normal(size=(70, 260)), brng.normal(size=(5, 16))]),
               ra([brng.normal(size=(260, 1)), brng.normal(size=(16, 1))]),
               ra([brng.normal(size=(70, 1)), brng.normal(size=(5, 1))]),
               ra([[0], [1]], np.int32), ra([[0], [1]], np.int32), 0.5, 0.6, 0.7)

    # ---------------- elementwise / neuron block tables ----------------
    rng = np.random.RandomState(7)
    sizes = [100, 1000, 37, 2049]
    J = ra([rng.normal(scale=1.2, size=n) for n in sizes])
    V = ra([rng.uniform(0, 1, size=n) for n in sizes])
    W = ra([rng.uniform(-5e-3, 5e-3, size=n) for n in sizes])
    S = ra([np.zeros(n) for n in sizes])
    taus = [0.02, 0.05, 0.015, 0.08]
    T = ra([t * np.ones(n) for t, n in zip(taus, sizes)])
    clJ, clV, clW, clS, clT = (CLRA(queue, r) for r in (J, V, W, S, T))
    for upsample in (1, 4):
        for r, c in ((V, clV), (W, clW), (S, clS)):
            c.cl_buf._arr[...] = r.buf
        plan, cap, progs = capture(lambda: nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0,
                                                       upsample=upsample))
        key = "lif_up%d" % upsample
        tables[key + "/gsize"] = np.array(plan.gsize)
        tables[key + "/bw"] = np.array(plan.bw_per_call)
        tables[key + "/sizes"] = cap[0]
        for j, nm in enumerate(["J", "V", "W", "outV", "outW", "outS", "tau"]):
            tables["%s/%s_starts" % (key, nm)] = cap[1 + j]
        refkernels.run_plan(plan, progs[-1], "cl_lif")
        kernels[key + "/J"] = J.buf.copy()
        kernels[key + "/V0"] = V.buf.copy()
        kernels[key + "/W0"] = W.buf.copy()
        kernels[key + "/tau"] = T.buf.copy()
        kernels[key + "/V1"] = clV.cl_buf._arr.copy()
        kernels[key + "/W1"] = clW.cl_buf._arr.copy()
        kernels[key + "/S1"] = clS.cl_buf._arr.copy()
    kernels["lif/sizes"] = np.array(sizes)

    # adaptive LIF (cl_alif): three consecutive steps with the adaptation state carried
    Na = ra([rng.uniform(0, 0.5, size=n) for n in sizes])
    clNa = CLRA(queue, Na)
    for r, c in ((V, clV), (W, clW), (S, clS)):
        c.cl_buf._arr[...] = r.buf
    plan, cap, progs = capture(lambda: nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0, N=clNa,
                                                   tau_n=0.1, inc_n=0.05))
    kernels["alif/N0"] = Na.buf.copy()
    for step in range(3):
        refkernels.run_plan(plan, progs[-1], "cl_alif")
        for nm, c in (("V", clV), ("W", clW), ("S", clS), ("N", clNa)):
            kernels["alif/%s%d" % (nm, step + 1)] = c.cl_buf._arr.copy()

    # the `fastlif` variant of cl_lif (:1079-1114): three consecutive steps, upsample 1 and 2
    for upsample in (1, 2):
        for r, c in ((V, clV), (W, clW), (S, clS)):
            c.cl_buf._arr[...] = r.buf
        plan, cap, progs = capture(lambda: nl.plan_lif(queue, 1e-3, clJ, clV, clW, clS, 2e-3, clT, 1.0,
                                                       upsample=upsample, fastlif=True))
        for step in range(3):
            refkernels.run_plan(plan, progs[-1], "cl_lif")
            for nm, c in (("V", clV), ("W", clW), ("S", clS)):
                kernels["fastlif_up%d/%s%d" % (upsample, nm, step + 1)] = c.cl_buf._arr.copy()

    # timeupdate: 5 consecutive calls
    st = CLRA(queue, ra([np.zeros((1, 1))]))
    tm = CLRA(queue, ra([np.zeros((1, 1))]))
    plan, cap, progs = capture(lambda: nl.plan_timeupdate(queue, st, tm, 0.001))
    seq = []
    for _ in range(5):
        refkernels.run_plan(plan, progs[-1], "timeupdate")
        seq.append([st.cl_buf._arr[0], tm.cl_buf._arr[0]])
    kernels["timeupdate/step_time"] = np.array(seq, dtype=np.float32)

    # presentinput: table playback by step index and by presentation time
    prng = np.random.RandomState(21)
    tabs = ra([prng.normal(size=(7, 3)), prng.normal(size=(4, 1))])
    Yp = ra([np.zeros((3, 1)), np.zeros((1, 1))])
    tp = ra([np.zeros((1, 1)), np.zeros((1, 1))])
    kernels["presentinput/tables"] = tabs.buf.copy()
    for mode, pres in (("index", None), ("time", refstubs.to_device(queue, np.array([0.003, 0.002], np.float32)))):
        clYp, cltp, cltabs = CLRA(queue, Yp), CLRA(queue, tp), CLRA(queue, tabs)
        plan, cap, progs = capture(lambda: nl.plan_presentinput(queue, clYp, cltp, cltabs, 0.001, pres_t=pres))
        outs = []
        for step in range(1, 13):
            cltp.cl_buf._arr[...] = step
            refkernels.run_plan(plan, progs[-1], "presentinput")
            outs.append(clYp.cl_buf._arr.copy())
        kernels["presentinput/%s" % mode] = np.array(outs)

    # several consecutive LIF steps on one population (state carried)
    n = 4096
    Jm = ra([rng.uniform(-1, 4, size=n)])
    Vm = ra([np.zeros(n)])
    Wm = ra([np.zeros(n)])
    Sm = ra([np.zeros(n)])
    clJm, clVm, clWm, clSm = (CLRA(queue, r) for r in (Jm, Vm, Wm, Sm))
    plan, cap, progs = capture(lambda: nl.plan_lif(queue, 1e-3, clJm, clVm, clWm, clSm, 2e-3, 0.02, 1.0))
    spikes = []
    for _ in range(50):
        refkernels.run_plan(plan, progs[-1], "cl_lif")
        spikes.append(clSm.cl_buf._arr.copy())
    kernels["lif50/J"] = Jm.buf.copy()
    kernels["lif50/V"] = clVm.cl_buf._arr.copy()
    kernels["lif50/W"] = clWm.cl_buf._arr.copy()
    kernels["lif50/spike_counts"] = (np.array(spikes) > 0).sum(axis=0).astype(np.int32)

    # LIF rate / ReLU / spiking ReLU / sigmoid
    R = ra([np.zeros(n) for n in sizes])
    clR = CLRA(queue, R)
    plan, cap, progs = capture(lambda: nl.plan_lif_rate(queue, 1e-3, clJ, clR, 2e-3, clT, 1.0))
    refkernels.run_plan(plan, progs[-1], "cl_lif_rate")
    kernels["lif_rate/R"] = clR.cl_buf._arr.copy()
    amp = CLRA(queue, ra([1.5 * np.ones(n) for n in sizes]))
    plan, cap, progs = capture(lambda: nl.plan_rectified_linear(queue, clJ, clR, amp))
    refkernels.run_plan(plan, progs[-1], "cl_relu")
    kernels["relu/R"] = clR.cl_buf._arr.copy()
    clV.cl_buf._arr[...] = V.buf
    plan, cap, progs = capture(lambda: nl.plan_spiking_rectified_linear(queue, 1e-3, clJ, clV, clR, amp))
    clJ.cl_buf._arr[...] = J.buf * 300
    refkernels.run_plan(plan, progs[-1], "cl_spikingrelu")
    kernels["spikingrelu/J"] = clJ.cl_buf._arr.copy()
    kernels["spikingrelu/V1"] = clV.cl_buf._arr.copy()
    kernels["spikingrelu/S"] = clR.cl_buf._arr.copy()
    clJ.cl_buf._arr[...] = J.buf * 30
    plan, cap, progs = capture(lambda: nl.plan_sigmoid(queue, clJ, clR, 0.0025))
    refkernels.run_plan(plan, progs[-1], "cl_sigmoid")
    kernels["sigmoid/J"] = clJ.cl_buf._arr.copy()
    kernels["sigmoid/R"] = clR.cl_buf._arr.copy()
    clJ.cl_buf._arr[...] = J.buf

    # copy / elementwise_inc / reset / slicedcopy tables + executed outputs
    rng = np.random.RandomState(11)
    shapes = [(3, 5), (1, 1), (700, 1), (40, 13)]
    Xc = ra([rng.normal(size=s) for s in shapes])
    Yc = ra([rng.normal(size=s) for s in shapes])
    clXc, clYc = CLRA(queue, Xc), CLRA(queue, Yc)
    incs = np.array([0, 1, 1, 0], dtype=np.int32)
    plan, cap, progs = capture(lambda: nl.plan_copy(queue, clXc, clYc, incs))
    tables["copy/gsize"] = np.array(plan.gsize)
    for j, nm in enumerate(["offsets", "shape0s", "shape1s", "Xstride0s", "Xstarts", "Ystride0s", "Ystarts",
                            "incs"]):
        tables["copy/" + nm] = cap[j]
    refkernels.run_plan(plan, progs[-1], "copy")
    kernels["copy/X"] = Xc.buf.copy()
    kernels["copy/Y0"] = Yc.buf.copy()
    kernels["copy/Y1"] = clYc.cl_buf._arr.copy()

    Ae = ra([rng.normal(size=s) for s in [(3, 5), (1, 1), (700, 1), (1, 13)]])
    Xe = ra([rng.normal(size=s) for s in [(3, 1), (1, 1), (1, 1), (40, 13)]])
    clAe, clXe = CLRA(queue, Ae), CLRA(queue, Xe)
    clYc.cl_buf._arr[...] = Yc.buf
    plan, cap, progs = capture(lambda: nl.plan_elementwise_inc(queue, clAe, clXe, clYc))
    tables["ewinc/gsize"] = np.array(plan.gsize)
    tables["ewinc/offsets"] = cap[0]
    tables["ewinc/Astarts"] = cap[4]
    tables["ewinc/Ystarts"] = cap[12]
    refkernels.run_plan(plan, progs[-1], "elementwise_inc")
    kernels["ewinc/A"] = Ae.buf.copy()
    kernels["ewinc/X"] = Xe.buf.copy()
    kernels["ewinc/Y1"] = clYc.cl_buf._arr.copy()

    # PES-style outer product with per-item alpha, set (inc=False)
    Eo = ra([rng.normal(size=(d, 1)) for d in (4, 1, 16)])
    Po = ra([rng.normal(size=(n, 1)) for n in (50, 300, 1024)])
    Do = ra([np.zeros((d, n)) for d, n in ((4, 50), (1, 300), (16, 1024))])
    clEo, clPo, clDo = CLRA(queue, Eo), CLRA(queue, Po), CLRA(queue, Do)
    alpha = np.array([-1e-4 * 1e-3 / n for n in (50, 300, 1024)])
    plan, cap, progs = capture(lambda: nl.plan_elementwise_inc(queue, clEo, clPo, clDo, alpha=alpha,
                                                               outer=True, inc=False))
    refkernels.run_plan(plan, progs[-1], "elementwise_inc")
    kernels["outer/E"] = Eo.buf.copy()
    kernels["outer/P"] = Po.buf.copy()
    kernels["outer/alpha"] = alpha
    kernels["outer/D"] = clDo.cl_buf._arr.copy()

    # reset
    Yr = ra([rng.normal(size=s) for s in [(3, 5), (1, 1), (70, 1), (4, 13)]])
    clYr = CLRA(queue, Yr)
    vals = refstubs.to_device(queue, np.array([0.0, 1.5, -2.0, 7.0], dtype=np.float32))
    plan, cap, progs = capture(lambda: nl.plan_reset(queue, clYr, vals))
    tables["reset/gsize"] = np.array(plan.gsize)
    tables["reset/lsize"] = np.array(plan.lsize)
    tables["reset/sizes"] = cap[0]
    tables["reset/starts"] = cap[1]
    tables["reset/values"] = cap[2]
    refkernels.run_plan(plan, progs[-1], "reset")
    kernels["reset/Y1"] = clYr.cl_buf._arr.copy()

    # slicedcopy
    Xs = ra([rng.normal(size=(n, 1)) for n in (10, 50, 33)])
    Ys = ra([rng.normal(size=(n, 1)) for n in (20, 50, 40)])
    xi = [np.arange(10)[::2], np.arange(50)[::-1].copy(), np.arange(33)[5:25]]
    yi = [np.arange(20)[3:8], np.arange(50), np.arange(40)[::2]]
    clXs, clYs = CLRA(queue, Xs), CLRA(queue, Ys)
    clXi, clYi = CLRA(queue, ra(xi, np.int32)), CLRA(queue, ra(yi, np.int32))
    incs3 = np.array([1, 0, 1], dtype=np.int32)
    plan, cap, progs = capture(lambda: nl.plan_slicedcopy(queue, clXs, clYs, clXi, clYi, incs3))
    tables["slicedcopy/gsize"] = np.array(plan.gsize)
    tables["slicedcopy/sizes"] = cap[4]
    tables["slicedcopy/XIstarts"] = cap[5]
    tables["slicedcopy/YIstarts"] = cap[6]
    refkernels.run_plan(plan, progs[-1], "slicedcopy")
    kernels["slicedcopy/X"] = Xs.buf.copy()
    kernels["slicedcopy/Y0"] = Ys.buf.copy()
    kernels["slicedcopy/Y1"] = clYs.cl_buf._arr.copy()

    # linear filters: lowpass (na=1, nb=1), pure gain (na=0), and a 2nd-order IIR
    dens = [[-0.9], [], [-1.6, 0.64]]
    nums = [[0.1], [0.5], [0.02, 0.02]]
    shapes = [(300, 1), (5, 1), (64, 1)]
    Xf = ra([rng.normal(size=s) for s in shapes])
    Yf = ra([np.zeros(s) for s in shapes])
    Af = ra(dens)
    Bf = ra(nums)
    Xb = ra([np.zeros((len(b), s[0])) for b, s in zip(nums, shapes)])
    Yb = ra([np.zeros((len(a), s[0])) for a, s in zip(dens, shapes)])
    cl = [CLRA(queue, r) for r in (Xf, Yf, Af, Bf, Xb, Yb)]
    plans, cap, progs = capture(lambda: nl.plan_linearfilter(queue, *cl))
    tables["linearfilter/gsize"] = np.array(plans[0].gsize)
    tables["linearfilter/lsize"] = np.array(plans[0].lsize)
    tables["linearfilter/offsets"] = cap[2]
    xs_seq, ys_seq = [], []
    for step in range(6):
        xnew = rng.normal(size=Xf.buf.shape).astype(np.float32)
        cl[0].cl_buf._arr[...] = xnew
        refkernels.run_plan_grouped(plans[0], progs[-1], "linearfilter", passes=2, group_axis=1)
        if len(plans) > 1:
            refkernels.run_plan(plans[1], progs[-1], "linearfilter_inc")
        xs_seq.append(xnew.copy())
        ys_seq.append(cl[1].cl_buf._arr.copy())
    kernels["linearfilter/xs"] = np.array(xs_seq)
    kernels["linearfilter/ys"] = np.array(ys_seq)

    # ---------------- learning-rule deltas: bcm, oja, voja kernels ----------------
    lrng = np.random.RandomState(31)
    shapes = [(5, 3), (1, 7), (12, 12)]  # (post, pre)
    pre_h = ra([lrng.normal(size=(n, 1)) for _, n in shapes])
    post_h = ra([lrng.normal(size=(m_, 1)) for m_, _ in shapes])
    theta_h = ra([lrng.normal(size=(m_, 1)) for m_, _ in shapes])
    mat_h = ra([lrng.normal(size=sh) for sh in shapes])
    scale_h = ra([lrng.uniform(0.5, 2, size=(m_, 1)) for m_, _ in shapes])
    learn_h = ra([lrng.normal(size=(1, 1)) for _ in shapes])
    alpha_h = lrng.uniform(-1, 1, size=3).astype(np.float32)
    beta_h = lrng.uniform(0, 2, size=3).astype(np.float32)
    for name, arr in (("pre", pre_h), ("post", post_h), ("theta", theta_h), ("mat", mat_h), ("scale", scale_h),
                      ("learn", learn_h)):
        kernels["learning/%s_buf" % name] = arr.buf.copy()
    kernels["learning/alpha"], kernels["learning/beta"] = alpha_h, beta_h
    kernels["learning/shapes"] = np.array(shapes)
    dev = lambda a: CLRA(queue, a)
    dalpha, dbeta = refstubs.to_device(queue, alpha_h), refstubs.to_device(queue, beta_h)
    delta = dev(ra([np.zeros(sh) for sh in shapes]))
    plan, _, progs = capture(lambda: nl.plan_bcm(queue, dev(pre_h), dev(post_h), dev(theta_h), delta, dalpha))
    refkernels.run_plan(plan, progs[-1], "bcm")
    kernels["learning/bcm_delta"] = delta.cl_buf._arr.copy()
    tables["learning/bcm_gsize"] = np.array(plan.gsize)
    delta = dev(ra([np.zeros(sh) for sh in shapes]))
    plan, _, progs = capture(lambda: nl.plan_oja(queue, dev(pre_h), dev(post_h), dev(mat_h), delta, dalpha, dbeta))
    refkernels.run_plan(plan, progs[-1], "oja")
    kernels["learning/oja_delta"] = delta.cl_buf._arr.copy()
    delta = dev(ra([np.zeros(sh) for sh in shapes]))
    plan, _, progs = capture(lambda: nl.plan_voja(queue, dev(pre_h), dev(post_h), dev(mat_h), delta, dev(learn_h),
                                                  dev(scale_h), dalpha))
    refkernels.run_plan(plan, progs[-1], "voja")
    kernels["learning/voja_delta"] = delta.cl_buf._arr.copy()

    # ---------------- sparse transforms: host tables, heuristic, CSR kernel ----------------
    import scipy.sparse as sp

    HSM = mods["utils"].HostSparseMatrix
    srng = np.random.RandomState(77)
    sparse_cases = {
        "small": sp.random(7, 5, density=0.4, random_state=srng, format="csr", dtype=np.float32),
        "empty_rows": sp.csr_matrix(np.array([[0, 0, 0], [1.5, 0, -2.0], [0, 0, 0], [0, 3.0, 0]], dtype=np.float32)),
        "all_zero": sp.csr_matrix((4, 6), dtype=np.float32),
        "wide_row": sp.vstack([sp.random(1, 300, density=0.9, random_state=srng, dtype=np.float32),
                               sp.random(40, 300, density=0.02, random_state=srng, dtype=np.float32)]).tocsr(),
        "banded": sp.diags([srng.normal(size=199), srng.normal(size=200), srng.normal(size=199)], [-1, 0, 1],
                           format="csr", dtype=np.float32),
    }
    for tag, mat in sparse_cases.items():
        hA = HSM(mat)
        key = "sparse/" + tag
        tables[key + "/dense"] = np.asarray(mat.todense(), dtype=np.float32)
        ell = gemv.plan_ellpack.scipy2elldata(hA)
        for name in ("columns", "entries", "rowlens"):
            tables["%s/ell_%s" % (key, name)] = np.asarray(getattr(ell, name))
        tables[key + "/ell_width_nnz"] = np.array([ell.ellwidth, ell.nnz])
        csr = gemv.plan_csr.scipy2csrdata(hA)
        for name in ("indices", "indptr", "data"):
            tables["%s/csr_%s" % (key, name)] = np.asarray(getattr(csr, name))
        tables[key + "/heuristic"] = np.array(gemv.spmv_algorithm_heuristic(queue, hA))
        # the reference's CSR kernel, set and increment mode
        x = srng.normal(size=(mat.shape[1], 1)).astype(np.float32)
        y0 = srng.normal(size=(mat.shape[0], 1)).astype(np.float32)
        kernels[key + "/x"], kernels[key + "/y0"] = x, y0
        for inc in (False, True):
            clX, clY = CLRA(queue, ra([x])), CLRA(queue, ra([y0]))
            plan, _, progs = capture(lambda: gemv.spmv_csr_impl(
                queue, refstubs.to_device(queue, csr.indices if csr.indices.size else np.zeros(1, np.int32)),
                refstubs.to_device(queue, csr.indptr),
                refstubs.to_device(queue, csr.data if csr.data.size else np.zeros(1, np.float32)), clX, clY, inc=inc))
            refkernels.run_plan(plan, progs[-1], "sparsedot_inc")
            kernels["%s/y_%s" % (key, "inc" if inc else "set")] = clY.cl_buf._arr.copy()
    # footprint heuristic on a device with little memory (the three branches)
    class SmallDevice:
        global_mem_size = 0

    class SmallQueue:
        device = SmallDevice()

    big = HSM(sparse_cases["wide_row"])
    for mem, tag in ((10 ** 3, "hard"), (3 * 10 ** 4, "mid"), (10 ** 9, "soft")):
        SmallDevice.global_mem_size = mem
        tables["sparse/heuristic_%s" % tag] = np.array(gemv.spmv_algorithm_heuristic(SmallQueue(), big))

    if write_fixtures:
        np.savez_compressed(os.path.join(HERE, "tables.npz"), **tables)
        np.savez_compressed(os.path.join(HERE, "kernels.npz"), **kernels)
        print("wrote %d table entries, %d kernel entries" % (len(tables), len(kernels)))
    return tables, kernels


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/nengo-ocl")
    main(sys.argv[1])
