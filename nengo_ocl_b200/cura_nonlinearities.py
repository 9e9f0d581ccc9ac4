"""Plans for everything other than GEMV: clock, reset, copies, elementwise
increment (PES), linear filters, probes, node functions, table playback and
the neuron models.

Function-for-function the planning surface of the reference's
``nengo_ocl/clra_nonlinearities.py`` (same names, arguments, asserts and plan
attributes such as ``bw_per_call``, ``description``, ``cl_bufpositions``,
``Y``).  Each function builds the int32 block tables the reference would
upload -- kept on the plan as ``plan.tables`` so they can be compared bit for
bit -- and hands them to the matching CUDA entry point.
"""

import ctypes

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.curaggedarray import CUDARaggedArray, to_device
from nengo_ocl_b200.plan import Plan
from nengo_ocl_b200.utils import is_number, nonelist, round_up


def get_mwgs(queue, cap=256):
    return min(queue.device.max_work_group_size, cap)


# ---- blockify helpers (clra_nonlinearities.py:22-110) ------------------------
def blockify_ij(max_size, ra):
    """Split each item's flat extent into chunks: (sizes, item index, offset)."""
    sizes, inds, offsets = [], [], []
    for k, size in enumerate(ra.sizes):
        size = int(size)
        for offset in range(0, size, max_size):
            inds.append(k)
            sizes.append(min(size - offset, max_size))
            offsets.append(offset)
    as32 = lambda v: np.array(v, dtype=np.int32)
    return as32(sizes), as32(inds), as32(offsets)


def _blockify(max_size, ras, lengths, step_fn):
    ras = list(ras)
    sizes, inds = [], []
    starts = [[] for _ in ras]
    for i, length in enumerate(lengths):
        length = int(length)
        cursors = [int(ra.starts[i]) for ra in ras]
        while length > 0:
            sizes.append(min(length, max_size))
            inds.append(i)
            length -= max_size
            for k, ra in enumerate(ras):
                starts[k].append(cursors[k])
                cursors[k] += step_fn(ra, i)
    return (np.array(sizes, dtype=np.int32), np.array(inds, dtype=np.int32),
            np.array(starts, dtype=np.int32).reshape(len(ras), len(sizes)))


def blockify_matrices(max_size, ras):
    """Chunk contiguous matrices of identical shapes; starts advance by max_size."""
    ras = list(ras)
    ra0 = ras[0]
    for ra in ras:
        assert len(ra) == len(ra0)
        assert (ra.shape1s == ra0.shape1s).all()
        assert (ra.shape0s == ra0.shape0s).all()
        assert (ra.shape1s == ra.stride0s).all(), "not contiguous"
    return _blockify(max_size, ras, ra0.sizes, lambda ra, i: max_size)


def blockify_matrix(max_size, ra):
    sizes, inds, starts = blockify_matrices(max_size, [ra])
    return sizes, inds, starts[0]


def blockify_vectors(max_size, ras):
    """Chunk vectors of identical lengths; starts advance by max_size * stride0."""
    ras = list(ras)
    if not ras:
        return np.zeros(0, np.int32), np.zeros(0, np.int32), np.zeros((0, 0), np.int32)
    ra0 = ras[0]
    for ra in ras:
        assert len(ra) == len(ra0)
        assert (ra.shape1s == 1).all()
        assert (ra.shape0s == ra0.shape0s).all()
    return _blockify(max_size, ras, ra0.shape0s, lambda ra, i: max_size * int(ra.stride0s[i]))


def blockify_vector(max_size, ra):
    sizes, inds, starts = blockify_vectors(max_size, [ra])
    return sizes, inds, starts[0]


def _describe(ra):
    s = ra.sizes
    return "groups: %d; items: %d; items/group: %0.1f [%d, %d]" % (len(ra), s.sum(), s.mean(), s.min(), s.max())


def _ptr(arr):
    return None if arr is None else arr.ptr


def _inc_mode(queue, incs, inds):
    """0 = all set, 1 = all inc, 2 = per-block flags (uploaded)."""
    incs = np.asarray(incs)
    if (incs == 0).all():
        return 0, None
    if (incs == 1).all():
        return 1, None
    return 2, to_device(queue, incs[inds].astype(np.int32))


# ---- plans -------------------------------------------------------------------
def plan_timeupdate(queue, step, time, dt):
    assert len(step) == len(time) == 1
    assert step.ctype == time.ctype == "float"
    assert step.shape0s[0] == step.shape1s[0] == 1
    assert time.shape0s[0] == time.shape1s[0] == 1
    step_ptr = ctypes.c_void_p(step.cl_buf.data + 4 * int(step.starts[0]))
    time_ptr = ctypes.c_void_p(time.cl_buf.data + 4 * int(time.starts[0]))
    fn, check, dt = _capi.lib().nb2_timeupdate, _capi.check, float(dt)

    def launch(stream):
        check(fn(stream, step_ptr, time_ptr, dt))

    plan = Plan(queue, launch, (1,), lsize=None, name="cl_timeupdate")
    plan.phase = _capi.phase("timeupdate", step_ptr, time_ptr, dt)
    plan.full_args = (step.cl_buf, time.cl_buf)
    return plan


def plan_reset(queue, Y, values, tag=None):
    assert len(Y) == len(values)
    assert (Y.stride0s == Y.shape1s).all()
    assert (Y.stride1s == 1).all()
    assert Y.ctype == values.ctype

    lsize0 = 16
    lsize1 = get_mwgs(queue, cap=256) // lsize0
    Ysizes, Yinds, Ystarts = blockify_matrix(lsize0, Y)
    host_values = values.get()
    clvalues = to_device(queue, host_values[Yinds])
    clYsizes = to_device(queue, Ysizes)
    clYstarts = to_device(queue, Ystarts)
    N = len(Ysizes)
    fn, check = _capi.lib().nb2_reset, _capi.check
    args = (N, clvalues.ptr, clYsizes.ptr, clYstarts.ptr, Y.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (lsize0, max(round_up(N, lsize1), lsize1)), lsize=(lsize0, lsize1),
                name="cl_reset", tag=tag)
    plan.full_args = (clvalues, clYsizes, clYstarts, Y.cl_buf)
    plan.tables = dict(sizes=Ysizes, inds=Yinds, starts=Ystarts)
    plan.bw_per_call = Y.nbytes + host_values.nbytes + clYsizes.nbytes + clYstarts.nbytes
    plan.description = _describe(Y)
    return plan


def plan_copy(queue, X, Y, incs, tag=None):
    assert len(X) == len(Y)
    assert (X.shape0s == Y.shape0s).all()
    assert (X.shape1s == Y.shape1s).all()
    assert (X.stride1s == 1).all()
    assert (Y.stride1s == 1).all()
    assert X.ctype == Y.ctype

    lsize0 = get_mwgs(queue, cap=256)
    sizes, inds, offsets = blockify_ij(lsize0, Y)
    tables = dict(offsets=offsets, shape0s=X.shape0s[inds], shape1s=X.shape1s[inds],
                  Xstride0s=X.stride0s[inds], Xstarts=X.starts[inds],
                  Ystride0s=Y.stride0s[inds], Ystarts=Y.starts[inds])
    dev = {k: to_device(queue, v) for k, v in tables.items()}
    inc_mode, incdata = _inc_mode(queue, incs, inds)
    n_blocks = len(sizes)
    fn, check = _capi.lib().nb2_copy, _capi.check
    args = (n_blocks, inc_mode, _ptr(incdata), dev["offsets"].ptr, dev["shape0s"].ptr, dev["shape1s"].ptr,
            dev["Xstride0s"].ptr, dev["Xstarts"].ptr, X.cl_buf.ptr, dev["Ystride0s"].ptr,
            dev["Ystarts"].ptr, Y.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (lsize0, max(n_blocks, 1)), lsize=None, name="cl_copy", tag=tag)
    plan.full_args = (dev, incdata, X.cl_buf, Y.cl_buf)
    plan.tables = dict(tables, sizes=sizes, inds=inds)
    plan.bw_per_call = X.nbytes + Y.nbytes
    plan.description = _describe(X)
    return plan


def plan_slicedcopy(queue, X, Y, Xinds, Yinds, incs, tag=None):
    assert len(X) == len(Y) == len(Xinds) == len(Yinds)
    for arr in [X, Y, Xinds, Yinds]:
        assert (arr.shape1s == 1).all()
        assert (arr.stride1s == 1).all()
    for arr in [Xinds, Yinds]:
        assert (arr.stride0s == 1).all()
    assert (Xinds.shape0s == Yinds.shape0s).all()
    assert X.ctype == Y.ctype
    assert Xinds.ctype == Yinds.ctype == "int"

    lsize0 = 16
    lsize1 = get_mwgs(queue) // lsize0
    sizes, inds, (XIstarts, YIstarts) = blockify_vectors(lsize0, [Xinds, Yinds])
    N = len(sizes)
    tables = dict(Xstride0s=X.stride0s[inds], Xstarts=X.starts[inds], Ystride0s=Y.stride0s[inds],
                  Ystarts=Y.starts[inds], sizes=sizes, XIstarts=XIstarts, YIstarts=YIstarts)
    dev = {k: to_device(queue, v) for k, v in tables.items()}
    inc_mode, incdata = _inc_mode(queue, incs, inds)
    fn, check = _capi.lib().nb2_slicedcopy, _capi.check
    args = (N, inc_mode, _ptr(incdata), dev["Xstride0s"].ptr, dev["Xstarts"].ptr, X.cl_buf.ptr,
            dev["Ystride0s"].ptr, dev["Ystarts"].ptr, Y.cl_buf.ptr, dev["sizes"].ptr, dev["XIstarts"].ptr,
            Xinds.cl_buf.ptr, dev["YIstarts"].ptr, Yinds.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (lsize0, max(round_up(N, lsize1), lsize1)), lsize=(lsize0, lsize1),
                name="cl_slicedcopy", tag=tag)
    plan.full_args = (dev, incdata, X.cl_buf, Y.cl_buf, Xinds.cl_buf, Yinds.cl_buf)
    plan.tables = dict(tables, inds=inds)
    plan.bw_per_call = 2 * (Xinds.nbytes + int(Xinds.sizes.sum()) * X.dtype.itemsize)
    plan.description = _describe(Xinds)
    return plan


def plan_elementwise_inc(queue, A, X, Y, alpha=None, outer=False, inc=True, tag=None):
    """``Y (+)= alpha * A * X`` with broadcasting; ``outer=True`` is
    ``alpha * a_i * x_j`` for vectors A, X (the PES weight delta)."""
    assert len(Y) == len(X) == len(A)
    for arr in [A, X, Y]:
        assert (arr.stride1s == 1).all()
    if outer:
        assert (A.shape1s == 1).all()
        assert (X.shape1s == 1).all()
        assert ((A.shape0s == 1) | (A.shape0s == Y.shape0s)).all()
        assert ((X.shape0s == 1) | (X.shape0s == Y.shape1s)).all()
    else:
        assert ((X.shape0s == 1) | (X.shape0s == Y.shape0s)).all()
        assert ((X.shape1s == 1) | (X.shape1s == Y.shape1s)).all()
        assert ((A.shape0s == 1) | (A.shape0s == Y.shape0s)).all()
        assert ((A.shape1s == 1) | (A.shape1s == Y.shape1s)).all()
    assert X.ctype == Y.ctype
    assert A.ctype == Y.ctype
    if alpha is not None:
        assert isinstance(alpha, np.ndarray)
        assert alpha.shape == (len(Y),)

    lsize0 = get_mwgs(queue, cap=256)
    sizes, inds, offsets = blockify_ij(lsize0, Y)
    cl_alpha = None if alpha is None else to_device(queue, alpha[inds].astype(Y.dtype))
    tables = dict(offsets=offsets,
                  Ashape0s=A.shape0s[inds], Ashape1s=A.shape1s[inds], Astride0s=A.stride0s[inds],
                  Astarts=A.starts[inds],
                  Xshape0s=X.shape0s[inds], Xshape1s=X.shape1s[inds], Xstride0s=X.stride0s[inds],
                  Xstarts=X.starts[inds],
                  Yshape0s=Y.shape0s[inds], Yshape1s=Y.shape1s[inds], Ystride0s=Y.stride0s[inds],
                  Ystarts=Y.starts[inds])
    dev = {k: to_device(queue, v) for k, v in tables.items()}
    n_blocks = len(sizes)
    fn, check = _capi.lib().nb2_elementwise_inc, _capi.check
    args = (n_blocks, int(bool(outer)), int(bool(inc)), _ptr(cl_alpha), dev["offsets"].ptr,
            dev["Ashape0s"].ptr, dev["Ashape1s"].ptr, dev["Astride0s"].ptr, dev["Astarts"].ptr, A.cl_buf.ptr,
            dev["Xshape0s"].ptr, dev["Xshape1s"].ptr, dev["Xstride0s"].ptr, dev["Xstarts"].ptr, X.cl_buf.ptr,
            dev["Yshape0s"].ptr, dev["Yshape1s"].ptr, dev["Ystride0s"].ptr, dev["Ystarts"].ptr, Y.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (lsize0, max(n_blocks, 1)), lsize=None, name="cl_elementwise_inc", tag=tag)
    plan.full_args = (dev, cl_alpha, A.cl_buf, X.cl_buf, Y.cl_buf)
    plan.tables = dict(tables, sizes=sizes, inds=inds)
    plan.flops_per_call = 2 * int(Y.sizes.sum())
    plan.bw_per_call = A.nbytes + X.nbytes + Y.nbytes + (0 if cl_alpha is None else cl_alpha.nbytes)
    plan.description = _describe(Y)
    return plan


def plan_linearfilter(queue, X, Y, A, B, Xbuf, Ybuf, tag=None):
    """``y[n+1] + a[0] y[n] + ... + a[i] y[n-i] = b[0] x[n] + ... + b[j] x[n-j]``"""
    assert len(X) == len(Y) == len(A) == len(B) == len(Xbuf) == len(Ybuf)
    assert (X.shape0s == Y.shape0s).all()
    assert (X.shape1s == Y.shape1s).all()
    for arr in [A, B, Xbuf, Ybuf]:
        assert (arr.shape1s == arr.stride0s).all()
        assert (arr.stride1s == 1).all()
    for arr in [A, B]:
        assert (arr.shape1s == 1).all()
    assert (B.shape0s >= 1).all()
    assert ((B.shape0s == 1) | (Xbuf.shape0s == B.shape0s)).all()
    assert ((A.shape0s == 1) | (Ybuf.shape0s == A.shape0s)).all()
    assert (Xbuf.shape1s == X.sizes).all()
    assert (Ybuf.shape1s == Y.sizes).all()
    assert X.ctype == Xbuf.ctype
    assert Y.ctype == Ybuf.ctype

    na_max = int(A.sizes.max())
    nb_max = int(B.sizes.max())
    assert nb_max >= 1
    uses_buf = na_max > 1 or nb_max > 1

    max_len = int(X.sizes.max())
    lsize0 = min(max(max_len, na_max, nb_max), get_mwgs(queue))
    assert na_max <= lsize0 and nb_max <= lsize0
    sizes, inds, offsets = blockify_ij(lsize0, X)
    n = len(sizes)

    Xbufpos = to_device(queue, np.zeros(n if uses_buf else 0, dtype="int32"))
    Ybufpos = to_device(queue, np.zeros(n if uses_buf else 0, dtype="int32"))
    tables = dict(offsets=offsets, shape0s=X.shape0s[inds], shape1s=X.shape1s[inds],
                  Xstride0s=X.stride0s[inds], Xstride1s=X.stride1s[inds], Xstarts=X.starts[inds],
                  Ystride0s=Y.stride0s[inds], Ystride1s=Y.stride1s[inds], Ystarts=Y.starts[inds],
                  Ashape0s=A.shape0s[inds], Astarts=A.starts[inds],
                  Bshape0s=B.shape0s[inds], Bstarts=B.starts[inds],
                  Xbufstarts=Xbuf.starts[inds], Ybufstarts=Ybuf.starts[inds])
    dev = {k: to_device(queue, v) for k, v in tables.items()}
    fn, check = _capi.lib().nb2_linearfilter, _capi.check
    args = (n, lsize0, int(uses_buf), dev["offsets"].ptr, dev["shape0s"].ptr, dev["shape1s"].ptr,
            dev["Xstride0s"].ptr, dev["Xstride1s"].ptr, dev["Xstarts"].ptr, X.cl_buf.ptr,
            dev["Ystride0s"].ptr, dev["Ystride1s"].ptr, dev["Ystarts"].ptr, Y.cl_buf.ptr,
            dev["Ashape0s"].ptr, dev["Astarts"].ptr, A.cl_buf.ptr,
            dev["Bshape0s"].ptr, dev["Bstarts"].ptr, B.cl_buf.ptr,
            dev["Xbufstarts"].ptr, Xbuf.cl_buf.ptr, dev["Ybufstarts"].ptr, Ybuf.cl_buf.ptr,
            Xbufpos.ptr, Ybufpos.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (lsize0, max(n, 1)), lsize=(lsize0, 1), n_launches=2 if uses_buf else 1,
                name="cl_linearfilter", tag=tag)
    if not uses_buf:
        plan.phase = _capi.phase("linearfilter", *args)
    plan.full_args = (dev, X.cl_buf, Y.cl_buf, A.cl_buf, B.cl_buf, Xbuf.cl_buf, Ybuf.cl_buf, Xbufpos, Ybufpos)
    plan.tables = dict(tables, sizes=sizes, inds=inds)
    plan.Xbufpos, plan.Ybufpos = Xbufpos, Ybufpos
    plan.bw_per_call = X.nbytes + Y.nbytes + A.nbytes + B.nbytes + Xbuf.nbytes + Ybuf.nbytes
    plan.description = _describe(Y)
    # The ring-position update (the reference's second plan, `cl_linearfilter_inc`)
    # is issued by the same C-ABI call, so a single plan is returned.
    return [plan]


def _plan_learning_delta(queue, rule, name, pre, post, aux, delta, alpha, beta=None, learn=None, scale=None,
                         flops_per_element=4, tag=None):
    """Common launch of plan_bcm / plan_oja / plan_voja (``nb2_learning_delta``)."""
    N = len(pre)
    p = lambda a: None if a is None else a.ptr
    fn, check = _capi.lib().nb2_learning_delta, _capi.check
    max_size = int(delta.sizes.max()) if N else 0
    args = (rule, N, max_size, delta.cl_shape0s.ptr, delta.cl_shape1s.ptr,
            pre.cl_stride0s.ptr, pre.cl_starts.ptr, pre.cl_buf.ptr,
            post.cl_stride0s.ptr, post.cl_starts.ptr, post.cl_buf.ptr,
            aux.cl_stride0s.ptr, aux.cl_starts.ptr, aux.cl_buf.ptr,
            delta.cl_stride0s.ptr, delta.cl_starts.ptr, delta.cl_buf.ptr, alpha.ptr, p(beta),
            None if learn is None else learn.cl_starts.ptr, None if learn is None else learn.cl_buf.ptr,
            None if scale is None else scale.cl_stride0s.ptr, None if scale is None else scale.cl_starts.ptr,
            None if scale is None else scale.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (max_size, N), lsize=None, name=name, tag=tag)
    plan.full_args = (pre, post, aux, delta, alpha, beta, learn, scale)
    plan.flops_per_call = flops_per_element * int(delta.sizes.sum())
    plan.bw_per_call = sum(a.nbytes for a in (pre, post, aux, delta, alpha, beta, learn, scale) if a is not None)
    plan.description = _describe(delta)
    return plan


def plan_bcm(queue, pre, post, theta, delta, alpha, tag=None):
    """``delta = alpha * post * (post - theta) * pre`` (outer product over post x pre)."""
    assert len(pre) == len(post) == len(theta) == len(delta) == alpha.size
    for arr in (pre, post, theta):  # vectors
        assert (arr.shape1s == 1).all()
    for arr in (delta,):  # matrices
        assert (arr.stride1s == 1).all()
    assert (post.shape0s == delta.shape0s).all()
    assert (pre.shape0s == delta.shape1s).all()
    assert (post.shape0s == theta.shape0s).all()
    assert pre.ctype == post.ctype == theta.ctype == delta.ctype
    return _plan_learning_delta(queue, 0, "cl_bcm", pre, post, theta, delta, alpha, flops_per_element=4, tag=tag)


def plan_oja(queue, pre, post, weights, delta, alpha, beta, tag=None):
    """``delta = alpha * post * (pre - beta * weights * post)``"""
    assert len(pre) == len(post) == len(weights) == len(delta) == alpha.size == beta.size
    for arr in (pre, post):  # vectors
        assert (arr.shape1s == 1).all()
    for arr in (delta, weights):  # matrices
        assert (arr.stride1s == 1).all()
    assert (post.shape0s == weights.shape0s).all()
    assert (pre.shape0s == weights.shape1s).all()
    assert (weights.shape0s == delta.shape0s).all()
    assert (weights.shape1s == delta.shape1s).all()
    assert pre.ctype == post.ctype == weights.ctype == delta.ctype
    return _plan_learning_delta(queue, 1, "cl_oja", pre, post, weights, delta, alpha, beta=beta,
                                flops_per_element=5, tag=tag)


def plan_voja(queue, pre, post, enc, delta, learn, scale, alpha, tag=None):
    """``delta = alpha * learn * post * (scale * pre - enc)``"""
    assert len(pre) == len(post) == len(enc) == len(delta) == len(learn) == alpha.size == len(scale)
    for arr in (learn,):  # scalars
        assert (arr.shape0s == 1).all()
        assert (arr.shape1s == 1).all()
    for arr in (pre, post, scale):  # vectors
        assert (arr.shape1s == 1).all()
    for arr in (enc, delta):  # matrices
        assert (arr.stride1s == 1).all()
    assert (post.shape0s == enc.shape0s).all()
    assert (pre.shape0s == enc.shape1s).all()
    assert (enc.shape0s == delta.shape0s).all()
    assert (enc.shape1s == delta.shape1s).all()
    assert pre.ctype == post.ctype == enc.ctype == delta.ctype == learn.ctype == scale.ctype
    return _plan_learning_delta(queue, 2, "cl_voja", pre, post, enc, delta, alpha, learn=learn, scale=scale,
                                flops_per_element=5, tag=tag)


PROBE_WIDE_ELEMENTS = 4096  # probes larger than this are copied by several CTAs


def plan_probes(queue, periods, X, Y, tag=None):
    """Sample ``X[i]`` into row ``bufpositions[i]`` of ``Y[i]`` every ``periods[i]`` steps."""
    assert len(X) == len(Y)
    assert len(X) == len(periods)
    assert X.ctype == Y.ctype
    N = len(X)
    assert (X.shape0s * X.shape1s == Y.shape1s).all()
    assert (Y.stride0s == Y.shape1s).all()
    assert (Y.stride1s == 1).all()

    periods = np.asarray(periods, dtype="float32")
    cl_periods = to_device(queue, periods)
    cl_countdowns = to_device(queue, periods - 1)
    cl_bufpositions = to_device(queue, np.zeros(N, dtype="int32"))
    max_len = int(min(max(X.shape0s), get_mwgs(queue)))
    check = _capi.check
    tables = (cl_countdowns.ptr, cl_bufpositions.ptr, cl_periods.ptr, X.cl_starts.ptr,
              X.cl_shape0s.ptr, X.cl_shape1s.ptr, X.cl_stride0s.ptr, X.cl_stride1s.ptr, X.cl_buf.ptr,
              Y.cl_starts.ptr, Y.cl_buf.ptr)
    largest = int(max(X.shape0s * X.shape1s))
    cl_arrive = None
    if largest > PROBE_WIDE_ELEMENTS:
        # a probe of a whole population: several CTAs per probe (one CTA would copy it serially)
        chunks = int(min(-(-largest // PROBE_WIDE_ELEMENTS), 128))
        cl_arrive = to_device(queue, np.zeros(N, dtype="int32"))
        fn = _capi.lib().nb2_probes_wide
        args = (N, chunks) + tables + (cl_arrive.ptr,)
    else:
        fn = _capi.lib().nb2_probes
        args = (N, max_len) + tables

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (max_len, N), lsize=(max_len, 1), name="cl_probes", tag=tag)
    if cl_arrive is None:
        plan.phase = _capi.phase("probes", *args)
    plan.full_args = (cl_countdowns, cl_bufpositions, cl_periods, X, Y, cl_arrive)
    plan.cl_bufpositions = cl_bufpositions
    plan.cl_countdowns = cl_countdowns
    plan.periods = periods
    plan.Y = Y
    plan.bw_per_call = 2 * X.nbytes + cl_periods.nbytes + cl_countdowns.nbytes + cl_bufpositions.nbytes
    plan.description = _describe(X)
    return plan


def plan_direct(queue, code, init, input_names, inputs, output, tag=None):
    """Run a translated node function, one instance per item.

    ``code`` is a ``DeviceFunction`` (postfix program + constant pool) from
    ``nengo_ocl_b200.ast_conversion``; ``init`` is unused and kept for
    signature parity with the reference (clra_nonlinearities.py:954)."""
    assert len(input_names) == len(inputs)
    assert len(inputs) <= 2
    N = len(output)
    for x in inputs:
        assert len(x) == len(output)
    for x in list(inputs) + [output]:
        assert (x.shape1s == 1).all() and (x.stride1s == 1).all()
        assert (x.stride0s == 1).all()

    prog = to_device(queue, np.asarray(code.program, dtype=np.int32).reshape(-1, 2))
    # (the pool travels as raw 64-bit words: device arrays are float32 / int32 typed)
    consts = to_device(queue, np.asarray(list(code.constants) + [0.0], dtype=np.float64).view(np.int32))
    n_ops = len(code.program)
    ins = list(inputs) + [None, None]
    fn, check = _capi.lib().nb2_direct, _capi.check
    args = (N, prog.ptr, n_ops, code.max_depth, consts.ptr, int(output.shape0s.max()),
            None if ins[0] is None else ins[0].cl_starts.ptr, None if ins[0] is None else ins[0].cl_buf.ptr,
            None if ins[1] is None else ins[1].cl_starts.ptr, None if ins[1] is None else ins[1].cl_buf.ptr,
            output.cl_starts.ptr, output.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (max(N, 1),), lsize=None, name="cl_direct", tag=tag)
    plan.phase = _capi.phase("direct", *args)
    plan.full_args = (prog, consts, inputs, output)
    plan.description = _describe(output)
    return plan


# ---- convolution and pooling on one image ----------------------------------------------
def _contiguous_item(ary):
    assert len(ary.shape) in (1, 2)
    assert ary.strides[-1] == ary.dtype.itemsize
    if len(ary.shape) == 2:
        assert ary.strides[0] == ary.dtype.itemsize * ary.shape[1]


def plan_conv2d(queue, X, Y, filters, shape_in, shape_out, kernel_shape, conv=True, biases=None, padding=(0, 0),
                strides=(1, 1), channels_last=True, tag=None, transposed=False, inc=False):
    """``Y = conv(X, filters)`` (``inc``: ``Y +=``) on one image (reference: plan_conv2d, clra_nonlinearities.py:1762-1969).

    ``X``, ``Y``, ``filters``: single device items (``CUDARaggedArray.getitem_device``), contiguous.
    ``filters``: (size_i, size_j, channels, n_filters) when ``conv``; for local filtering
    (``conv=False``) (n_filters, channels, size_i, size_j, rows_out, cols_out).  ``padding``:
    "valid", "same" or a pair."""
    assert biases is None, "Not tested with biases (strides may be wrong)"
    assert not transposed
    for ary in (X, Y, filters):
        _contiguous_item(ary)
        assert ary.ctype == Y.ctype
    si, sj = (int(v) for v in kernel_shape)
    sti, stj = (int(v) for v in strides)
    if channels_last:
        (nxi, nxj, nc), (nyi, nyj, nf) = shape_in, shape_out
    else:
        (nc, nxi, nxj), (nf, nyi, nyj) = shape_in, shape_out
    if padding == "valid":
        pi, pj = 0, 0
    elif padding == "same":
        pi, pj = (si - 1) // 2, (sj - 1) // 2
    elif isinstance(padding, (tuple, list)) and len(padding) == 2:
        pi, pj = padding
    else:
        raise ValueError("Unsupported padding (must be 'same', 'valid', or 2-tuple)")
    assert X.size == nc * nxi * nxj and Y.size == nf * nyi * nyj
    assert filters.size == (si * sj * nc * nf if conv else nf * nc * si * sj * nyi * nyj)
    fn, check = _capi.lib().nb2_conv2d, _capi.check
    args = (X.ptr, filters.ptr, Y.ptr, int(nc), int(nxi), int(nxj), int(nf), int(nyi), int(nyj), si, sj, sti, stj,
            int(pi), int(pj), int(bool(channels_last)), int(bool(conv)), int(bool(inc)))

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (int(nyj), int(nyi), int(nf)), lsize=None, name="cl_conv2d", tag=tag)
    plan.full_args = (X, filters, Y)
    plan.flops_per_call = 2 * nyi * nyj * nf * nc * si * sj
    plan.bw_per_call = X.nbytes + filters.nbytes + Y.nbytes
    plan.description = "shape_in=%s, shape_out=%s, kernel=%s, conv=%s" % (shape_in, shape_out, kernel_shape, conv)
    return plan


def plan_pool2d(queue, X, Y, shape, pool_size, strides, tag=None):
    """Average pooling of one (channels, rows, cols) image (reference: plan_pool2d, :1972-2079);
    ``shape`` = (channels, rows_out, cols_out, rows_in, cols_in)."""
    for ary in (X, Y):
        _contiguous_item(ary)
    assert X.ctype == Y.ctype
    nc, nyi, nyj, nxi, nxj = (int(v) for v in shape)
    si, sj = (int(v) for v in pool_size)
    sti, stj = (int(v) for v in strides)
    assert X.size == nc * nxi * nxj and Y.size == nc * nyi * nyj
    fn, check = _capi.lib().nb2_pool2d, _capi.check
    args = (X.ptr, Y.ptr, nc, nyi, nyj, nxi, nxj, si, sj, sti, stj)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (nyj, nyi, nc), lsize=None, name="cl_pool2d", tag=tag)
    plan.full_args = (X, Y)
    plan.flops_per_call = X.size
    plan.bw_per_call = X.nbytes + Y.nbytes
    return plan


# ---- white noise ---------------------------------------------------------------------
def create_rngs(queue, n):
    """Generator "states" of n noise processes.  The reference allocates up to 32 RANLUX states
    of 28 words per process (clra_nonlinearities.py:1486-1493); the counter-based Philox
    generator used here has no state, only a 64-bit key per process: an (n, 2) uint32 array."""
    return to_device(queue, np.zeros((n, 2), dtype=np.uint32).view(np.int32))


def init_rngs(queue, rngs, seeds):
    """Write the processes' seeds as Philox keys (reference: init_rngs, :1499-1532)."""
    seeds = [int(s) for s in seeds]
    assert len(seeds) == rngs.shape[0]
    keys = np.array([[s & 0xFFFFFFFF, (s >> 32) & 0xFFFFFFFF] for s in seeds], dtype=np.uint32)
    rngs.set(keys.view(np.int32))


_dist_enums = {"Uniform": 0, "Gaussian": 1}


def get_dist_enums_params(dists):
    """(enums, params) ragged arrays of a list of distributions (:1571-1574): Uniform -> 0,
    (low, high); Gaussian -> 1, (mean, std)."""
    from nengo_ocl_b200.raggedarray import RaggedArray

    enums = [np.array([_dist_enums[type(d).__name__]]) for d in dists]
    params = [np.array([d.low, d.high] if type(d).__name__ == "Uniform" else [d.mean, d.std], dtype=np.float32)
              for d in dists]
    return RaggedArray(enums, dtype=np.int32), RaggedArray(params, dtype=np.float32)


def plan_whitenoise(queue, Y, dist_enums, dist_params, scale, inc, dt, rngs, t, tag=None):
    """``Y[k] (+)= sample of dist k [* 1/sqrt(dt)]`` every step (reference: plan_whitenoise,
    :1577-1675).  ``rngs``: the Philox keys from ``create_rngs`` / ``init_rngs``; ``t``: the
    step-counter signal, one (view of the) item per process, which makes the stream a function of
    (seed, step, element) alone.  ``scale`` / ``inc``: int32 device arrays as in the reference."""
    N = len(Y)
    assert N == len(dist_enums) == len(dist_params) == len(t) == scale.size == inc.size == rngs.shape[0]
    assert dist_enums.ctype == "int"
    for arr in [Y, dist_enums, dist_params]:
        assert (arr.shape1s == 1).all()
        assert (arr.stride0s == 1).all()
        assert (arr.stride1s == 1).all()
    assert (dist_enums.shape0s == 1).all() and (dist_params.shape0s == 2).all()
    assert (t.shape0s == 1).all() and (t.shape1s == 1).all()
    # one enum and two parameters per item, packed in item order
    enums = to_device(queue, np.array([int(dist_enums[k][0, 0]) for k in range(N)], dtype=np.int32))
    params = to_device(queue, np.array([np.asarray(dist_params[k]).reshape(2) for k in range(N)], dtype=np.float32))
    max_len = int(max(Y.shape0s))
    fn, check = _capi.lib().nb2_whitenoise, _capi.check
    args = (N, max_len, Y.cl_shape0s.ptr, Y.cl_starts.ptr, Y.cl_buf.ptr, t.cl_starts.ptr, t.cl_buf.ptr, enums.ptr,
            params.ptr, scale.ptr, inc.ptr, rngs.ptr, float(dt))

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (min(max_len, 256), N), lsize=(min(max_len, 256), 1), name="cl_whitenoise", tag=tag)
    plan.full_args = (Y, t, enums, params, scale, inc, rngs)
    plan.bw_per_call = int(Y.nbytes)
    plan.description = _describe(Y)
    return plan


def plan_presentinput(queue, Y, t, signals, dt, pres_t=None, tag=None):
    """``Y[k] = signals[k][ti]`` with ``ti = step % nt`` or the presentation-time form."""
    N = len(Y)
    assert len(Y) == len(t) == len(signals)
    assert pres_t is None or pres_t.shape == (N,)
    for arr in [Y, t, signals]:
        assert (arr.stride1s == 1).all()
    assert (Y.shape1s == 1).all()
    assert (Y.stride0s == 1).all()
    assert (t.shape0s == 1).all()
    assert (t.shape1s == 1).all()
    assert (Y.shape0s == signals.shape1s).all()

    max_len = int(min(max(Y.shape0s), get_mwgs(queue)))
    fn, check = _capi.lib().nb2_presentinput, _capi.check
    packed = bool((signals.stride0s == signals.shape1s).all())
    args = (N, max_len, _ptr(pres_t), float(dt), Y.cl_shape0s.ptr, Y.cl_starts.ptr, Y.cl_buf.ptr,
            t.cl_starts.ptr, t.cl_buf.ptr, signals.cl_shape0s.ptr, signals.cl_starts.ptr,
            None if packed else signals.cl_stride0s.ptr, signals.cl_buf.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (max_len, N), lsize=(max_len, 1), name="cl_presentinput", tag=tag)
    plan.phase = _capi.phase("presentinput", *args)
    plan.full_args = (pres_t, Y, t, signals)
    return plan


# ---- neuron models -----------------------------------------------------------
def _plan_template(queue, name, kind, tag=None, blockify=True, inputs=None, outputs=None, parameters=None,
                   dt=0.001, upsample=1, adaptive=False, fastlif=False):
    """Blocked element-wise launch over lists of vectors.

    Same contract as the reference's ``_plan_template``
    (clra_nonlinearities.py:1286-1483): all inputs/outputs/array parameters are
    ragged lists of contiguous vectors of equal lengths; float parameters are
    compile-time constants there and kernel arguments here.  The block size is
    the one in {16..1024} giving the fewest blocks (ties -> smallest).
    """
    inputs = {} if inputs is None else inputs
    outputs = {} if outputs is None else outputs
    parameters = {} if parameters is None else parameters
    input0 = list(inputs.values())[0]

    static_params, params = {}, {}
    for k, v in parameters.items():
        if isinstance(v, CUDARaggedArray):
            params[k] = v
        elif is_number(v):
            static_params[k] = float(v)
        else:
            raise ValueError("Parameter %r must be CLRaggedArray or float (got %s)" % (k, type(v)))

    bw_per_call = 0
    seen = set()
    for vname, v in list(inputs.items()) + list(outputs.items()) + list(params.items()):
        assert vname not in seen, "Name clash"
        seen.add(vname)
        assert len(v) == len(input0)
        assert (v.shape0s == input0.shape0s).all()
        assert (v.stride0s == v.shape1s).all()
        assert (v.stride1s == 1).all()
        assert (v.shape1s == 1).all()
        bw_per_call += v.nbytes

    if blockify:
        best = None
        for block_size_i in [16, 32, 64, 128, 256, 512, 1024]:
            sizes_i, inds_i, _ = blockify_vector(block_size_i, input0)
            if best is None or len(sizes_i) < len(best[1]):
                best = (block_size_i, sizes_i, inds_i)
        block_size, sizes, inds = best
        starts_of = lambda ra: blockify_vector(block_size, ra)[2]
    else:
        block_size = int(min(input0.shape0s.max(), 1024))
        assert input0.shape0s.max() <= 1024, "blockify=False needs vectors of <= 1024 elements"
        sizes = input0.shape0s.copy()
        inds = np.arange(len(input0), dtype=np.int32)
        starts_of = lambda ra: np.asarray(ra.starts)

    clsizes = to_device(queue, sizes)
    args = _capi.nb2_neuron_args()
    keep = [clsizes]
    tables = {"sizes": sizes, "inds": inds}
    # variable name in the reference's template -> field of nb2_neuron_args
    field_of = {"J": "J", "V": "V", "W": "W", "N": "N", "outV": "V", "outW": "W", "outN": "N",
                "outS": "S", "R": "S", "tau": "tau", "ref": "ref", "amp": "amp", "tau_n": "tau_n",
                "inc_n": "inc_n"}
    for vname, v in list(inputs.items()) + list(outputs.items()) + list(params.items()):
        starts = starts_of(v)
        tables[vname + "_starts"] = starts
        field = getattr(args, field_of[vname])
        if field.buf and field.buf != v.cl_buf.data:
            raise NotImplementedError("in-place variables must share one buffer (%s)" % vname)
        d_starts = to_device(queue, starts)
        keep += [d_starts, v.cl_buf]
        field.starts = d_starts.data
        field.buf = v.cl_buf.data
    for vname, value in static_params.items():
        field = getattr(args, field_of[vname])
        field.buf = None
        field.value = value
    args.dt = float(dt)
    args.upsample = int(upsample)
    args.adaptive = int(bool(adaptive))
    args.fastlif = int(bool(fastlif))
    n_blocks = len(sizes)
    fn, check = _capi.lib().nb2_neurons, _capi.check
    args_ref = ctypes.byref(args)

    def launch(stream):
        check(fn(stream, kind, n_blocks, block_size, clsizes.ptr, args_ref))

    plan = Plan(queue, launch, (block_size, max(n_blocks, 1)), lsize=None, name=name, tag=tag)
    plan.full_args = (keep, args)
    plan.tables = tables
    plan.block_size = block_size
    plan.bw_per_call = bw_per_call
    plan.description = "groups: %d; items: %d; items/group: %0.1f [%d, %d]" % (
        n_blocks, input0.sizes.sum(), input0.sizes.mean(), input0.sizes.min(), input0.sizes.max())
    return plan


def plan_lif(queue, dt, J, V, W, outS, ref, tau, amp, N=None, tau_n=None, inc_n=None, upsample=1,
             fastlif=False, **kwargs):
    adaptive = N is not None
    assert J.ctype == "float"
    for x in [V, W, outS]:
        assert x.ctype == J.ctype
    inputs = dict(J=J, V=V, W=W)
    outputs = dict(outV=V, outW=W, outS=outS)
    parameters = dict(tau=tau, ref=ref, amp=amp)
    if adaptive:
        assert all(x is not None for x in [N, tau_n, inc_n])
        assert N.ctype == J.ctype
        inputs["N"] = N
        outputs["outN"] = N
        parameters.update(tau_n=tau_n, inc_n=inc_n)
    return _plan_template(queue, "cl_alif" if adaptive else "cl_lif", _capi.NEURON_LIF, inputs=inputs,
                          outputs=outputs, parameters=parameters, dt=float(dt), upsample=upsample,
                          adaptive=adaptive, fastlif=fastlif, **kwargs)


def plan_lif_rate(queue, dt, J, R, ref, tau, amp, N=None, tau_n=None, inc_n=None, **kwargs):
    assert J.ctype == "float"
    assert R.ctype == J.ctype
    adaptive = N is not None
    inputs = dict(J=J)
    outputs = dict(R=R)
    parameters = dict(tau=tau, ref=ref, amp=amp)
    if adaptive:
        assert all(x is not None for x in [N, tau_n, inc_n])
        assert N.ctype == J.ctype
        inputs["N"] = N
        outputs["outN"] = N
        parameters.update(tau_n=tau_n, inc_n=inc_n)
    return _plan_template(queue, "cl_alif_rate" if adaptive else "cl_lif_rate", _capi.NEURON_LIF_RATE,
                          inputs=inputs, outputs=outputs, parameters=parameters, dt=float(dt),
                          adaptive=adaptive, **kwargs)


def plan_spiking_rectified_linear(queue, dt, J, V, outS, amp, **kwargs):
    assert J.ctype == "float"
    for x in [V, outS, amp]:
        assert x.ctype == J.ctype
    return _plan_template(queue, "cl_spikingrelu", _capi.NEURON_SPIKING_RELU, inputs=dict(J=J, V=V),
                          outputs=dict(outV=V, outS=outS), parameters=dict(amp=amp), dt=float(dt), **kwargs)


def plan_rectified_linear(queue, J, R, amp, **kwargs):
    assert J.ctype == "float"
    for x in [R, amp]:
        assert x.ctype == J.ctype
    return _plan_template(queue, "cl_relu", _capi.NEURON_RELU, inputs=dict(J=J), outputs=dict(R=R),
                          parameters=dict(amp=amp), **kwargs)


def plan_sigmoid(queue, J, R, ref, **kwargs):
    assert J.ctype == "float"
    assert R.ctype == J.ctype
    return _plan_template(queue, "cl_sigmoid", _capi.NEURON_SIGMOID, inputs=dict(J=J), outputs=dict(R=R),
                          parameters=dict(ref=ref), **kwargs)


__all__ = [n for n in dir() if n.startswith(("plan_", "blockify", "get_mwgs"))] + ["nonelist"]
