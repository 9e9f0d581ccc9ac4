"""CPU restatement (numpy, float32) of the reference's device kernels.

TEST INFRASTRUCTURE ONLY: this module is the checker the CUDA path is compared
against.  Nothing in the product package imports it; only ``tests/``, the
smoke check and the CPU-baseline leg of the benchmark do.

Each function works on host ``RaggedArray`` objects in place and follows the
arithmetic and the operation order of the OpenCL kernel it cites (paths are
relative to the nengo-ocl source tree).  Arithmetic is IEEE float32 without
fused multiply-add; ``expm1``/``log1p``/``exp`` are evaluated in float64 and
rounded once, i.e. a correctly-rounded float32 math library.

Parity status: the GEMV, copy, elementwise, reset and sliced-copy kernels are
pinned by the reference's own known-answer tests and by index tables captured
from the reference's planners (tests/golden).  The LIF / LIF-rate / linear
filter kernels are pinned against outputs of the reference's own kernel source
executed on the CPU (tests/golden/make_golden.py); the reference's tests pin
them only against nengo's numpy neuron models, which are not available here.
"""

import numpy as np

f32 = np.float32


def _f(x):
    return np.asarray(x, dtype=np.float32)


# ---- GEMV --------------------------------------------------------------------
def _scale(arg, bb):
    """Scalar (python float -> double, as rendered into the kernel text) or
    per-item float32 vector."""
    if isinstance(arg, (float, int)):
        return float(arg), True
    arr = np.asarray(arg)
    if arr.ndim == 0:
        return float(arr), True
    if len(set(arr.tolist())) == 1:
        return float(arr[0]), True
    return f32(arr[bb]), False


def gemv_ref(alpha, A, A_js, X, X_js, beta, Y, Y_in=None, gamma=0.0):
    """``ref_impl`` (nengo_ocl/clra_gemv.py:330-385): per output row
    ``Y = gamma + beta*Y_in``; one running float sum over all terms in list
    order and n ascending; ``Y += alpha * sum``.  beta/gamma are float
    variables there; a python-float alpha is a double literal."""
    Y_in = Y if Y_in is None else Y_in
    out = []
    for bb in range(len(Y)):
        M = int(Y.shape0s[bb])
        b, _ = _scale(beta, bb)
        g, _ = _scale(gamma, bb)
        yin = _f(Y_in[bb][:, 0])
        y = f32(g) + f32(b) * yin
        acc = np.zeros(M, dtype=np.float32)
        if A_js is not None:
            ajs = np.asarray(A_js[bb]).ravel()
            xjs = np.asarray(X_js[bb]).ravel()
            for aj, xj in zip(ajs, xjs):
                a = A[int(aj)]
                x = X[int(xj)][:, 0]
                for nn in range(a.shape[1]):
                    acc = acc + x[nn] * a[:, nn]
        a_val, a_is_double = _scale(alpha, bb)
        if a_is_double:
            y = (y.astype(np.float64) + a_val * acc.astype(np.float64)).astype(np.float32)
        else:
            y = y + a_val * acc
        out.append(y)
    for bb, y in enumerate(out):
        Y[bb][:, 0] = y


def gemv_many_dots(alpha, A, A_js, X, X_js, beta, Y, Y_in=None, gamma=0.0, max_work_group_size=1024):
    """``many_dots_impl`` (clra_gemv.py:749-827): terms are dealt round-robin to
    ``dot_block_size`` partial sums (each serial in n), the partial sums are
    added in order, and ``Y = (beta*Y_in [+ gamma]) + alpha*sum`` with the
    scalar products evaluated in double."""
    Y_in = Y if Y_in is None else Y_in
    max_n_dots = int(max(A_js.shape0s))
    max_y_len = int(max(Y.shape0s))
    segment_size = min(max_y_len, 16)
    dbs = min(max(max_n_dots, 1), int(max_work_group_size / segment_size))
    out = []
    for bb in range(len(Y)):
        M = int(Y.shape0s[bb])
        yin = _f(Y_in[bb][:, 0])
        b, _ = _scale(beta, bb)
        g, _ = _scale(gamma, bb)
        pre = (b * yin.astype(np.float64)).astype(np.float32) if b != 0 else np.zeros(M, np.float32)
        if g != 0:
            pre = (pre.astype(np.float64) + g).astype(np.float32)
        ajs = np.asarray(A_js[bb]).ravel()
        xjs = np.asarray(X_js[bb]).ravel()
        partial = np.zeros((dbs, M), dtype=np.float32)
        for ii, (aj, xj) in enumerate(zip(ajs, xjs)):
            a = A[int(aj)]
            x = X[int(xj)][:, 0]
            blk = ii % dbs
            for nn in range(a.shape[1]):
                partial[blk] = partial[blk] + a[:, nn] * x[nn]
        total = partial[0].copy()
        for ii in range(1, dbs):
            total = total + partial[ii]
        a_val, _ = _scale(alpha, bb)
        out.append((pre.astype(np.float64) + a_val * total.astype(np.float64)).astype(np.float32))
    for bb, y in enumerate(out):
        Y[bb][:, 0] = y


def gemv_block(alpha, A, A_js, X, X_js, beta, Y, Y_in=None, gamma=0.0, block_y=32, block_x=128, lsize0=4):
    """``block_impl`` (clra_gemv.py:1018-1058,1137-1153): every (32 x 128) tile
    is reduced by 4 strided lanes, combined as ``(s0 + s2) + (s1 + s3)`` and
    scaled by alpha (double literal) into a scratch buffer; the reduce pass
    computes ``beta*y_in + tiles in order + gamma``."""
    Y_in = Y if Y_in is None else Y_in
    alpha = float(alpha)
    beta = float(beta)
    gamma = float(gamma)
    out = []
    for n in range(len(Y)):
        M = int(Y.shape0s[n])
        yin = _f(Y_in[n][:, 0])
        total = (beta * yin.astype(np.float64)).astype(np.float32)
        ajs = np.asarray(A_js[n]).ravel()
        xjs = np.asarray(X_js[n]).ravel()
        for aj, xj in zip(ajs, xjs):
            a = A[int(aj)]
            x = X[int(xj)][:, 0]
            N = a.shape[1]
            for j0 in range(0, N, block_x):
                w = min(N - j0, block_x)
                lanes = np.zeros((lsize0, M), dtype=np.float32)
                for jj in range(w):
                    lane = jj % lsize0
                    lanes[lane] = lanes[lane] + a[:, j0 + jj] * x[j0 + jj]
                # tree over lanes: k = log2(lsize0)-1 .. 1, then (s0 + s1)
                k = lsize0 // 2
                while k > 1:
                    lanes[:k] = lanes[:k] + lanes[k : 2 * k]
                    k //= 2
                tile = (alpha * (lanes[0] + lanes[1]).astype(np.float64)).astype(np.float32)
                total = total + tile
        out.append((total.astype(np.float64) + gamma).astype(np.float32))
    for n, y in enumerate(out):
        Y[n][:, 0] = y


def gemv_exact(alpha, A, A_js, X, X_js, beta, Y, Y_in=None, gamma=0.0):
    """float64 value of the same expression and the sum of |terms| per row
    (the scale a float32 evaluation's error is measured against)."""
    Y_in = Y if Y_in is None else Y_in
    vals, mags = [], []
    for bb in range(len(Y)):
        b, _ = _scale(beta, bb)
        g, _ = _scale(gamma, bb)
        a_val, _ = _scale(alpha, bb)
        yin = Y_in[bb][:, 0].astype(np.float64)
        y = g + b * yin
        mag = np.abs(g) + np.abs(b * yin)
        if A_js is not None:
            for aj, xj in zip(np.asarray(A_js[bb]).ravel(), np.asarray(X_js[bb]).ravel()):
                a = A[int(aj)].astype(np.float64)
                x = X[int(xj)][:, 0].astype(np.float64)
                y = y + a_val * (a @ x)
                mag = mag + np.abs(a_val) * (np.abs(a) @ np.abs(x))
        vals.append(y)
        mags.append(mag)
    return vals, mags


# ---- elementwise family ---------------------------------------------------------
def timeupdate(step, time, dt):
    """clra_nonlinearities.py:128-131: ``step += 1; time = dt * step`` (dt double literal)."""
    s = f32(step[0][0, 0] + f32(1))
    step[0][0, 0] = s
    time[0][0, 0] = f32(float(dt) * float(s))


def reset(Y, values):
    """clra_nonlinearities.py:163-170"""
    for n in range(len(Y)):
        Y[n][...] = f32(values[n])


def copy(X, Y, incs):
    """clra_nonlinearities.py:242-260"""
    for n in range(len(X)):
        if incs[n]:
            Y[n][...] = Y[n] + X[n]
        else:
            Y[n][...] = X[n]


def slicedcopy(X, Y, Xinds, Yinds, incs):
    """clra_nonlinearities.py:340-362 (X, Y lists of vectors; index lists per item)"""
    for n in range(len(X)):
        xi = np.asarray(Xinds[n]).ravel()
        yi = np.asarray(Yinds[n]).ravel()
        x = X[n][:, 0]
        y = Y[n][:, 0]
        if incs[n]:
            y[yi] = y[yi] + x[xi]
        else:
            y[yi] = x[xi]


def elementwise_inc(A, X, Y, alpha=None, outer=False, inc=True):
    """clra_nonlinearities.py:489-523: ``y (+)= alpha * aa * xx`` (left to right)."""
    for n in range(len(Y)):
        a, x, y = A[n], X[n], Y[n]
        al = f32(1) if alpha is None else f32(alpha[n])
        if outer:
            aa = a[:, 0][:, None] if a.shape[0] > 1 else a[0, 0]
            xx = x[:, 0][None, :] if x.shape[0] > 1 else x[0, 0]
        else:
            aa, xx = a, x  # numpy broadcasting matches get_element's rules
        v = _f(al * aa) * xx
        if inc:
            y[...] = y + v
        else:
            y[...] = np.broadcast_to(v, y.shape)


def linearfilter(X, Y, A, B, Xbuf, Ybuf, Xpos, Ypos):
    """clra_nonlinearities.py:632-709; ``Xpos``/``Ypos`` are per-item ring
    positions (numpy int arrays, updated in place like ``linearfilter_inc``)."""
    for k in range(len(X)):
        x = X[k]
        y = Y[k]
        a = A[k][:, 0]
        b = B[k][:, 0]
        na, nb = len(a), len(b)
        if na == 0 and nb == 1:
            y[...] = b[0] * x
        elif na == 1 and nb == 1:
            y[...] = b[0] * x - a[0] * y
        else:
            xb = Xbuf[k]  # (nb, size)
            yb = Ybuf[k]  # (na, size)
            ix, iy = int(Xpos[k]), int(Ypos[k])
            iy1 = iy - 1 if iy > 0 else na - 1
            xf = x.reshape(-1)
            yi = b[0] * xf
            if nb > 1:
                xb[ix] = xf
                for p in range(1, nb):
                    yi = yi + b[p] * xb[(ix + p) % nb]
            if na > 0:
                yi = yi - a[0] * y.reshape(-1)
                if na > 1:
                    for p in range(1, na):
                        yi = yi - a[p] * yb[(iy + p) % na]
                    yb[iy1] = yi
            y[...] = yi.reshape(y.shape)
            Xpos[k] = ix - 1 if ix > 0 else nb - 1
            Ypos[k] = iy - 1 if iy > 0 else na - 1


def probes(countdowns, bufpositions, periods, X, Y):
    """clra_nonlinearities.py:846-900"""
    for n in range(len(X)):
        c = f32(countdowns[n])
        if c <= 0:
            pos = int(bufpositions[n])
            Y[n][pos, :] = np.asarray(X[n]).reshape(-1)
            countdowns[n] = f32(f32(c + f32(periods[n])) - f32(1))
            bufpositions[n] = pos + 1
        else:
            countdowns[n] = f32(c - f32(1))


def presentinput(Y, t, signals, dt, pres_t=None):
    """clra_nonlinearities.py:1710-1728"""
    for k in range(len(Y)):
        it = int(t[k][0, 0])
        nt = int(signals.shape0s[k])
        if pres_t is not None:
            v = f32(f32(f32(it) - f32(0.5)) * f32(f32(dt) / f32(pres_t[k])))
            ti = int(np.fmod(int(v), nt))  # C remainder: sign follows the dividend
        else:
            ti = it % nt
        Y[k][:, 0] = signals[k][ti, :]


# ---- white noise (plan_whitenoise, clra_nonlinearities.py:1573-1675) -----------------------
# The reference draws from RANLUX (pyopencl-ranluxcl.cl, not part of its source tree): its random
# STREAM cannot be restated, only the use it makes of a sample (:1536-1551, :1625-1637):
#   uniform:  low + (high - low) * u        gaussian:  mean + std * z
#   then `sample *= 1/sqrt(dt)` (a double literal) when `scale`, then `y += sample` or `y = sample`.
# The generator here is Philox4x32-10 (Salmon et al., SC'11, "Parallel random numbers: as easy as
# 1, 2, 3"): counter = (step, element // 4, 0, 0), key = the 64-bit seed of the process; word e % 4
# of the output belongs to element e.  u = (word >> 8) * 2^-24 in [0, 1); normals by Box-Muller in
# double on the word pairs (0, 1) and (2, 3), rounded to float32 once.
PHILOX_M0, PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
PHILOX_W0, PHILOX_W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)


def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds on arrays of uint32: counter = 4 words, key = 2 words."""
    c = [np.asarray(x, dtype=np.uint32) for x in counter]
    k = [np.asarray(x, dtype=np.uint32) for x in key]
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = PHILOX_M0 * c[0].astype(np.uint64)
            p1 = PHILOX_M1 * c[2].astype(np.uint64)
            hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), p0.astype(np.uint32)
            hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), p1.astype(np.uint32)
            c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
            k = [k[0] + PHILOX_W0, k[1] + PHILOX_W1]
    return c


def whitenoise_samples(seed, step, m, dist_enum, params, scale, dt):
    """The m float32 samples of one process at one step (before the inc / set)."""
    quads = (m + 3) // 4
    q = np.arange(quads, dtype=np.uint32)
    zero = np.zeros(quads, dtype=np.uint32)
    seed = int(seed)
    w = philox4x32_10([np.full(quads, step, dtype=np.uint32), q, zero, zero],
                      [np.full(quads, seed & 0xFFFFFFFF, dtype=np.uint32),
                       np.full(quads, (seed >> 32) & 0xFFFFFFFF, dtype=np.uint32)])
    p0, p1 = f32(params[0]), f32(params[1])
    if dist_enum == 0:
        u = [(x >> np.uint32(8)).astype(np.float32) * f32(2.0 ** -24) for x in w]
        vals = [(p0 + ((p1 - p0) * ui).astype(np.float32)).astype(np.float32) for ui in u]
    elif dist_enum == 1:
        z = []
        for a, b in ((w[0], w[1]), (w[2], w[3])):
            u1 = ((a >> np.uint32(8)).astype(np.float64) + 1.0) * 2.0 ** -24  # (0, 1]
            u2 = (b >> np.uint32(8)).astype(np.float64) * 2.0 ** -24          # [0, 1)
            r = np.sqrt(-2.0 * np.log(u1))
            z += [(r * np.cos(2.0 * np.pi * u2)).astype(np.float32), (r * np.sin(2.0 * np.pi * u2)).astype(np.float32)]
        vals = [(p0 + (p1 * zi).astype(np.float32)).astype(np.float32) for zi in z]
    else:
        raise NotImplementedError(dist_enum)
    out = np.stack(vals, axis=1).reshape(-1)[:m]
    if scale:
        out = (out.astype(np.float64) * (1.0 / np.sqrt(dt))).astype(np.float32)
    return out


def whitenoise(Y, t, dist_enums, dist_params, scales, incs, dt, seeds):
    for k in range(len(Y)):
        m = int(Y.shape0s[k])
        s = whitenoise_samples(seeds[k], int(t[k][0, 0]), m, int(dist_enums[k][0, 0]),
                               np.asarray(dist_params[k]).reshape(-1), bool(scales[k]), dt)
        if incs[k]:
            Y[k][:, 0] = (Y[k][:, 0] + s).astype(np.float32)
        else:
            Y[k][:, 0] = s


# ---- convolution and pooling on one image -----------------------------------------
def conv2d(x, filters, shape_in, shape_out, kernel_shape, conv=True, padding=(0, 0), strides=(1, 1),
           channels_last=True):
    """clra_nonlinearities.py:1799-1873: y[k,i,j] = sum over c, ii, jj (in that order, from zero) of
    filter * x[c, i*sti - pi + ii, j*stj - pj + jj], zero outside the image, float32, each product
    rounded before it is added.  filters: (si, sj, nc, nf) when ``conv`` else (nf, nc, si, sj, nyi, nyj)."""
    si, sj = kernel_shape
    sti, stj = strides
    (nxi, nxj, nc), (nyi, nyj, nf) = (shape_in, shape_out) if channels_last else (
        (shape_in[1], shape_in[2], shape_in[0]), (shape_out[1], shape_out[2], shape_out[0]))
    if padding == "valid":
        pi, pj = 0, 0
    elif padding == "same":
        pi, pj = (si - 1) // 2, (sj - 1) // 2
    else:
        pi, pj = padding
    x = np.asarray(x, dtype=np.float32).reshape(shape_in)
    xc = x.transpose(2, 0, 1) if channels_last else x  # (nc, nxi, nxj)
    padded = np.zeros((nc, nxi + 2 * pi + si * sti + sti, nxj + 2 * pj + sj * stj + stj), dtype=np.float32)
    padded[:, pi:pi + nxi, pj:pj + nxj] = xc
    f = np.asarray(filters, dtype=np.float32)
    f = f.reshape(si, sj, nc, nf) if conv else f.reshape(nf, nc, si, sj, nyi, nyj)
    out = np.zeros((nf, nyi, nyj), dtype=np.float32)
    for c in range(nc):
        for ii in range(si):
            for jj in range(sj):
                patch = padded[c, ii:ii + nyi * sti:sti, jj:jj + nyj * stj:stj][:nyi, :nyj]
                w = f[ii, jj, c, :][:, None, None] if conv else f[:, c, ii, jj]
                out = out + (w * patch[None]).astype(np.float32)
    return (out.transpose(1, 2, 0) if channels_last else out).reshape(-1)


def pool2d(x, shape, pool_size, strides):
    """clra_nonlinearities.py:1984-2030: mean over the part of each window inside the image."""
    nc, nyi, nyj, nxi, nxj = shape
    si, sj = pool_size
    sti, stj = strides
    x = np.asarray(x, dtype=np.float32).reshape(nc, nxi, nxj)
    out = np.zeros((nc, nyi, nyj), dtype=np.float32)
    cnt = np.zeros((nyi, nyj), dtype=np.int32)
    for ii in range(si):
        for jj in range(sj):
            for i in range(nyi):
                for j in range(nyj):
                    xi, xj = i * sti + ii, j * stj + jj
                    if xi < nxi and xj < nxj:
                        out[:, i, j] = out[:, i, j] + x[:, xi, xj]
                        cnt[i, j] += 1
    return (out / cnt[None].astype(np.float32)).astype(np.float32).reshape(-1)


# ---- neuron models ------------------------------------------------------------
def _expm1(x):
    return np.expm1(x.astype(np.float64)).astype(np.float32)


def _log1p(x):
    with np.errstate(divide="ignore", invalid="ignore"):
        return np.log1p(x.astype(np.float64)).astype(np.float32)


def lif(dt, J, V, W, tau, ref, amp, upsample=1, N=None, tau_n=None, inc_n=None, fastlif=False):
    """``cl_lif`` / ``cl_alif`` (clra_nonlinearities.py:1087-1132) on flat
    float32 arrays; returns (V, W, S[, N]).  ``fastlif`` (:1079-1114): the whole
    substep is always integrated, the refractory period scales the voltage
    afterwards, and the spike time is interpolated linearly."""
    J, V, W = _f(J), _f(V).copy(), _f(W).copy()
    tau, ref, amp = _f(tau), _f(ref), _f(amp)
    dtu = f32(float(dt) / upsample)
    dtu_inv = f32(upsample / float(dt))
    dt_inv = f32(1.0 / float(dt))
    one = f32(1)
    spiked = np.zeros(J.shape, dtype=bool)
    for _ in range(upsample):
        W = W - dtu
        if fastlif:
            delta_t = np.full(J.shape, dtu, dtype=np.float32)
        else:
            delta_t = np.where(W > dtu, f32(0), np.where(W < 0, dtu, dtu - W)).astype(np.float32)
        drive = (J - _f(N) - V) if N is not None else (J - V)
        dV = (-_expm1(-delta_t / tau) * drive).astype(np.float32)
        V = (V + dV).astype(np.float32)
        if fastlif:
            scaled = (V * (one - W * dtu_inv)).astype(np.float32)
            V = np.where((V < 0) | (W > dtu), f32(0), np.where(W >= 0, scaled, V)).astype(np.float32)
        over = V > one
        with np.errstate(divide="ignore", invalid="ignore"):
            if fastlif:
                overshoot = (dtu * (V - one) / dV).astype(np.float32)
                w_spike = (ref - overshoot + dtu).astype(np.float32)
            else:
                w_spike = ref + (dtu + tau * _log1p(-(V - one) / (J - one)))
        W = np.where(over, w_spike, W).astype(np.float32)
        if fastlif:
            V = np.where(over, f32(0), V).astype(np.float32)
        else:
            V = np.where(over, f32(0), np.where(V < 0, f32(0), V)).astype(np.float32)
        spiked |= over
    S = np.where(spiked, amp * dt_inv, f32(0)).astype(np.float32)
    if N is not None:
        N = _f(N)
        Nn = N + (f32(dt) / _f(tau_n)) * (_f(inc_n) * S - N)
        return V, W, S, Nn.astype(np.float32)
    return V, W, S


def lif_rate(J, tau, ref, amp):
    """``cl_lif_rate`` (clra_nonlinearities.py:1178-1180); 1/0 -> inf -> rate 0."""
    J = np.maximum(_f(J) - f32(1), f32(0))
    with np.errstate(divide="ignore"):
        return (_f(amp) / (_f(ref) + _f(tau) * _log1p(f32(1) / J))).astype(np.float32)


def relu(J, amp):
    """``cl_relu`` (clra_nonlinearities.py:1245)"""
    return (_f(amp) * np.maximum(_f(J), f32(0))).astype(np.float32)


def spiking_relu(dt, J, V, amp):
    """``cl_spikingrelu`` (clra_nonlinearities.py:1217-1221); returns (V, S)."""
    J, V = _f(J), _f(V)
    dtf = f32(float(dt))
    dt_inv = f32(1.0 / float(dt))
    V = V + np.where(J > 0, dtf * J, f32(0)).astype(np.float32)
    n = np.floor(V)
    return (V - n).astype(np.float32), (_f(amp) * n * dt_inv).astype(np.float32)


def sigmoid(J, ref):
    """``cl_sigmoid`` (clra_nonlinearities.py:1267-1268)"""
    J, ref = _f(J), _f(ref)
    e = np.exp(-J.astype(np.float64)).astype(np.float32)
    mid = f32(1) / (ref * (f32(1) + e))
    return np.where(J < f32(-88), f32(0), np.where(J > f32(15), f32(1) / ref, mid)).astype(np.float32)


def spmv_csr(indices, indptr, data, x, y, inc=False):
    """``sparsedot_inc`` (clra_gemv.py:1591-1617): one row per work-item,
    ``y[row]`` (zeroed first unless ``inc``) accumulates ``A_data[k] * x[A_indices[k]]``
    in storage order, every operation rounded to float32.  Returns the new y."""
    indices, indptr = np.asarray(indices), np.asarray(indptr)
    data, x = _f(data), _f(x).reshape(-1)
    out = _f(y).reshape(-1).copy()
    for row in range(len(indptr) - 1):
        acc = out[row] if inc else f32(0)
        for k in range(int(indptr[row]), int(indptr[row + 1])):
            acc = f32(acc + f32(data[k] * x[indices[k]]))
        out[row] = acc
    return out.reshape(np.shape(y))


def spmv_ell(columns, entries, x, y, inc=False):
    """``sparsedot_inc`` in ELLPACK form (clra_gemv.py:1666-1716): every padded
    entry of a row contributes ``entry * x[column]`` (padding is 0 * x[0]); the
    work-group reduces the products pairwise, halving the stride each time.
    Returns the new y."""
    columns, entries = np.asarray(columns), _f(entries)
    x = _f(x).reshape(-1)
    out = _f(y).reshape(-1).copy()
    n_rows, width = columns.shape
    wg = 1
    while wg < max(width, 1):
        wg *= 2
    for row in range(n_rows):
        prod = np.zeros(wg, dtype=np.float32)
        prod[:width] = entries[row] * x[columns[row]]
        off = wg // 2
        while off > 0:
            prod[:off] = prod[:off] + prod[off:2 * off]
            off //= 2
        out[row] = f32(out[row] + prod[0]) if inc else prod[0]
    return out.reshape(np.shape(y))


def _outer_terms(pre, post):
    return _f(post).reshape(-1, 1), _f(pre).reshape(1, -1)


def bcm(pre, post, theta, alpha):
    """``bcm`` (clra_nonlinearities.py:2126-2129): ``alpha * post * (post - theta) * pre``,
    multiplied left to right in float32; returns the (post, pre) delta matrix."""
    po, pr = _outer_terms(pre, post)
    th = _f(theta).reshape(-1, 1)
    return (((f32(alpha) * po) * (po - th)) * pr).astype(np.float32)


def oja(pre, post, weights, alpha, beta):
    """``oja`` (clra_nonlinearities.py:2232-2235): ``alpha * post * (pre - beta * weights * post)``."""
    po, pr = _outer_terms(pre, post)
    w = _f(weights)
    inner = pr - ((f32(beta) * w) * po)
    return ((f32(alpha) * po) * inner).astype(np.float32)


def voja(pre, post, enc, learn, scale, alpha):
    """``voja`` (clra_nonlinearities.py:2356-2359): ``alpha * learn * post * (scale * pre - enc)``."""
    po, pr = _outer_terms(pre, post)
    sc = _f(scale).reshape(-1, 1)
    return (((f32(alpha) * f32(learn)) * po) * (sc * pr - _f(enc))).astype(np.float32)
