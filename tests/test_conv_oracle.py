"""The oracle's conv2d / pool2d restatement (clra_nonlinearities.py:1799-1873, :1984-2030) against an
independent direct evaluation of the definition, and the ConvInc operator in the oracle simulator."""

import numpy as np
import pytest

from nengo_ocl_b200 import synth
from oracle import kernels as K
from oracle.simulator import OracleSimulator


def direct_conv(x, f, nxi, nxj, nc, nf, si, sj, pi, pj, sti, stj):
    nyi, nyj = (nxi + 2 * pi - si) // sti + 1, (nxj + 2 * pj - sj) // stj + 1
    y = np.zeros((nyi, nyj, nf))
    for i in range(nyi):
        for j in range(nyj):
            for k in range(nf):
                acc = 0.0
                for c in range(nc):
                    for ii in range(si):
                        for jj in range(sj):
                            xi, xj = i * sti - pi + ii, j * stj - pj + jj
                            if 0 <= xi < nxi and 0 <= xj < nxj:
                                acc += float(f[ii, jj, c, k]) * float(x[xi, xj, c])
                y[i, j, k] = acc
    return y


@pytest.mark.parametrize("padding,strides", [("valid", (1, 1)), ("same", (2, 1)), ((1, 0), (1, 2))])
@pytest.mark.parametrize("channels_last", [True, False])
def test_conv2d_oracle_follows_the_definition(padding, strides, channels_last):
    rng = np.random.RandomState(0)
    nxi, nxj, nc, nf, si, sj = 7, 9, 3, 4, 3, 2
    x = rng.normal(size=(nxi, nxj, nc)).astype(np.float32)
    f = rng.normal(size=(si, sj, nc, nf)).astype(np.float32)
    pi, pj = (0, 0) if padding == "valid" else ((si - 1) // 2, (sj - 1) // 2) if padding == "same" else padding
    want = direct_conv(x, f, nxi, nxj, nc, nf, si, sj, pi, pj, *strides)
    nyi, nyj = want.shape[:2]
    if channels_last:
        got = K.conv2d(x, f, (nxi, nxj, nc), (nyi, nyj, nf), (si, sj), True, padding, strides, True)
        got = got.reshape(nyi, nyj, nf)
    else:
        got = K.conv2d(x.transpose(2, 0, 1), f, (nc, nxi, nxj), (nf, nyi, nyj), (si, sj), True, padding, strides,
                       False)
        got = got.reshape(nf, nyi, nyj).transpose(1, 2, 0)
    assert got.dtype == np.float32
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_local_filters_and_pooling():
    rng = np.random.RandomState(1)
    nxi, nxj, nc, nf, si, sj = 5, 6, 2, 3, 2, 2
    nyi, nyj = nxi - si + 1, nxj - sj + 1
    x = rng.normal(size=(nc, nxi, nxj)).astype(np.float32)
    f = rng.normal(size=(nf, nc, si, sj, nyi, nyj)).astype(np.float32)
    got = K.conv2d(x, f, (nc, nxi, nxj), (nf, nyi, nyj), (si, sj), False, "valid", (1, 1), False).reshape(nf, nyi, nyj)
    want = np.zeros((nf, nyi, nyj))
    for k in range(nf):
        for i in range(nyi):
            for j in range(nyj):
                want[k, i, j] = sum(float(f[k, c, ii, jj, i, j]) * float(x[c, i + ii, j + jj])
                                    for c in range(nc) for ii in range(si) for jj in range(sj))
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
    # pooling: windows that overhang the image average what lies inside
    xp = rng.normal(size=(2, 5, 7)).astype(np.float32)
    yp = K.pool2d(xp, (2, 3, 4, 5, 7), (2, 2), (2, 2)).reshape(2, 3, 4)
    assert np.isclose(yp[0, 0, 0], xp[0, :2, :2].mean(), rtol=1e-6)
    assert np.isclose(yp[1, 2, 3], xp[1, 4:6, 6:8].mean(), rtol=1e-6)  # a 1 x 1 remainder
    assert np.isclose(yp[1, 2, 0], xp[1, 4:6, 0:2].mean(), rtol=1e-6)  # a 1 x 2 remainder


@pytest.mark.parametrize("one_d", [False, True])
def test_oracle_runs_a_convolution_model(one_d):
    mdl = synth.convolution_model(one_d=one_d)
    ora = OracleSimulator(mdl)
    ora.run_steps(5)
    conv1, conv2 = mdl.info["convs"]
    y = np.array(ora.probe_data[mdl.probes[0]])
    assert y.shape == (5, int(np.prod(conv2.output_shape))) and np.isfinite(y).all() and np.abs(y).max() > 0
