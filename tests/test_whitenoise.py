"""White-noise processes on the CPU side: the Philox4x32-10 restatement against the generator's
published known-answer vectors, the distributions it is turned into, and the oracle's
operator.  (The reference draws from RANLUX, clra_nonlinearities.py:1486-1568, whose source is
not part of its tree: the random stream itself has no counterpart to compare with.)"""

import numpy as np
import pytest
from scipy import stats

from nengo_ocl_b200 import synth
from oracle import kernels as K
from oracle.simulator import OracleSimulator


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 as published with the generator (Random123's kat_vectors:
    zeros, ones, digits of pi)."""
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
        ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
        ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
         [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]),
    ]
    for counter, key, want in kat:
        got = K.philox4x32_10([np.array([c], dtype=np.uint32) for c in counter],
                              [np.array([k], dtype=np.uint32) for k in key])
        assert [int(g[0]) for g in got] == want


def test_samples_follow_their_distributions():
    u = K.whitenoise_samples(12345, 7, 200001, 0, (-1.0, 2.0), False, 0.001)
    assert u.dtype == np.float32 and u.min() >= -1.0 and u.max() < 2.0
    assert stats.kstest((u.astype(np.float64) + 1) / 3, "uniform").pvalue > 1e-3
    z = K.whitenoise_samples((7 << 32) | 99, 3, 400000, 1, (0.5, 2.0), False, 0.001)
    assert stats.kstest((z.astype(np.float64) - 0.5) / 2, "norm").pvalue > 1e-3
    assert abs(z.mean() - 0.5) < 0.02 and abs(z.std() - 2.0) < 0.02
    # consecutive steps and different seeds are uncorrelated; the same (seed, step) repeats
    a = K.whitenoise_samples(5, 10, 100000, 1, (0, 1), False, 0.001)
    b = K.whitenoise_samples(5, 11, 100000, 1, (0, 1), False, 0.001)
    c = K.whitenoise_samples(6, 10, 100000, 1, (0, 1), False, 0.001)
    assert abs(np.corrcoef(a, b)[0, 1]) < 0.02 and abs(np.corrcoef(a, c)[0, 1]) < 0.02
    assert np.array_equal(a, K.whitenoise_samples(5, 10, 100000, 1, (0, 1), False, 0.001))
    # a prefix of a longer vector is the shorter vector (element e depends on (seed, step, e) only)
    assert np.array_equal(a[:1001], K.whitenoise_samples(5, 10, 1001, 1, (0, 1), False, 0.001))
    # scale: 1/sqrt(dt), applied in double and rounded once
    s = K.whitenoise_samples(5, 10, 1000, 1, (0, 1), True, 0.001)
    assert np.array_equal(s, (a[:1000].astype(np.float64) / np.sqrt(0.001)).astype(np.float32))


def test_oracle_runs_a_noise_model():
    mdl = synth.white_noise_model(seed=21, n=300)
    ora = OracleSimulator(mdl)
    ora.run_steps(50)
    want = K.whitenoise_samples(mdl.info["seeds"][0], 50, 300, 1, (0.1, 0.5), True, 0.001)
    assert np.array_equal(ora[mdl.info["noise"]].reshape(-1), want)
    walk = np.array(ora.probe_data[mdl.probes[1]])
    assert walk.shape == (50, 7) and np.all(np.abs(np.diff(walk, axis=0)) <= 1.0)
