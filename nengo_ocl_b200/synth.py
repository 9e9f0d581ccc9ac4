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
