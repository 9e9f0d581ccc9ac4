"""Sparse transforms: host tables and heuristic against the reference's own
planners (golden fixtures), the oracle against the reference's CSR kernel run
on the CPU, and (GPU) the CUDA kernels against the oracle."""

import numpy as np
import pytest
import scipy.sparse as sp

from nengo_ocl_b200 import cura_spmv
from nengo_ocl_b200.raggedarray import RaggedArray as RA
from oracle import kernels as K

CASES = ["small", "empty_rows", "all_zero", "wide_row", "banded"]


def _matrix(golden_tables, tag):
    return sp.csr_matrix(golden_tables["sparse/%s/dense" % tag])


@pytest.mark.parametrize("tag", CASES)
def test_host_tables_match_the_reference(golden_tables, tag):
    hA = cura_spmv.HostSparseMatrix(_matrix(golden_tables, tag))
    ell = cura_spmv.plan_ellpack.scipy2elldata(hA)
    for name in ("columns", "entries", "rowlens"):
        want = golden_tables["sparse/%s/ell_%s" % (tag, name)]
        got = np.asarray(getattr(ell, name))
        assert got.dtype == want.dtype and np.array_equal(got, want), name
    assert [ell.ellwidth, ell.nnz] == list(golden_tables["sparse/%s/ell_width_nnz" % tag])
    csr = cura_spmv.plan_csr.scipy2csrdata(hA)
    for name in ("indices", "indptr", "data"):
        want = golden_tables["sparse/%s/csr_%s" % (tag, name)]
        got = np.asarray(getattr(csr, name))
        assert got.dtype == want.dtype and np.array_equal(got, want), name


def test_heuristic_matches_the_reference(golden_tables):
    class Device:
        global_mem_size = 0

    class Queue:
        device = Device()

    hA = cura_spmv.HostSparseMatrix(_matrix(golden_tables, "wide_row"))
    for mem, tag in ((10 ** 3, "hard"), (3 * 10 ** 4, "mid"), (10 ** 9, "soft")):
        Device.global_mem_size = mem
        assert cura_spmv.spmv_algorithm_heuristic(Queue(), hA) == str(golden_tables["sparse/heuristic_%s" % tag])
    assert set(cura_spmv.algostr_to_planner) == {"ELLPACK", "ELLPACK-tree", "ELLPACK-twostep", "CSR"}


@pytest.mark.parametrize("tag", CASES)
def test_oracle_matches_the_reference_csr_kernel(golden_tables, golden_kernels, tag):
    mat = _matrix(golden_tables, tag)
    x, y0 = golden_kernels["sparse/%s/x" % tag], golden_kernels["sparse/%s/y0" % tag]
    for inc in (False, True):
        want = golden_kernels["sparse/%s/y_%s" % (tag, "inc" if inc else "set")]
        got = K.spmv_csr(mat.indices, mat.indptr, mat.data, x, y0, inc=inc)
        assert np.array_equal(got.reshape(-1), want.reshape(-1))  # same operations in the same order
        ell = cura_spmv.plan_ellpack.scipy2elldata(cura_spmv.HostSparseMatrix(mat))
        got_ell = K.spmv_ell(ell.columns, ell.entries, x, y0, inc=inc)
        assert np.allclose(got_ell.reshape(-1), want.reshape(-1), rtol=1e-5, atol=1e-6)


def test_known_answer():
    A = sp.csr_matrix(np.array([[1.0, 0, 2.0], [0, 0, 0], [0, -3.0, 0.5]], dtype=np.float32))
    x = np.array([1.0, 2.0, 4.0], dtype=np.float32)
    y = np.array([10.0, 20.0, 30.0], dtype=np.float32)
    assert np.array_equal(K.spmv_csr(A.indices, A.indptr, A.data, x, y), [9.0, 0.0, -4.0])
    assert np.array_equal(K.spmv_csr(A.indices, A.indptr, A.data, x, y, inc=True), [19.0, 20.0, 26.0])


# ---- GPU -----------------------------------------------------------------------------
def _run(queue, mat, x, y0, algorithm, inc):
    from nengo_ocl_b200.curaggedarray import CUDARaggedArray

    # the operands sit at an offset inside their buffers, as signals do in the packed store
    clX = CUDARaggedArray(queue, RA([np.zeros((3, 1), np.float32), x.reshape(-1, 1)], dtype=np.float32))
    clY = CUDARaggedArray(queue, RA([np.ones((5, 1), np.float32), y0.reshape(-1, 1)], dtype=np.float32))
    prog = cura_spmv.plan_sparse_dot_inc(queue, cura_spmv.HostSparseMatrix(mat), clX[[1]], clY[[1]], inc=inc,
                                         algorithm=algorithm)
    for plan in prog.plans:
        plan()
    out = clY.to_host()
    assert np.array_equal(out[0], np.ones((5, 1), np.float32))  # the neighbour is untouched
    return out[1].reshape(-1), prog


@pytest.mark.gpu
@pytest.mark.parametrize("algorithm", ["CSR", "ELLPACK", "ELLPACK-tree", "ELLPACK-twostep", None])
@pytest.mark.parametrize("tag", CASES)
def test_kernels_match_oracle(queue, golden_tables, golden_kernels, tag, algorithm):
    mat = _matrix(golden_tables, tag)
    x, y0 = golden_kernels["sparse/%s/x" % tag].reshape(-1), golden_kernels["sparse/%s/y0" % tag].reshape(-1)
    for inc in (False, True):
        want = K.spmv_csr(mat.indices, mat.indptr, mat.data, x, y0, inc=inc)
        got, prog = _run(queue, mat, x, y0, algorithm, inc)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
        assert prog.plans[0].bw_per_call > 0 and prog.plans[0].flops_per_call == 2 * mat.nnz


@pytest.mark.gpu
@pytest.mark.parametrize("algorithm", ["CSR", "ELLPACK"])
def test_block_structured_matrix(queue, algorithm):
    """Neuron-to-neuron weights of a ring of ensembles: dense 50 x 50 blocks, 8 per block row."""
    rng = np.random.RandomState(5)
    n_ens, n = 40, 50
    blocks = [[None] * n_ens for _ in range(n_ens)]
    for i in range(n_ens):
        for o in (-4, -3, -2, -1, 1, 2, 3, 4):
            blocks[i][(i + o) % n_ens] = rng.normal(size=(n, n)).astype(np.float32)
    mat = sp.bmat(blocks, format="csr", dtype=np.float32)
    x = rng.normal(size=n_ens * n).astype(np.float32)
    y0 = rng.normal(size=n_ens * n).astype(np.float32)
    want = (mat.astype(np.float64) @ x.astype(np.float64))
    got, prog = _run(queue, mat, x, y0, algorithm, inc=False)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    got, _ = _run(queue, mat, x, y0, algorithm, inc=True)
    assert np.allclose(got, want + y0, rtol=1e-4, atol=1e-4)
