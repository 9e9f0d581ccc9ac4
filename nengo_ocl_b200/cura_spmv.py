"""Sparse matrix-vector plans: ``Y (+)= A . X`` for one sparse transform.

Same planning surface as the sparse part of the reference's GEMV module
(nengo_ocl/clra_gemv.py:1242-1997): ``HostSparseMatrix`` (utils.py:83-106),
``ell_matdata`` / ``csr_matdata``, ``spmv_prog`` and its subclasses
``plan_ellpack`` / ``plan_ellpack_tree`` / ``plan_ellpack_twostep`` /
``plan_csr``, ``spmv_algorithm_heuristic``, ``plan_sparse_dot_inc`` with the
``NENGO_OCL_SPMV_ALGORITHM`` environment override and ``algostr_to_planner``.
The host tables (``scipy2elldata``, ``scipy2csrdata``) are the reference's,
element for element; the device layout of a narrow ELLPACK matrix is
transposed (column-major) so that one thread per row reads contiguous lines,
and all variants are one launch without a scratch buffer
(csrc/nb2_spmv.cu).
"""

import os
from collections import namedtuple

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.plan import Plan
from nengo_ocl_b200.runtime import to_device

try:
    import scipy.sparse as scipy_sparse
except ImportError:  # pragma: no cover
    scipy_sparse = None

ell_matdata = namedtuple("ell_matdata", ["columns", "entries", "rowlens", "ellwidth", "nnz", "shape"])
csr_matdata = namedtuple("csr_matdata", ["indices", "indptr", "data", "nnz", "shape"])

ELL_COLUMN_MAJOR_WIDTH = 32  # widest matrix with few rows that is stored column-major on the device
ELL_COLUMN_MAJOR_ROWS = 4096  # from this many rows on, one thread per row fills the GPU at any width


class HostSparseMatrix:
    """A sparse matrix on the host with a cached CSR form (utils.py:83-106)."""

    def __init__(self, spmatrix):
        if scipy_sparse is None:
            raise NotImplementedError("Sparse matrices not supported without Scipy")
        if not isinstance(spmatrix, (np.ndarray, scipy_sparse.spmatrix)):
            raise NotImplementedError("Sparse matrices must be instances of `scipy.sparse.spmatrix`")
        self.matrix = spmatrix
        self.clear_cache()

    def clear_cache(self):
        self._csr = None

    @property
    def csr(self):
        if self._csr is None:
            self._csr = scipy_sparse.csr_matrix(self.matrix)
        return self._csr


class spmv_prog:
    """Formats the matrix, uploads it, validates the operands and makes the plans
    (clra_gemv.py:1249-1319)."""

    def __init__(self, queue, hA, X, Y, inc=False, tag=None):
        if not isinstance(hA, HostSparseMatrix):
            hA = HostSparseMatrix(hA)
        self.queue, self.hA, self.X, self.Y, self.inc, self.tag = queue, hA, X, Y, inc, tag
        self.hAstruct = None  # host tables
        self.dAstruct = None  # device twins
        self.to_hostdata()
        if queue is not None:
            self.to_device()
            self.validate_data()
            self.plans = self.choose_plans()
            self.assign_plan_characteristics(self.plans)
        else:  # host-only planning (tests of the tables)
            self.plans = []

    def assign_plan_characteristics(self, plans):
        pass

    def choose_plans(self):
        raise NotImplementedError("Subclass must implement")

    def to_device(self):
        raise NotImplementedError("Subclass must implement")

    def to_hostdata(self):
        raise NotImplementedError("Subclass must implement")

    def validate_data(self):
        assert len(self.X) == len(self.Y) == 1
        for arr in (self.X, self.Y):
            assert (np.asarray(arr.stride1s) == 1).all()
            if not ((np.asarray(arr.shape1s) == 1).all() and (np.asarray(arr.stride0s) == 1).all()):
                raise NotImplementedError("SparseDot only supports matrix-vector currently, not matrix-matrix.")
        shape = self.hAstruct.shape
        assert shape[0] == int(self.Y.shape0s[0]) and shape[1] == int(self.X.shape0s[0])
        assert self.X.dtype == self.Y.dtype == np.float32

    def _xy(self):
        import ctypes

        x = ctypes.c_void_p(self.X.cl_buf.data + 4 * int(self.X.starts[0]))
        y = ctypes.c_void_p(self.Y.cl_buf.data + 4 * int(self.Y.starts[0]))
        return x, y


class plan_ellpack(spmv_prog):
    """ELLPACK storage; the kernel variant follows the width (clra_gemv.py:1322-1408)."""

    @staticmethod
    def scipy2elldata(sparse_mat, force_nonempty=True):
        csrmat = sparse_mat.csr
        shape = csrmat.shape
        rowlens = np.diff(csrmat.indptr).astype(np.int32)
        assert rowlens.size == shape[0]
        ellwidth = int(rowlens.max()) if rowlens.size else 0
        make_nonempty = force_nonempty and ellwidth == 0
        matwidth = 1 if make_nonempty else ellwidth
        columns = np.zeros((shape[0], matwidth), dtype=np.int32)
        entries = np.zeros((shape[0], matwidth), dtype=np.float32)
        nnz = csrmat.nnz
        assert rowlens.sum() == nnz
        # row r takes its run of the CSR arrays: vectorised form of the per-row copy
        if nnz:
            rows = np.repeat(np.arange(shape[0]), rowlens)
            pos = np.arange(nnz) - np.repeat(csrmat.indptr[:-1], rowlens)
            columns[rows, pos] = csrmat.indices
            entries[rows, pos] = csrmat.data
        if make_nonempty:
            rowlens[0] = 1
        return ell_matdata(columns, entries, rowlens, ellwidth, nnz, shape)

    @property
    def subplanner(self):
        return (plan_ellpack_twostep if self.dAstruct.ellwidth > self.queue.device.max_work_group_size
                else plan_ellpack_tree)

    def to_hostdata(self):
        self.hAstruct = plan_ellpack.scipy2elldata(self.hA)

    def to_device(self):
        h = self.hAstruct
        self.row_major = h.columns.shape[1] > ELL_COLUMN_MAJOR_WIDTH and h.shape[0] < ELL_COLUMN_MAJOR_ROWS
        lay = (lambda a: np.ascontiguousarray(a)) if self.row_major else (lambda a: np.ascontiguousarray(a.T))
        self.dAstruct = ell_matdata(to_device(self.queue, lay(h.columns)), to_device(self.queue, lay(h.entries)),
                                    to_device(self.queue, h.rowlens), h.ellwidth, h.nnz, h.shape)

    def validate_data(self):
        super().validate_data()
        h = self.hAstruct
        assert h.columns.shape == h.entries.shape and h.columns.shape[0] == int(self.Y.shape0s[0])
        assert h.columns.dtype == np.int32 and h.entries.dtype == np.float32

    def _impl(self, name):
        d, h = self.dAstruct, self.hAstruct
        x, y = self._xy()
        n_rows, width = int(h.shape[0]), int(h.columns.shape[1])
        fn, check = _capi.lib().nb2_spmv_ell, _capi.check
        args = (d.columns.ptr, d.entries.ptr, d.rowlens.ptr, n_rows, width, int(self.row_major), x, y, int(self.inc))

        def launch(stream):
            check(fn(stream, *args))

        plan = Plan(self.queue, launch, (n_rows * (32 if self.row_major else 1), 1), lsize=None, name=name,
                    tag=self.tag)
        plan.full_args = (d.columns, d.entries, d.rowlens, self.X.cl_buf, self.Y.cl_buf)
        return plan

    def choose_plans(self):
        return self.subplanner.choose_plans(self)

    def assign_plan_characteristics(self, plans):
        return self.subplanner.assign_plan_characteristics(self, plans)

    def _characteristics(self, plans, groups):
        h = self.hAstruct
        plan = plans[0]
        plan.flops_per_call = 2 * h.nnz
        plan.bw_per_call = (8 * h.nnz + h.rowlens.nbytes + self.X.nbytes + self.Y.nbytes)
        plan.description = "groups: %d; shape: (%d, %d); nonzeros: %d; width: %d" % (
            groups, h.shape[0], h.shape[1], h.nnz, h.ellwidth)


class plan_ellpack_tree(plan_ellpack):
    """Counterpart of the work-group-per-row tree reduction (clra_gemv.py:1411-1443)."""

    def choose_plans(self):
        return [plan_ellpack._impl(self, "cura_sparsedot_ellpack")]

    def assign_plan_characteristics(self, plans):
        plan_ellpack._characteristics(self, plans, int(self.hAstruct.shape[0]))


class plan_ellpack_twostep(plan_ellpack):
    """Counterpart of the two-kernel variant for very wide rows (clra_gemv.py:1446-1491):
    here the same single launch, one warp per row."""

    def choose_plans(self):
        return [plan_ellpack._impl(self, "cura_sparsedot_ellpack_wide")]

    def assign_plan_characteristics(self, plans):
        plan_ellpack._characteristics(self, plans, int(self.hAstruct.shape[0]))


class plan_csr(spmv_prog):
    """Compressed sparse rows (clra_gemv.py:1494-1567)."""

    @staticmethod
    def scipy2csrdata(sparse_mat, force_nonempty=True):
        scipy_csr = sparse_mat.csr
        return csr_matdata(np.asarray(scipy_csr.indices, dtype=np.int32), np.asarray(scipy_csr.indptr, dtype=np.int32),
                           np.asarray(scipy_csr.data, dtype=np.float32), scipy_csr.nnz, scipy_csr.shape)

    def to_hostdata(self):
        self.hAstruct = plan_csr.scipy2csrdata(self.hA)

    def to_device(self):
        h = self.hAstruct
        pad = lambda a: a if a.size else np.zeros(1, a.dtype)
        self.dAstruct = csr_matdata(to_device(self.queue, pad(h.indices)), to_device(self.queue, h.indptr),
                                    to_device(self.queue, pad(h.data)), h.nnz, h.shape)

    def validate_data(self):
        super().validate_data()
        h = self.hAstruct
        assert h.indices.ndim == h.indptr.ndim == h.data.ndim == 1 and h.indices.size == h.data.size
        assert h.indices.dtype == h.indptr.dtype == np.int32 and h.data.dtype == np.float32

    @staticmethod
    def lanes_log2(nnz, n_rows):
        """Lanes that share a row: about 8 nonzeros per lane, so that a warp works on several
        rows at once and every lane has several independent loads in flight (at most 32 lanes)."""
        mean = nnz / max(n_rows, 1)
        return int(np.clip(np.floor(np.log2(max(mean / 8.0, 1.0))), 0, 5))

    def choose_plans(self):
        d, h = self.dAstruct, self.hAstruct
        x, y = self._xy()
        n_rows = int(h.shape[0])
        logg = self.lanes_log2(h.nnz, n_rows)
        fn, check = _capi.lib().nb2_spmv_csr, _capi.check
        args = (d.indices.ptr, d.indptr.ptr, d.data.ptr, n_rows, logg, x, y, int(self.inc))

        def launch(stream):
            check(fn(stream, *args))

        plan = Plan(self.queue, launch, (n_rows << logg, 1), lsize=None, name="cura_sparsedot", tag=self.tag)
        plan.full_args = (d.indices, d.indptr, d.data, self.X.cl_buf, self.Y.cl_buf)
        return [plan]

    def assign_plan_characteristics(self, plans):
        h = self.hAstruct
        plan = plans[0]
        plan.flops_per_call = 2 * h.data.size
        plan.bw_per_call = h.data.nbytes + h.indices.nbytes + h.indptr.nbytes + self.X.nbytes + self.Y.nbytes
        plan.description = "groups: %d; shape: (%d, %d); nonzeros: %d" % (1, h.shape[0], h.shape[1], h.nnz)


def spmv_algorithm_heuristic(queue, hA, footprint_hard_limit=0.8, footprint_soft_limit=0.05, soft_limit_ratio=0.1):
    """CSR or ELLPACK by memory footprint (clra_gemv.py:1951-1989): ELLPACK unless
    its padded arrays would take too much of the device memory."""
    csr = hA.csr
    ellwidth = max(np.diff(csr.indptr))
    ell_bytes = 2 * 4 * ellwidth * csr.shape[1]
    csr_bytes = 2 * 4 * csr.nnz
    ell_device_ratio = ell_bytes / queue.device.global_mem_size
    if ell_device_ratio > footprint_hard_limit:
        return "CSR"
    elif ell_device_ratio < footprint_soft_limit:
        return "ELLPACK"
    else:
        return "CSR" if csr_bytes / ell_bytes < soft_limit_ratio else "ELLPACK"


#: Map of strings to planners
algostr_to_planner = {
    "ELLPACK": plan_ellpack,
    "ELLPACK-tree": plan_ellpack_tree,
    "ELLPACK-twostep": plan_ellpack_twostep,
    "CSR": plan_csr,
}


def plan_sparse_dot_inc(queue, hA, X, Y, inc=False, tag=None, algorithm=None):
    """Planner for ``Y (+)= hA . X`` (clra_gemv.py:1919-1948): the algorithm comes
    from the argument, else from ``NENGO_OCL_SPMV_ALGORITHM``, else from the
    footprint heuristic."""
    assert isinstance(hA, HostSparseMatrix)
    if algorithm is None:
        algorithm = os.environ.get("NENGO_OCL_SPMV_ALGORITHM", None)
    if algorithm is None:
        algorithm = spmv_algorithm_heuristic(queue, hA)
    planner_type = algostr_to_planner[algorithm]
    return planner_type(queue, hA, X, Y, inc=inc, tag=tag)
