"""Ragged gather-GEMV plans: ``Y = gamma + beta * Y_in + alpha * sum_j A_j X_j``.

Planner surface of the reference's ``nengo_ocl/clra_gemv.py`` (``gemv_prog``
:100-261 and the ``plan_*_gemv`` classes :1178-1239): same constructor
arguments, ``.plans``, ``.geometry``, ``cl_geometry_and_textconf``,
``geometry_summary``, ``flops_from_geometry`` / ``bw_from_geometry`` and the
same ``NotImplementedError`` conventions.  Every planner ends in the same
single-pass CUDA kernel family (csrc/nb2_gemv.cu); what differs between them
is the item selection and the launch geometry they report, which follow the
reference so that plan listings stay comparable.  The integer index tables
(per-item ``gstructure`` and the 32x128 tile tables of ``block_impl``) are
built bit-identically to the reference and kept on the plan objects.
"""

from collections import defaultdict

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.curaggedarray import CUDARaggedArray, to_device
from nengo_ocl_b200.plan import Plan
from nengo_ocl_b200.runtime import zeros

# default staging variant of the CTA kernel (can be overridden per planner call)
DEFAULT_CTA_KIND = 3  # GEMV_PIPE


def float_cl_clra(queue, arg, cl_dtype, N):
    """Classify a scale argument: python float, per-item device vector, or ragged.

    Same three-way split as the reference (clra_gemv.py:17-32).
    """
    if isinstance(arg, CUDARaggedArray):
        assert arg.dtype == cl_dtype
        return None, None, arg
    if isinstance(arg, (float, int, np.floating, np.integer)):
        return float(arg), None, None
    if len(set(arg)) == 1:
        return float(arg[0]), None, None
    host = np.asarray(arg, cl_dtype)
    assert host.shape == (N,)
    return None, to_device(queue, host), None


def flops_from_geometry(geometry, items):
    """2 flops per A element plus 3 per output row (clra_gemv.py:35-46)."""
    total = 0
    for ii in items:
        gi = geometry[ii]
        total += sum(int(d["a_shape1"]) for d in gi["dots"]) * int(gi["y_len"]) * 2
        total += int(gi["y_len"]) * 3
    return total


def bw_from_geometry(geometry, items):
    """Algorithmic bytes of one call (clra_gemv.py:49-70): A and X of every
    term, two scalars, Y_in read and Y write."""
    total = 0
    for ii in items:
        gi = geometry[ii]
        y_len = int(gi["y_len"])
        for d in gi["dots"]:
            n = int(d["a_shape1"])
            total += 4 * (n * y_len + n)
        total += 8 + 8 * y_len
    return total


class DotSignature:
    def __init__(self, dct):
        self.y_len = dct["y_len"]
        self.Ax_dims = tuple((d["a_shape1"], d["a_stride0"]) for d in dct["dots"])

    def __eq__(self, other):
        return type(self) == type(other) and (self.y_len, self.Ax_dims) == (other.y_len, other.Ax_dims)

    def __hash__(self):
        return hash((self.y_len, self.Ax_dims))

    def __lt__(self, other):
        return (self.y_len, self.Ax_dims) < (other.y_len, other.Ax_dims)

    def __str__(self):
        counts = defaultdict(int)
        for dim_stride in self.Ax_dims:
            counts[dim_stride] += 1
        body = ", ".join("(%s x d=%s,s=%s)" % (c, d, s) for (d, s), c in counts.items())
        return "yd=%s <- %s" % (self.y_len, body)


def build_worklist(gstructure, D):
    """Split items into equal-bytes work units for the CUDA kernels.

    Returns ``(cta_units, warp_units)``, int32 arrays of shape (n, 4) holding
    {row of ``gstructure``, first output row, row count, 0}.  Tiny items
    (<= 32 rows and <= 1024 matrix elements) go to the warp kernel; everything
    else is cut into row ranges whose staged A rows fill about one shared-memory
    buffer (``GEMV_ABUF`` floats) so a 65,000x spread in item size does not
    turn into load imbalance.
    """
    n_items = gstructure.shape[0]
    if n_items == 0:
        empty = np.zeros((0, 4), dtype=np.int32)
        return empty, empty
    n_dots = gstructure[:, 4 * D + 2].astype(np.int64)
    M = gstructure[:, 4 * D + 3].astype(np.int64)
    if D > 0:
        Ns = gstructure[:, 3 * D : 4 * D].astype(np.int64)
        mask = np.arange(D)[None, :] < n_dots[:, None]
        row_floats = (Ns * mask).sum(axis=1)
    else:
        row_floats = np.zeros(n_items, dtype=np.int64)

    small = (M <= 32) & (M * row_floats <= 1024)
    rows = np.arange(n_items)

    warp_rows = rows[small & (M > 0)]
    warp_units = np.zeros((len(warp_rows), 4), dtype=np.int32)
    warp_units[:, 0] = warp_rows
    warp_units[:, 2] = M[warp_rows]

    big = rows[~small & (M > 0)]
    if len(big) == 0:
        return np.zeros((0, 4), dtype=np.int32), warp_units
    Mb = M[big]
    budget = _capi.GEMV_ABUF - 4 * np.maximum(n_dots[big], 1) - 4
    R = budget // np.maximum(row_floats[big], 1)
    R = np.maximum(R, np.minimum(Mb, 8))  # keep all warps busy on long rows
    R = np.clip(R, 1, _capi.GEMV_RMAX)
    R = np.minimum(R, Mb)
    n_units = -(-Mb // R)
    R = -(-Mb // n_units)  # even out the row ranges
    item_of_unit = np.repeat(big, n_units)
    first_unit = np.cumsum(n_units) - n_units
    local = np.arange(int(n_units.sum())) - np.repeat(first_unit, n_units)
    r0 = local * np.repeat(R, n_units)
    cnt = np.minimum(np.repeat(R, n_units), np.repeat(Mb, n_units) - r0)
    cta_units = np.zeros((len(item_of_unit), 4), dtype=np.int32)
    cta_units[:, 0] = item_of_unit
    cta_units[:, 1] = r0
    cta_units[:, 2] = cnt
    return cta_units, warp_units


GEMV_ROWS = 4  # row-group kernel, direct global loads (csrc/nb2_gemv.cu)
ROWS_PER_THREAD = 8


def build_rows_worklist(gstructure, D):
    """Units for the row-group kernel: {item row, first row, rows, log2 G}.

    G lanes per row = next power of two >= the widest term (at most 32), so a
    warp's loads cover contiguous row chunks; a unit spans 8 * (256 / G) rows.
    Tiny items still go to the warp kernel."""
    n_items = gstructure.shape[0]
    empty = np.zeros((0, 4), dtype=np.int32)
    if n_items == 0:
        return empty, empty
    n_dots = gstructure[:, 4 * D + 2].astype(np.int64)
    M = gstructure[:, 4 * D + 3].astype(np.int64)
    if D > 0:
        Ns = gstructure[:, 3 * D:4 * D].astype(np.int64)
        mask = np.arange(D)[None, :] < n_dots[:, None]
        row_floats = (Ns * mask).sum(axis=1)
        wmax = np.maximum((Ns * mask).max(axis=1), 1)
    else:
        row_floats = np.zeros(n_items, dtype=np.int64)
        wmax = np.ones(n_items, dtype=np.int64)
    small = (M <= 32) & (M * row_floats <= 1024) & (n_dots <= 64)
    rows = np.arange(n_items)
    warp_rows = rows[small & (M > 0)]
    warp_units = np.zeros((len(warp_rows), 4), dtype=np.int32)
    warp_units[:, 0] = warp_rows
    warp_units[:, 2] = M[warp_rows]
    big = rows[~small & (M > 0)]
    if len(big) == 0:
        return empty, warp_units
    logG = np.minimum(np.ceil(np.log2(wmax[big])).astype(np.int64), 5)
    Mb = M[big]
    # few rows: widen G so that the threads of the CTA are not left idle
    logG = np.maximum(logG, np.minimum(5, np.floor(np.log2(np.maximum(256 * ROWS_PER_THREAD // np.maximum(Mb, 1), 1)))
                                       .astype(np.int64) - 3))
    logG = np.clip(logG, 0, 5)
    R = ROWS_PER_THREAD * (256 >> logG)
    n_units = -(-Mb // R)
    Re = -(-Mb // n_units)
    item_of_unit = np.repeat(big, n_units)
    first_unit = np.cumsum(n_units) - n_units
    local = np.arange(int(n_units.sum())) - np.repeat(first_unit, n_units)
    r0 = local * np.repeat(Re, n_units)
    cnt = np.minimum(np.repeat(Re, n_units), np.repeat(Mb, n_units) - r0)
    units = np.zeros((len(item_of_unit), 4), dtype=np.int32)
    units[:, 0] = item_of_unit
    units[:, 1] = r0
    units[:, 2] = cnt
    units[:, 3] = np.repeat(logG, n_units)
    return units, warp_units


# geometry of the pipelined kernel: the same numbers the library was compiled with (include/nengo_b200.h)
_PIPE = _capi.header_constants("NB2_PIPE_")
PIPE_STAGE_FLOATS = _PIPE["NB2_PIPE_STAGE_FLOATS"]
PIPE_CONSUMER_WARPS = _PIPE["NB2_PIPE_WARPS"]  # warps per CTA, one stage each
PIPE_WARPS_PER_RECORD = 1
PIPE_CTAS_PER_SM = _PIPE["NB2_PIPE_CTAS_PER_SM"]
PIPE_RMAX = 128 * PIPE_WARPS_PER_RECORD
PIPE_MAXSEG, PIPE_REC = 4, 32
GEMV_PIPE = 3  # persistent producer/consumer kernel (csrc/nb2_gemv_pipe.cu)
PIPE_MIN_CHUNK = 128  # narrowest column chunk worth a record of its own (single-row records)


def _pipe_window(n):
    """Pool floats reserved for a staged copy of ``n`` floats: the copy is the
    enclosing 16-byte-aligned window of its source (<= 3 floats before, <= 3
    after), and windows start on 16-byte boundaries of the pool."""
    return (n + 6 + 3) & ~3


def _pipe_cost(R, w, staged_x):
    return _pipe_window(R * w) + (_pipe_window(w) if staged_x else 0)


def _pipe_template(R, terms):
    """Pack the terms of one row range of ``R`` rows into records.

    ``terms`` = [(N, staged_x)]; returns a list of records, each a list of
    (term index, c0, w, a_base, x_base) with 4-aligned pool offsets, or None
    if a whole row of some term does not fit an empty stage (whole rows are
    required when R > 1 so that every staged copy is one contiguous range;
    single-row records may cut a row into column chunks)."""
    C = PIPE_STAGE_FLOATS
    records, cur, used = [], [], 0
    for ti, (N, xs) in enumerate(terms):
        c0 = 0
        w_chunk = None
        while c0 < N:
            rem = N - c0
            if len(cur) < PIPE_MAXSEG and used + _pipe_cost(R, rem, xs) <= C:
                w = rem
            elif R == 1 and len(cur) < PIPE_MAXSEG and used + _pipe_cost(1, min(rem, PIPE_MIN_CHUNK), xs) <= C:
                wmax = ((C - used - 20) // (2 if xs else 1)) & ~3
                if w_chunk is None:  # equal chunks rather than one full stage and a sliver
                    n_chunks = -(-rem // max(wmax, 1))
                    w_chunk = (-(-rem // n_chunks) + 3) & ~3
                w = min(rem, wmax, w_chunk)
            elif cur:
                records.append(cur)
                cur, used = [], 0
                continue
            else:
                return None
            a_base = used
            x_base = used + _pipe_window(R * w)
            cur.append((ti, c0, w, a_base, x_base))
            used += _pipe_cost(R, w, xs)
            c0 += w
    records.append(cur)
    return records


def _pipe_rows(m, Ns, staged):
    """Rows per record for an item of ``m`` rows whose rows are contiguous."""
    C = PIPE_STAGE_FLOATS

    def largest(group):
        n = sum(Ns[t] for t in group)
        x = sum(_pipe_window(Ns[t]) for t in group if staged[t])
        R = (C - x - 9 * len(group)) // max(n, 1)
        while R > 0 and sum(_pipe_cost(R, Ns[t], staged[t]) for t in group) > C:
            R -= 1
        return R

    nd = len(Ns)
    groups = [range(t, min(t + PIPE_MAXSEG, nd)) for t in range(0, nd, PIPE_MAXSEG)]
    R = min(largest(g) for g in groups)
    if R < 1:  # not even one row of a full group: one term per segment, as many rows as fit
        R = min(largest([t]) for t in range(nd))
    R = max(0, min(R, PIPE_RMAX, m))
    lanes = 32 * PIPE_WARPS_PER_RECORD  # one lane per row: whole multiples keep every lane busy
    if R >= lanes:
        R = R // lanes * lanes
        n_units = -(-m // R)
        even = -(-(-(-m // n_units)) // lanes) * lanes  # even out the row ranges, still whole multiples
        R = min(R, even)
    return R


def build_pipe_records(gstructure, xstrides, D, n_ctas_max):
    """Work records and per-CTA record ranges for ``nb2_gemv_pipelined``.

    Record layout (32 int32): [0] flags (1 = first of its chain, 2 = last),
    [1] rows, [2] Y_in element index of the first row, [3] Y element index,
    [4] item id, [5] segment count, [6] 0, [7] bytes of the staged Y_in window
    (0 = none), then per segment 6 ints at 8 + 6q:
    A element index of the staged window (multiple of 4), its bytes, X element
    index of the staged window (or of the first column when X is read from
    global memory), its bytes (or minus the X stride), columns,
    (x offset << 16 | a offset) of the first payload element in the stage pool.
    Returns ``(records, ranges, warp_units, fallback_rows)``; tiny items with very
    many terms go to the warp kernel, items whose rows are not contiguous and too
    narrow for single-row records to the CTA kernel.
    """
    n_items = gstructure.shape[0]
    n_dots = gstructure[:, 4 * D + 2].astype(np.int64) if n_items else np.zeros(0, np.int64)
    M = gstructure[:, 4 * D + 3].astype(np.int64) if n_items else np.zeros(0, np.int64)
    recs = []
    chain_start = []  # record index where each chain starts
    warp_rows, fallback_rows = [], []
    for row in range(n_items):
        m, nd = int(M[row]), int(n_dots[row])
        if m == 0:
            continue
        g = gstructure[row]
        Ns = [int(v) for v in g[3 * D:3 * D + nd]]
        row_floats = sum(Ns)
        s0s = [int(v) for v in g[2 * D:2 * D + nd]]
        astarts = [int(v) for v in g[1 * D:1 * D + nd]]
        xstarts = [int(v) for v in g[0:nd]]
        xstr = [int(v) for v in xstrides[row, :nd]] if nd else []
        if nd > 4 * PIPE_MAXSEG and m <= 32 and m * row_floats <= 1024 and nd <= 64:
            warp_rows.append(row)  # a long chain of tiny segments: one warp walks the terms directly
            continue
        if any(s < 0 for s in xstr):
            fallback_rows.append(row)
            continue
        staged = [s == 1 for s in xstr]
        contiguous = all(s0 == N for s0, N in zip(s0s, Ns))
        if contiguous or nd == 0:
            R = _pipe_rows(m, Ns, staged) if nd else min(m, PIPE_RMAX)
            R = max(R, 1)
        elif min(Ns) >= PIPE_MIN_CHUNK:
            R = 1
        else:
            fallback_rows.append(row)
            continue
        template = _pipe_template(R, list(zip(Ns, staged)))
        if template is None:
            R = 1
            template = _pipe_template(R, list(zip(Ns, staged)))
        n_units = -(-m // R)
        y_in0, y0, bb = int(g[4 * D + 0]), int(g[4 * D + 1]), int(g[4 * D + 4])
        n_rec = len(template)
        block = np.zeros((n_units, n_rec, PIPE_REC), dtype=np.int64)
        r0 = np.arange(n_units, dtype=np.int64) * R
        rows_u = np.minimum(R, m - r0)
        for k, segs in enumerate(template):
            last = k == n_rec - 1
            block[:, k, 0] = (1 if k == 0 else 0) | (2 if last else 0)
            block[:, k, 1] = rows_u
            block[:, k, 2] = y_in0 + r0
            block[:, k, 3] = y0 + r0
            block[:, k, 4] = bb
            block[:, k, 5] = len(segs)
            if last:
                yi = y_in0 + r0
                block[:, k, 7] = 4 * ((((yi & 3) + rows_u + 3) & ~3))
            for q, (ti, c0, w, a_base, x_base) in enumerate(segs):
                gidx = astarts[ti] + r0 * s0s[ti] + c0
                n_a = (rows_u - 1) * w + w if s0s[ti] == Ns[ti] and w == Ns[ti] else w  # R == 1 otherwise
                o = 8 + 6 * q
                block[:, k, o + 0] = gidx & ~3
                block[:, k, o + 1] = 4 * (((gidx & 3) + n_a + 3) & ~3)
                xs = xstarts[ti] + c0 * xstr[ti]
                if staged[ti]:
                    block[:, k, o + 2] = xs & ~3
                    block[:, k, o + 3] = 4 * (((xs & 3) + w + 3) & ~3)
                    xoff = x_base + (xs & 3)
                else:
                    block[:, k, o + 2] = xs
                    block[:, k, o + 3] = -xstr[ti]
                    xoff = 0
                block[:, k, o + 4] = w
                block[:, k, o + 5] = (xoff << 16) | (a_base + (gidx & 3))
        base_index = sum(b.shape[0] for b in recs)
        flat = block.reshape(n_units * n_rec, PIPE_REC)
        chain_start.extend((base_index + np.arange(n_units) * n_rec).tolist())
        recs.append(flat)
    warp_units = np.zeros((len(warp_rows), 4), dtype=np.int32)
    if warp_rows:
        warp_units[:, 0] = warp_rows
        warp_units[:, 2] = M[warp_rows]
    fallback_rows = np.asarray(fallback_rows, dtype=np.int64)
    if not recs:
        return np.zeros((0, PIPE_REC), np.int32), np.zeros((0, 2), np.int32), warp_units, fallback_rows
    records = np.concatenate(recs, axis=0)
    assert records.max() < 2 ** 31 and records.min() >= -2 ** 31
    records = records.astype(np.int32)
    # cost of a record = staged bytes / 4 + a fixed overhead; chains are never split
    nseg = records[:, 5].astype(np.int64)
    cost = np.full(len(records), 256, dtype=np.int64)
    for q in range(PIPE_MAXSEG):
        cost += np.where(q < nseg, records[:, 8 + 6 * q + 1].astype(np.int64) // 4, 0)
    chain_start = np.asarray(chain_start, dtype=np.int64)
    chain_len = np.diff(np.concatenate([chain_start, [len(records)]]))
    csum = np.concatenate([[0], np.cumsum(cost)])
    chain_cost_end = csum[chain_start + chain_len]
    n_ctas = int(min(len(chain_start), n_ctas_max))
    targets = csum[-1] * np.arange(1, n_ctas) / n_ctas
    cut = np.unique(np.concatenate([[0], np.searchsorted(chain_cost_end, targets, side="left") + 1,
                                    [len(chain_start)]]))
    cut = cut[cut <= len(chain_start)]
    # Within a CTA, record i is consumed by warp group i % NW: deal the CTA's chains to the
    # groups round-robin and interleave the per-group sequences (padding with empty records).
    NW = PIPE_CONSUMER_WARPS // PIPE_WARPS_PER_RECORD
    out_blocks, ranges, pos = [], [], 0
    for c0, c1 in zip(cut[:-1], cut[1:]):
        lens = chain_len[c0:c1]
        first, last = chain_start[c0], chain_start[c1 - 1] + chain_len[c1 - 1]
        if (lens == 1).all():
            block = records[first:last]
        else:
            seqs = [[] for _ in range(NW)]
            for j in range(c1 - c0):
                st = chain_start[c0 + j]
                seqs[j % NW].extend(range(st, st + lens[j]))
            depth = max(len(q) for q in seqs)
            block = np.zeros((depth * NW, PIPE_REC), dtype=np.int32)
            for w, q in enumerate(seqs):
                block[w:len(q) * NW:NW] = records[q]
        out_blocks.append(block)
        ranges.append((pos, pos + len(block)))
        pos += len(block)
    records = np.concatenate(out_blocks, axis=0)
    return records, np.asarray(ranges, dtype=np.int32), warp_units, fallback_rows


class gemv_prog:
    """Base planner: classify scales, compute geometry, choose plans."""

    def __init__(self, queue, alpha, A, A_js, X, X_js, beta, Y, Y_in=None, gamma=0.0, tag=None,
                 cta_kind=None):
        self.float_alpha, self.cl_alpha, self.clra_alpha = float_cl_clra(queue, alpha, Y.dtype, len(Y))
        self.float_beta, self.cl_beta, self.clra_beta = float_cl_clra(queue, beta, Y.dtype, len(Y))
        self.float_gamma, self.cl_gamma, self.clra_gamma = float_cl_clra(queue, gamma, Y.dtype, len(Y))
        self.Y_in = Y if Y_in is None else Y_in
        self.queue = queue
        self.A = A
        self.A_js = A_js
        self.X = X
        self.X_js = X_js
        self.Y = Y
        self.tag = str(tag)
        self.cta_kind = DEFAULT_CTA_KIND if cta_kind is None else cta_kind
        self.geometry = self._geometry()
        self.plans = self.choose_plans()

    # ---- geometry ---------------------------------------------------------
    def _term_indices(self, bb):
        """(x_js, a_js) index lists of output ``bb`` as python ints."""
        if not self.X_js:
            return [], []
        xs = np.asarray(self.X_js[bb]).ravel()
        as_ = np.asarray(self.A_js[bb]).ravel()
        assert len(xs) == len(as_)
        return [int(v) for v in xs], [int(v) for v in as_]

    def _geometry(self):
        A, X, Y, Y_in = self.A, self.X, self.Y, self.Y_in
        out = []
        for bb in range(len(Y)):
            xs, as_ = self._term_indices(bb)
            dots = [
                {
                    "j": jj,
                    "x_j": xj,
                    "a_j": aj,
                    "x_start": X.starts[xj],
                    "a_start": A.starts[aj],
                    "a_stride0": A.stride0s[aj],
                    "a_shape1": A.shape1s[aj],
                }
                for jj, (xj, aj) in enumerate(zip(xs, as_))
            ]
            out.append({"y_len": Y.shape0s[bb], "dots": dots, "y_start": Y.starts[bb],
                        "y_in_start": Y_in.starts[bb]})
        return out

    def geometry_summary(self, items=None):
        gg = self.geometry if items is None else [self.geometry[i] for i in items]
        dots = np.array([len(g["dots"]) for g in gg])
        shape0s = np.array([g["y_len"] for g in gg])
        shape1s = np.hstack([[d["a_shape1"] for d in g["dots"]] for g in gg] or [[0]])
        if shape1s.size == 0:
            shape1s = np.zeros(1)
        return "outputs: %d; dots: %0.1f [%d, %d]; shape: %0.1f [%d, %d] x %0.1f [%d, %d]" % (
            len(gg), dots.mean(), dots.min(), dots.max(), shape0s.mean(), shape0s.min(), shape0s.max(),
            shape1s.mean(), shape1s.min(), shape1s.max())

    def print_geometry_summary(self, items=None, full=False):
        print("geometry_summary: tag=%s" % self.tag)
        gg = self.geometry if items is None else [self.geometry[i] for i in items]
        counts = defaultdict(int)
        for g in gg:
            counts[DotSignature(g)] += 1
        for sig in sorted(counts):
            print("  %6s\t%s" % (counts[sig], sig))

    def gstructure_table(self, items, padding=4):
        """Host int32 table for ``items`` in the reference's layout
        (clra_gemv.py:211-246) plus the X-stride side table."""
        items = list(items)
        geo = self.geometry
        D = max([len(geo[ii]["dots"]) for ii in items] + [0])
        n_vars = 4 * D + 5
        stride = int(padding * np.ceil(float(n_vars) / padding))
        table = np.zeros((len(items), stride), dtype=np.int32)
        xstrides = np.ones((len(items), max(D, 1)), dtype=np.int32)
        X_stride0s = self.X.stride0s
        for row, bb in enumerate(items):
            g = geo[bb]
            for ii, d in enumerate(g["dots"]):
                table[row, 0 * D + ii] = d["x_start"]
                table[row, 1 * D + ii] = d["a_start"]
                table[row, 2 * D + ii] = d["a_stride0"]
                table[row, 3 * D + ii] = d["a_shape1"]
                xstrides[row, ii] = X_stride0s[d["x_j"]]
            table[row, 4 * D + 0] = g["y_in_start"]
            table[row, 4 * D + 1] = g["y_start"]
            table[row, 4 * D + 2] = len(g["dots"])
            table[row, 4 * D + 3] = g["y_len"]
            table[row, 4 * D + 4] = bb
        return table, xstrides, D, n_vars, stride

    def cl_geometry_and_textconf(self, items, padding=4):
        table, _, D, n_vars, stride = self.gstructure_table(items, padding)
        textconf = {
            "n_structure_vars": n_vars,
            "structure_vars_stride": stride,
            "x_starts": "lstructure[0 * %s + ii]" % D,
            "a_starts": "lstructure[1 * %s + ii]" % D,
            "a_s0": "lstructure[2 * %s + ii]" % D,
            "N_i": "lstructure[3 * %s + ii]" % D,
            "y_in_starts": "lstructure[4 * %s + 0]" % D,
            "y_offset": "lstructure[4 * %s + 1]" % D,
            "n_dot_products": "lstructure[4 * %s + 2]" % D,
            "y_len": "lstructure[4 * %s + 3]" % D,
            "bb": "lstructure[4 * %s + 4]" % D,
        }
        return to_device(self.queue, table), textconf

    # ---- device plan ------------------------------------------------------
    def _check_supported(self, per_item_scales):
        """Raise NotImplementedError for layouts the kernels do not take."""
        if self.clra_alpha is not None or self.clra_gamma is not None or self.clra_beta is not None:
            raise NotImplementedError("per-row ragged alpha/beta/gamma")
        if not per_item_scales and (self.cl_alpha is not None or self.cl_gamma is not None):
            raise NotImplementedError("per-item alpha/gamma vectors")
        if not all(s == 1 for s in self.A.stride1s):
            raise NotImplementedError("A.stride1 != 1")
        for arr in (self.Y, self.Y_in):
            if not (all(s == 1 for s in arr.stride0s) and all(s == 1 for s in arr.shape1s)):
                raise NotImplementedError("Y must be a list of contiguous vectors")

    def _device_plan(self, items, name, gsize, lsize, per_item_scales=True):
        items = list(items)
        self._check_supported(per_item_scales)
        table, xstrides, D, _, stride = self.gstructure_table(items)
        queue = self.queue
        cta_kind = self.cta_kind
        if cta_kind == GEMV_PIPE:
            n_ctas_max = PIPE_CTAS_PER_SM * getattr(queue.device, "sm_count", 148)
            records, ranges, warp_units, fallback = build_pipe_records(table, xstrides, D, n_ctas_max)
            cta_units = np.zeros((0, 4), dtype=np.int32)
            if len(fallback):  # layouts the bulk copies cannot stage: the plain CTA kernel takes them
                cta_kind = _capi.GEMV_CTA
                cta_all, warp_all = build_worklist(table, D)
                cta_units = cta_all[np.isin(cta_all[:, 0], fallback)]
                warp_units = np.concatenate([warp_units, warp_all[np.isin(warp_all[:, 0], fallback)]], axis=0)
        elif cta_kind == GEMV_ROWS:
            cta_units, warp_units = build_rows_worklist(table, D)
            records = ranges = np.zeros((0, 2), dtype=np.int32)
        else:
            cta_units, warp_units = build_worklist(table, D)
            records = ranges = np.zeros((0, 2), dtype=np.int32)
        d_table = to_device(queue, table)
        d_xstr = to_device(queue, xstrides[:, :max(D, 1)]) if np.any(xstrides != 1) else None
        d_cta = to_device(queue, cta_units) if len(cta_units) else None
        d_warp = to_device(queue, warp_units) if len(warp_units) else None
        d_records = to_device(queue, records) if len(records) else None
        d_ranges = to_device(queue, ranges) if len(ranges) else None
        status = zeros(queue, (1,), np.int32)
        A, X, Y, Y_in = self.A.cl_buf, self.X.cl_buf, self.Y.cl_buf, self.Y_in.cl_buf
        alpha = self.float_alpha if self.float_alpha is not None else 1.0
        beta = self.float_beta if self.float_beta is not None else 1.0
        gamma = self.float_gamma if self.float_gamma is not None else 0.0
        p = lambda arr: None if arr is None else arr.ptr
        n_cta, n_warp, n_rec, n_ranges = len(cta_units), len(warp_units), len(records), len(ranges)
        fn = _capi.lib().nb2_gemv_ragged
        fn_pipe = _capi.lib().nb2_gemv_pipelined
        check = _capi.check
        scales = (alpha, beta, gamma, p(self.cl_alpha), p(self.cl_beta), p(self.cl_gamma), status.ptr)

        def launch(stream):
            if n_rec:
                check(fn_pipe(stream, d_records.ptr, n_rec, d_ranges.ptr, n_ranges, A.ptr, X.ptr, Y_in.ptr, Y.ptr,
                              *scales))
            if n_cta:
                check(fn(stream, cta_kind, d_table.ptr, stride, D, p(d_xstr), d_cta.ptr, n_cta, A.ptr, X.ptr,
                         Y_in.ptr, Y.ptr, *scales))
            if n_warp:
                check(fn(stream, _capi.GEMV_WARP, d_table.ptr, stride, D, p(d_xstr), d_warp.ptr, n_warp, A.ptr,
                         X.ptr, Y_in.ptr, Y.ptr, *scales))

        plan = Plan(queue, launch, gsize, lsize, n_launches=int(n_cta > 0) + int(n_warp > 0) + int(n_rec > 0),
                    name=name, tag=self.tag, bw_per_call=bw_from_geometry(self.geometry, items),
                    flops_per_call=flops_from_geometry(self.geometry, items))
        plan.full_args = (d_table, d_xstr, d_cta, d_warp, d_records, d_ranges, status, A, X, Y, Y_in,
                          self.cl_alpha, self.cl_beta, self.cl_gamma)  # keep device arrays alive
        plan.gstructure = table
        plan.worklist = (cta_units, warp_units)
        plan.records = records
        plan.ranges = ranges
        plan.status = status
        plan.description = self.geometry_summary(items) if items else "empty"
        return plan

    # ---- the reference's four launch geometries ---------------------------
    def _max_y_len(self, items):
        return max(int(self.geometry[ii]["y_len"]) for ii in items)

    def ref_impl(self, items):
        """Thread-per-row geometry of ``ref_impl`` (clra_gemv.py:264-444)."""
        items = list(items)
        if self.clra_alpha is not None or self.clra_gamma is not None:
            raise NotImplementedError()
        gsize = (max(self._max_y_len(items), 1), len(items))
        return self._device_plan(items, "cura_gemv.ref_impl", gsize, None)

    def reduce_launch_shape(self, items, group_size=None, segment_size=None):
        """(gsize, lsize) of ``reduce_impl`` (clra_gemv.py:481-493)."""
        items = list(items)
        max_y_len = self._max_y_len(items)
        group_size = 32 if group_size is None else group_size
        if segment_size is None:
            segment_size = min(max_y_len, 2 if len(items) < 4 else 4)
        g_segments = int(np.ceil(float(max_y_len) / max(segment_size, 1)))
        return (group_size, g_segments * segment_size, len(items)), (group_size, segment_size, 1)

    def many_dots_launch_shape(self, items):
        """(gsize, lsize) of ``many_dots_impl`` (clra_gemv.py:713-725)."""
        items = list(items)
        max_n_dots = int(max(self.A_js.shape0s))
        max_y_len = self._max_y_len(items)
        segment_size = min(max_y_len, 16)
        dot_block_size = min(max(max_n_dots, 1),
                             int(self.queue.device.max_work_group_size / max(segment_size, 1)))
        n_segments = int(np.ceil(float(max_y_len) / max(segment_size, 1)))
        return (n_segments * segment_size, dot_block_size, len(items)), (segment_size, dot_block_size, 1)

    def reduce_impl(self, items, group_size=None, segment_size=None):
        """Items in the launch geometry of ``reduce_impl`` (clra_gemv.py:447-670)."""
        items = list(items)
        if self.cl_alpha is not None or self.cl_gamma is not None:
            raise NotImplementedError()
        self._check_supported(True)
        gsize, lsize = self.reduce_launch_shape(items, group_size, segment_size)
        return self._device_plan(items, "cura_gemv.reduce_impl", gsize, lsize)

    def many_dots_impl(self, items):
        """Items in the launch geometry of ``many_dots_impl`` (clra_gemv.py:673-858)."""
        items = list(items)
        if self.cl_alpha is not None or self.cl_gamma is not None:
            raise NotImplementedError()
        if self.A_js is None:
            raise NotImplementedError()
        self._check_supported(True)
        gsize, lsize = self.many_dots_launch_shape(items)
        return self._device_plan(items, "cura_gemv.many_dots_impl", gsize, lsize)

    def block_tile_tables(self, items, block_y=32, block_x=128):
        """Tile and reduce tables of ``block_impl`` (clra_gemv.py:911-969,1081-1095).

        One tile row per (item, 32-row block, term, 128-column block):
        ``[rows, cols, A stride0, A stride1, A start, X stride0, X start, Ybuf start]``;
        one reduce row per (item, row block).
        """
        A, X, Y, Y_in = self.A, self.X, self.Y, self.Y_in
        tiles = []
        reduce_rows = []
        reduce_inds = []
        ybuf = 0
        bw_reduce = 0
        for n in items:
            assert Y_in.shape0s[n] == Y.shape0s[n]
            M = int(Y.shape0s[n])
            xs, as_ = self._term_indices(n)
            for aj, xj in zip(as_, xs):
                assert A.shape0s[aj] == M
                assert A.shape1s[aj] == X.shape0s[xj]
                assert X.shape1s[xj] == 1
            for i in range(0, M, block_y):
                rows = min(M - i, block_y)
                inds = []
                for aj, xj in zip(as_, xs):
                    N = int(A.shape1s[aj])
                    as0, as1 = int(A.stride0s[aj]), int(A.stride1s[aj])
                    xs0 = int(X.stride0s[xj])
                    for j in range(0, N, block_x):
                        tiles.append((rows, min(N - j, block_x), as0, as1,
                                      int(A.starts[aj]) + i * as0 + j * as1, xs0,
                                      int(X.starts[xj]) + j * xs0, ybuf))
                        inds.append(ybuf)
                        ybuf += block_y
                reduce_rows.append((rows, int(Y_in.stride0s[n]), int(Y_in.starts[n]) + i * int(Y_in.stride0s[n]),
                                    int(Y.stride0s[n]), int(Y.starts[n]) + i * int(Y.stride0s[n])))
                reduce_inds.append(inds)
                bw_reduce += rows * (len(inds) + 1) * Y.dtype.itemsize
        gstructure = np.array(tiles, dtype=np.int32).reshape(-1, 8)
        return {
            "gstructure": gstructure,
            "Ybuf_size": ybuf,
            "reduce": np.array(reduce_rows, dtype=np.int32).reshape(-1, 5),
            "reduce_inds": reduce_inds,
            "bw_reduce": bw_reduce,
        }

    def block_impl(self, items):
        """``block_impl`` (clra_gemv.py:861-1175) as one single-pass plan.

        The reference launches a tile kernel that writes partial sums to a
        scratch buffer and a second kernel that reduces them; here one kernel
        (``nb2_gemv_block``) forms the same tile values in the same order and adds
        them to the output directly, so results are bit-identical to the pair and
        one plan is returned.  The tile tables are still built
        (``plan.tile_tables``) because they define the reference's launch
        geometry and are part of the bit-exact index-plan contract.
        """
        items = list(items)
        if self.cl_alpha is not None or self.cl_beta is not None or self.cl_gamma is not None:
            raise NotImplementedError()
        if self.A_js is None:
            raise NotImplementedError()
        self._check_supported(False)
        tables = self.block_tile_tables(items)
        n_tiles = max(len(tables["gstructure"]), 1)
        table, xstrides, D, _, stride = self.gstructure_table(items)
        # work units = the reference's 32-row blocks; blocks of at most 8 rows and 8 tiles per row
        # (scalar gains, single-row decoders) are taken by one warp each
        M = table[:, 4 * D + 3].astype(np.int64) if len(table) else np.zeros(0, np.int64)
        if D > 0 and len(table):
            n_dots = table[:, 4 * D + 2].astype(np.int64)
            mask = np.arange(D)[None, :] < n_dots[:, None]
            tiles_per_row = ((-(-table[:, 3 * D:4 * D].astype(np.int64) // 128)) * mask).sum(axis=1)
        else:
            tiles_per_row = np.zeros(len(table), np.int64)
        # Rows per unit: the reference's 32, or fewer when that would leave most of the GPU idle (the
        # dense transforms of a model are a few hundred rows: 8-row units put their tiles on separate
        # warps of more CTAs; the sum of a row is formed in the same order either way).
        sm_count = getattr(self.queue.device, "sm_count", 148)
        rows_per_unit = 32
        while rows_per_unit > 8 and int((-(-M // rows_per_unit)).sum()) < sm_count:
            rows_per_unit //= 2
        n_blocks = -(-M // rows_per_unit)
        rows_of = np.repeat(np.arange(len(table)), n_blocks)
        first = np.arange(int(n_blocks.sum())) - np.repeat(np.cumsum(n_blocks) - n_blocks, n_blocks)
        units = np.zeros((len(rows_of), 4), dtype=np.int32)
        units[:, 0], units[:, 1] = rows_of, first * rows_per_unit
        units[:, 2] = np.minimum(rows_per_unit, M[rows_of] - first * rows_per_unit)
        # one warp takes a unit of at most 8 rows whose tiles it can walk one after the other: up to 8
        # tiles when there is work for every SM anyway, a single tile when the units were made small
        # to spread the tiles of a row over warps
        max_tiles = 8 if rows_per_unit == 32 else 1
        small = (units[:, 2] <= 8) & (tiles_per_row[rows_of] <= max_tiles)
        cta_units, warp_units = units[~small], units[small]
        queue = self.queue
        d_table = to_device(queue, table)
        d_xstr = to_device(queue, xstrides[:, :max(D, 1)]) if np.any(xstrides != 1) else None
        d_cta = to_device(queue, cta_units) if len(cta_units) else None
        d_warp = to_device(queue, warp_units) if len(warp_units) else None
        A, X, Y, Y_in = self.A.cl_buf, self.X.cl_buf, self.Y.cl_buf, self.Y_in.cl_buf
        p = lambda arr: None if arr is None else arr.ptr
        fn, check = _capi.lib().nb2_gemv_block, _capi.check
        args = (d_table.ptr, stride, D, p(d_xstr), p(d_cta), len(cta_units), p(d_warp), len(warp_units), A.ptr,
                X.ptr, Y_in.ptr, Y.ptr, self.float_alpha, self.float_beta, self.float_gamma)

        def launch(stream):
            check(fn(stream, *args))

        plan = Plan(queue, launch, (4, 32, n_tiles), (4, 32, 1),
                    n_launches=1, name="cura_gemv.block_impl",
                    tag=self.tag, bw_per_call=bw_from_geometry(self.geometry, items),
                    flops_per_call=flops_from_geometry(self.geometry, items))
        plan.phase = _capi.phase("gemv_block", *args)
        plan.full_args = (d_table, d_xstr, d_cta, d_warp, A, X, Y, Y_in)
        plan.gstructure = table
        plan.worklist = (cta_units, warp_units)
        plan.description = self.geometry_summary(items) if items else "empty"
        plan.tile_tables = tables
        return [plan]

    def choose_plans(self):
        raise NotImplementedError("use a plan_*_gemv subclass")


class gemv_geometry(gemv_prog):
    """Host-only planner: geometry and index tables, no device plans (accepts
    host ragged arrays and ``queue=None``)."""

    def choose_plans(self):
        return []


class plan_ref_gemv(gemv_prog):
    def choose_plans(self):
        return [self.ref_impl(range(len(self.Y)))]


class plan_many_dots_gemv(gemv_prog):
    def choose_plans(self):
        return [self.many_dots_impl(range(len(self.Y)))]


class plan_reduce_gemv(gemv_prog):
    def choose_plans(self):
        return [self.reduce_impl(range(len(self.Y)))]


class plan_block_gemv(gemv_prog):
    def choose_plans(self):
        return self.block_impl(list(range(len(self.Y))))


class plan_ragged_gather_gemv(gemv_prog):
    """The reference's dispatcher (clra_gemv.py:1198-1239): items with <= 2
    terms and a long inner product go to ``reduce_impl``, the rest to
    ``many_dots_impl``, leftovers to ``ref_impl``; ``NotImplementedError`` from a
    specialised variant falls through to the next one."""

    def choose_plans(self):
        remaining = list(range(len(self.Y)))
        plans = []
        long_dots = [
            ii for ii in remaining
            if len(self.geometry[ii]["dots"]) <= 2
            and max([0] + [d["a_shape1"] for d in self.geometry[ii]["dots"]]) > 16
        ]
        if long_dots:
            try:
                long_plan = self.reduce_impl(long_dots)
            except NotImplementedError:
                long_plan = self.ref_impl(long_dots)
            long_plan.tag += "-long%i" % len(long_dots)
            plans.append(long_plan)
            taken = set(long_dots)
            remaining = [ii for ii in remaining if ii not in taken]
        if remaining:
            try:
                many_plan = self.many_dots_impl(remaining)
                many_plan.tag += "-many%i" % len(remaining)
                plans.append(many_plan)
                remaining = []
            except NotImplementedError:
                pass
        if remaining:
            rest = self.ref_impl(remaining)
            rest.tag += "-remaining%i" % len(remaining)
            plans.append(rest)
        return plans


class plan_fused_gemv(gemv_prog):
    """All items in one single-pass plan (no reference counterpart; what the
    B200 simulator uses by default)."""

    def choose_plans(self):
        n = len(self.Y)
        return [self._device_plan(range(n), "cura_gemv.single_pass", (max(n, 1),), None)]
