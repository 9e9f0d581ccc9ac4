"""Integer index plans are bit-identical to what the reference's planners
upload (tests/golden/tables.npz, captured from the reference's own plan_*
functions by tests/golden/make_golden.py).  Host-only: no device needed."""

import numpy as np
import pytest

from nengo_ocl_b200 import cura_gemv, cura_nonlinearities as nl
from nengo_ocl_b200.raggedarray import RaggedArray
from nengo_ocl_b200.synth import gemv_workload

RA = lambda arrays, dtype=np.float32: RaggedArray(arrays, dtype=dtype)


class HostQueue:
    """Enough of a queue for the host-side planners."""

    class device:
        max_work_group_size = 1024


def gemv_cases():
    A = RA([[[0.1, 0.2], [0.3, 0.4]], [[0.5, 0.6]]])
    X = RA([[3, 5]])
    Y = RA([[0.0], [2, 3]])
    yield "basic", (A, RA([[1], [0]], np.int32), X, RA([[0], [0]], np.int32), Y), (1.0, 1.0, 0.0)
    rng = np.random.RandomState(1234)
    ND = 20
    A = RA([0.1 + rng.rand(10, 1 + ii % 2) for ii in range(ND)])
    X = RA([0.1 + rng.rand(1 + ii % 2, 1) for ii in range(ND)])
    Y = RA([0.1 + rng.rand(10, 1)])
    yield "manydots20", (A, RA([range(ND)], np.int32), X, RA([range(ND)], np.int32), Y), (0.5, 0.6, 0.7)
    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=64)
    yield "config2_k64", (A, A_js, X, X_js, Y), (0.5, 0.1, 0.0)


@pytest.mark.parametrize("case", list(gemv_cases()), ids=lambda c: c[0])
def test_gemv_index_tables_match_reference(case, golden_tables):
    tag, (A, A_js, X, X_js, Y), (alpha, beta, gamma) = case
    g = golden_tables
    prog = cura_gemv.gemv_geometry(HostQueue(), alpha, A, A_js, X, X_js, beta, Y, gamma=gamma)
    items = list(range(len(Y)))

    # per-item table of many_dots / reduce (cl_geometry_and_textconf)
    table, _, D, n_vars, stride = prog.gstructure_table(items)
    for pname in ("plan_many_dots_gemv", "plan_reduce_gemv"):
        ref = g["%s/%s/gstructure" % (tag, pname)]
        assert table.dtype == ref.dtype == np.int32
        assert np.array_equal(table, ref)
    assert tuple(g[tag + "/plan_many_dots_gemv/plan0/gsize"]) == prog.many_dots_launch_shape(items)[0]
    assert tuple(g[tag + "/plan_many_dots_gemv/plan0/lsize"]) == prog.many_dots_launch_shape(items)[1]
    assert tuple(g[tag + "/plan_reduce_gemv/plan0/gsize"]) == prog.reduce_launch_shape(items)[0]
    assert tuple(g[tag + "/plan_reduce_gemv/plan0/lsize"]) == prog.reduce_launch_shape(items)[1]
    assert int(g[tag + "/plan_many_dots_gemv/plan0/bw"]) == cura_gemv.bw_from_geometry(prog.geometry, items)
    assert int(g[tag + "/plan_many_dots_gemv/plan0/flops"]) == cura_gemv.flops_from_geometry(prog.geometry, items)

    # 32 x 128 tile table and reduce tables of block_impl
    t = prog.block_tile_tables(items)
    key = tag + "/plan_block_gemv"
    assert np.array_equal(t["gstructure"], g[key + "/gstructure"])
    assert t["Ybuf_size"] == int(g[key + "/Ybuf_size"])
    red = t["reduce"]
    for col, nm in enumerate(["Yshape0s", "Yinstride0s", "Yinstarts", "Ystride0s", "Ystarts"]):
        assert np.array_equal(red[:, col], g[key + "/reduce_" + nm])
    flat = RA(t["reduce_inds"], dtype=np.int32)
    assert np.array_equal(flat.starts, g[key + "/reduce_inds_starts"])
    assert np.array_equal(flat.shape0s, g[key + "/reduce_inds_shape0s"])
    assert np.array_equal(flat.buf, g[key + "/reduce_inds_buf"])
    assert tuple(g[key + "/plan0/gsize"]) == (4, 32, len(t["gstructure"]))
    assert tuple(g[key + "/plan1/gsize"]) == (32, len(red))
    assert int(g[key + "/plan1/bw"]) == t["bw_reduce"]


def test_dispatcher_item_split_matches_reference(golden_tables):
    """plan_ragged_gather_gemv: <=2 terms with a long inner product -> reduce,
    rest -> many_dots (nengo_ocl/clra_gemv.py:1206-1232)."""
    g = golden_tables
    A, A_js, X, X_js, Y = gemv_workload(seed=1, n_outputs=64)
    prog = cura_gemv.gemv_geometry(HostQueue(), 0.5, A, A_js, X, X_js, 0.1, Y)
    geo = prog.geometry
    long_dots = [i for i in range(len(Y)) if len(geo[i]["dots"]) <= 2
                 and max([0] + [d["a_shape1"] for d in geo[i]["dots"]]) > 16]
    rest = [i for i in range(len(Y)) if i not in set(long_dots)]
    key = "config2_k64/plan_ragged_gather_gemv"
    assert int(g[key + "/n_plans"]) == 2
    assert np.array_equal(prog.gstructure_table(long_dots)[0], g[key + "/gstructure0"])
    assert np.array_equal(prog.gstructure_table(rest)[0], g[key + "/gstructure1"])
    assert tuple(g[key + "/plan0/gsize"]) == prog.reduce_launch_shape(long_dots)[0]
    assert tuple(g[key + "/plan1/gsize"]) == prog.many_dots_launch_shape(rest)[0]


def test_worklist_covers_every_row_once():
    A, A_js, X, X_js, Y = gemv_workload(seed=3, n_outputs=200)
    prog = cura_gemv.gemv_geometry(HostQueue(), 1.0, A, A_js, X, X_js, 1.0, Y)
    table, _, D, _, _ = prog.gstructure_table(range(len(Y)))
    cta, warp = cura_gemv.build_worklist(table, D)
    seen = [np.zeros(int(m), dtype=int) for m in Y.shape0s]
    for item, r0, cnt, _ in np.vstack([cta, warp]):
        assert cnt >= 1
        seen[item][r0:r0 + cnt] += 1
    assert all((s == 1).all() for s in seen)
    assert (warp[:, 2] <= 32).all() and (cta[:, 2] <= 1024).all()
    # staged rows of a unit fit the shared-memory buffer when a single row does
    n_dots = table[:, 4 * D + 2]
    for item, r0, cnt, _ in cta:
        row = table[item, 3 * D:3 * D + n_dots[item]].sum()
        if row * 8 <= 8192 - 4 * n_dots[item] - 4:
            assert cnt * row + 4 * n_dots[item] + 4 <= 8192


# ---- blockify tables of the elementwise / neuron plans -------------------------
def test_template_block_tables_match_reference(golden_tables):
    g = golden_tables
    sizes = [100, 1000, 37, 2049]
    J = RA([np.zeros(n) for n in sizes])
    best = None
    for bs in [16, 32, 64, 128, 256, 512, 1024]:
        s, inds, starts = nl.blockify_vector(bs, J)
        if best is None or len(s) < len(best[1]):
            best = (bs, s, inds, starts)
    bs, s, inds, starts = best
    for up in (1, 4):
        key = "lif_up%d" % up
        assert tuple(g[key + "/gsize"]) == (bs, len(s))
        assert np.array_equal(s, g[key + "/sizes"])
        for nm in ["J", "V", "W", "outV", "outW", "outS", "tau"]:
            assert np.array_equal(starts, g["%s/%s_starts" % (key, nm)])
        assert int(g[key + "/bw"]) == 7 * 4 * sum(sizes)


def test_copy_elementwise_reset_slicedcopy_tables_match_reference(golden_tables):
    g = golden_tables
    shapes = [(3, 5), (1, 1), (700, 1), (40, 13)]
    X = RA([np.zeros(s) for s in shapes])
    sizes, inds, offsets = nl.blockify_ij(256, X)
    assert tuple(g["copy/gsize"]) == (256, len(sizes))
    assert np.array_equal(offsets, g["copy/offsets"])
    assert np.array_equal(X.shape0s[inds], g["copy/shape0s"])
    assert np.array_equal(X.shape1s[inds], g["copy/shape1s"])
    assert np.array_equal(X.stride0s[inds], g["copy/Xstride0s"])
    assert np.array_equal(X.starts[inds], g["copy/Xstarts"])
    assert np.array_equal(np.array([0, 1, 1, 0])[inds], g["copy/incs"])
    assert np.array_equal(offsets, g["ewinc/offsets"])
    assert np.array_equal(X.starts[inds], g["ewinc/Ystarts"])
    A = RA([np.zeros(s) for s in [(3, 5), (1, 1), (700, 1), (1, 13)]])
    assert np.array_equal(A.starts[inds], g["ewinc/Astarts"])

    Yr = RA([np.zeros(s) for s in [(3, 5), (1, 1), (70, 1), (4, 13)]])
    rs, rinds, rstarts = nl.blockify_matrix(16, Yr)
    assert np.array_equal(rs, g["reset/sizes"])
    assert np.array_equal(rstarts, g["reset/starts"])
    assert np.array_equal(np.array([0.0, 1.5, -2.0, 7.0], np.float32)[rinds], g["reset/values"])
    assert tuple(g["reset/lsize"]) == (16, 16)
    assert tuple(g["reset/gsize"]) == (16, -(-len(rs) // 16) * 16)

    xi = RA([np.arange(10)[::2], np.arange(50)[::-1].copy(), np.arange(33)[5:25]], np.int32)
    yi = RA([np.arange(20)[3:8], np.arange(50), np.arange(40)[::2]], np.int32)
    ss, sinds, (xs, ys) = nl.blockify_vectors(16, [xi, yi])
    assert np.array_equal(ss, g["slicedcopy/sizes"])
    assert np.array_equal(xs, g["slicedcopy/XIstarts"])
    assert np.array_equal(ys, g["slicedcopy/YIstarts"])
    assert tuple(g["slicedcopy/gsize"]) == (16, -(-len(ss) // 16) * 16)

    Xf = RA([np.zeros(s) for s in [(300, 1), (5, 1), (64, 1)]])
    fs, finds, foffs = nl.blockify_ij(256, Xf)
    assert tuple(g["linearfilter/lsize"]) == (256, 1)
    assert tuple(g["linearfilter/gsize"]) == (256, len(fs))
    assert np.array_equal(foffs, g["linearfilter/offsets"])


def _emulate_pipe_records(records, ranges, A, X, Yin, alpha, beta, gamma):
    """Host emulation of what nb2_gemv_pipelined does with its work records: the
    producer's bulk copies of 16-byte-aligned windows into the stage pool, then
    the consumer's reads from the pool."""
    Y = Yin.copy()
    assert ranges[0, 0] == 0 and ranges[-1, 1] == len(records)
    assert np.array_equal(ranges[1:, 0], ranges[:-1, 1])
    NW = cura_gemv.PIPE_CONSUMER_WARPS // cura_gemv.PIPE_WARPS_PER_RECORD  # warp groups
    C = cura_gemv.PIPE_STAGE_FLOATS

    def readable(buf, lo, nbytes):  # buffers are readable up to the next 16-byte boundary
        assert lo % 4 == 0 and nbytes % 16 == 0 and nbytes > 0
        n = nbytes // 4
        assert lo + n <= (len(buf) + 3) // 4 * 4
        out = np.full(n, np.nan)
        m = min(n, len(buf) - lo)
        out[:m] = buf[lo:lo + m]
        return out

    for b, e in ranges:
        for warp in range(NW):  # record i of a CTA range belongs to warp group i % NW
            acc = None
            for rec in records[b + warp:e:NW]:
                flags, R, y_in, y, bb, nseg, logG, yin_bytes = rec[:8]
                if R == 0:
                    assert flags == 0 and nseg == 0 and yin_bytes == 0  # padding record
                    continue
                assert 1 <= R <= cura_gemv.PIPE_RMAX and 0 <= nseg <= cura_gemv.PIPE_MAXSEG
                assert logG == 0
                if flags & 1:
                    acc = np.zeros(R, dtype=np.float64)
                assert acc is not None and len(acc) == R, "a chain stays within one warp"
                pool = np.full(C, np.nan)
                filled = np.zeros(C, dtype=bool)
                segs = []
                for q in range(nseg):
                    a_win, a_bytes, x_idx, x_bytes, w, packed = (int(v) for v in rec[8 + 6 * q: 14 + 6 * q])
                    aoff, xoff = packed & 0xFFFF, packed >> 16
                    dst = aoff & ~3
                    assert dst + a_bytes // 4 <= C and not filled[dst:dst + a_bytes // 4].any()
                    pool[dst:dst + a_bytes // 4] = readable(A, a_win, a_bytes)
                    filled[dst:dst + a_bytes // 4] = True
                    if x_bytes > 0:
                        dst = xoff & ~3
                        assert dst + x_bytes // 4 <= C and not filled[dst:dst + x_bytes // 4].any()
                        pool[dst:dst + x_bytes // 4] = readable(X, x_idx, x_bytes)
                        filled[dst:dst + x_bytes // 4] = True
                    segs.append((aoff, xoff, w, x_idx, x_bytes))
                for aoff, xoff, w, x_idx, x_bytes in segs:
                    a = pool[aoff:aoff + R * w].reshape(R, w)
                    x = pool[xoff:xoff + w] if x_bytes > 0 else X[x_idx + np.arange(w) * (-x_bytes)]
                    assert not np.isnan(a).any() and not np.isnan(x).any()
                    acc += a @ x.astype(np.float64)
                if flags & 2:
                    assert yin_bytes > 0
                    yin = readable(Yin, y_in & ~3, yin_bytes)[(y_in & 3):(y_in & 3) + R]
                    assert yin_bytes // 4 <= cura_gemv.PIPE_RMAX + 8 and np.array_equal(yin, Yin[y_in:y_in + R])
                    Y[y:y + R] = gamma + beta * yin + alpha * acc
                    acc = None
                else:
                    assert yin_bytes == 0
    return Y


@pytest.mark.parametrize("case", ["config2", "long_rows_many_terms"])
def test_pipe_records_cover_the_product(case):
    if case == "config2":
        A, A_js, X, X_js, Y = gemv_workload(seed=5, n_outputs=150)
    else:
        rng = np.random.RandomState(0)
        shapes = [(700, 3000), (700, 5), (9, 1200), (9, 40), (2, 1), (1000, 1)]
        A = RA([rng.normal(size=s) for s in shapes] + [rng.normal(size=(40, 7)) for _ in range(12)])
        X = RA([rng.normal(size=(s[1], 1)) for s in shapes] + [rng.normal(size=(7, 1)) for _ in range(12)])
        Y = RA([rng.normal(size=(700, 1)), rng.normal(size=(9, 1)), rng.normal(size=(2, 1)),
                rng.normal(size=(1000, 1)), rng.normal(size=(40, 1))])
        A_js = RA([[0, 1], [2, 3], [4], [5], list(range(6, 18))], np.int32)
        X_js = A_js
    prog = cura_gemv.gemv_geometry(HostQueue(), 0.5, A, A_js, X, X_js, 0.1, Y)
    table, xstrides, D, _, _ = prog.gstructure_table(range(len(Y)))
    records, ranges, warp, fallback = cura_gemv.build_pipe_records(table, xstrides, D, n_ctas_max=444)
    assert len(fallback) == 0
    assert records.dtype == np.int32 and records.shape[1] == 32
    got = _emulate_pipe_records(records, ranges, A.buf, X.buf, Y.buf, 0.5, 0.1, 0.0)
    from oracle import kernels as K

    vals, _ = K.gemv_exact(0.5, A, A_js, X, X_js, 0.1, Y)
    done_by_warp = set(int(table[r, 4 * D + 4]) for r in warp[:, 0])
    for i in range(len(Y)):
        lo = int(Y.starts[i])
        if i in done_by_warp:
            assert np.array_equal(got[lo:lo + len(vals[i])], Y.buf[lo:lo + len(vals[i])])
        else:
            assert np.allclose(got[lo:lo + len(vals[i])], vals[i], rtol=1e-6, atol=1e-6)
    assert len(ranges) <= 444


def test_stream_records_cover_every_ensemble_once():
    """Work records of the streamed fused kernel: every neuron is in exactly one E
    record and every decoder row in exactly one D record, copies are 16-byte
    aligned and fit a stage, and in list order no record waits for a later one."""
    from nengo_ocl_b200 import fusion

    rng = np.random.RandomState(0)
    ens, terms, conns, pos = [], [], [], 0

    def alloc(n):
        nonlocal pos
        start = pos
        pos += (n + 3) // 4 * 4
        return start

    for n, ds, dcs in [(1024, [16], [(16, True)]), (512, [8, 4], [(3, False), (16, True)]), (260, [], [(5, False)]),
                       (1024, [16], []), (300, [12], [(2, True)])] * 3 + [(200, [4], [(1, False)]),
                                                                          (1024, [16, 16, 16, 16, 4], [(1, False)])]:
        row = [n, -1, alloc(n), alloc(n), alloc(n) if rng.rand() < 0.5 else -1, alloc(n), len(ds), len(terms), len(dcs),
               len(conns), 0, 0, 0, 1, 0, 0]
        for d in ds:
            terms.append([alloc(n * d), d, alloc(d), 1])
        for d_c, pes in dcs:
            conns.append([alloc(d_c * n), d_c, alloc(d_c), alloc(d_c), 0, 0, int(pes), alloc(d_c), alloc(n), 0, 0, 0,
                          0, 0, 0, 0])
        ens.append(row)
    ens = np.asarray(ens, np.int32)
    terms = np.asarray(terms, np.int32).reshape(-1, 4)
    conns = np.asarray(conns, np.int32).reshape(-1, 16)
    rows = fusion.streamable(ens, terms, conns)
    assert set(rows) == set(range(15))  # not the 200-neuron one, not the one with five encoder terms
    records, ranges = fusion.stream_records(ens, terms, conns, rows, n_ctas_max=4)
    assert records.shape[1] == 32 and ranges[0, 0] == 0 and ranges[-1, 1] == len(records) and len(ranges) <= 4
    neurons = {int(r): np.zeros(ens[r, 0], int) for r in rows}
    dec_rows = {}
    seen_ens = set()
    for b, e in ranges:
        e_done = [0] * fusion.STREAM_SLOTS
        d_done = [0] * fusion.STREAM_SLOTS
        mine = set()
        for rec in records[b:e]:
            kind, r, slot, ncopy, target = int(rec[0]), int(rec[1]), int(rec[2]), int(rec[5]), int(rec[6])
            mine.add(r)
            used = np.zeros(fusion.STREAM_STAGE_FLOATS, bool)
            for q in range(ncopy):
                idx, nbytes, off = (int(v) for v in rec[8 + 3 * q:11 + 3 * q])
                assert idx % 4 == 0 and nbytes % 16 == 0 and nbytes > 0 and off % 4 == 0
                assert off + nbytes // 4 <= fusion.STREAM_STAGE_FLOATS and not used[off:off + nbytes // 4].any()
                assert idx + nbytes // 4 <= pos
                used[off:off + nbytes // 4] = True
            n = int(ens[r, 0])
            if kind == 1:
                assert d_done[slot] >= target, "an E record would wait for a later D record"
                i0, ne = int(rec[3]), int(rec[4])
                assert 0 < ne <= 192 and ne % 4 == 0 and i0 + ne <= n
                neurons[r][i0:i0 + ne] += 1
                nt, t0 = int(ens[r, 6]), int(ens[r, 7])
                assert ncopy == nt + 3 + (rec[7] >= 0)
                for k in range(nt):
                    assert rec[8 + 3 * k] == terms[t0 + k, 0] + i0 * terms[t0 + k, 1]
                assert rec[8 + 3 * nt] == ens[r, 5] + i0 and rec[8 + 3 * (nt + 1)] == ens[r, 2] + i0
                if rec[7] >= 0:
                    assert conns[rec[7], 6] == 1 and rec[8 + 3 * (nt + 3)] == conns[rec[7], 8] + i0
                e_done[slot] += 1
            else:
                assert kind == 2 and e_done[slot] >= target, "a D record would wait for a later E record"
                c, r0, nr = int(rec[3]), int(rec[4]), int(rec[7])
                assert int(ens[r, 9]) <= c < int(ens[r, 9]) + int(ens[r, 8]) and 0 < nr and nr * (-(-n // 128)) <= fusion.STREAM_DITEMS
                assert nr * n <= fusion.STREAM_STAGE_FLOATS
                dec_rows.setdefault(c, np.zeros(conns[c, 1], int))[r0:r0 + nr] += 1
                assert rec[8] == conns[c, 0] + r0 * n and rec[9] == 4 * nr * n
                d_done[slot] += 1
        assert not (mine & seen_ens), "an ensemble belongs to one CTA"
        seen_ens |= mine
    assert all((v == 1).all() for v in neurons.values())
    for r in rows:
        for c in range(int(ens[r, 9]), int(ens[r, 9]) + int(ens[r, 8])):
            assert (dec_rows[c] == 1).all()
