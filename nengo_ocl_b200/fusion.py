"""Fusion of ensemble-pattern operators into one kernel per step.

The reference runs one ragged kernel per operator group (nengo_ocl/
simulator.py:352-356): bias copy, encoder GEMV, neuron update, reset of the
decoded values, decoder GEMV, synapse filter, and for PES the activity filter,
the outer-product delta and the decoder increment -- about ten launches and
five passes over the encoder/decoder matrices.  This pass recognises that
pattern per population in the operator list and replaces all matching operators
by one ``FusedEnsembles`` operator, which the planner then schedules like any
other operator (so every dependency through shared signals is still honoured)
and which is executed by ``nb2_ensemble_step`` (csrc/nb2_fused.cu).

Per population (a ``SimNeurons`` operator with LIF neurons) the pattern is:

* ``J``: set by one un-sliced ``Copy`` (the bias) and incremented by exactly one
  ``MultiDotInc`` whose terms are dense row-major ``(n, d)`` matrices (or by
  none, when the simplifier removed a product with a constant-zero input);
  nothing else reads or writes ``J``;
* each decoded connection: a one-term ``MultiDotInc`` ``decoded += W . spikes``
  with row-major ``(d_c, n)`` weights onto a signal that is otherwise only
  reset to zero; optionally a first-order ``LinearFilter`` process (lowpass or
  pure gain, "update" mode) reading the decoded signal;
* optionally PES on that connection: a lowpass process spikes -> activity
  trace, a ``SimPES`` operator producing the delta from the trace and an error
  signal, and the un-sliced ``Copy(delta -> W, inc=True)``, with nothing else
  touching ``W`` or the delta.

Anything that does not match stays un-fused.  Two observable differences of the
fused path: ``J`` (and the spikes, when nothing else reads them) are not stored,
and the PES delta is applied to the decoders at the end of the step that
computes it instead of at the start of the next one, so between steps
``weights`` already contains the delta that the un-fused path still holds in
``delta`` (the decoded values of every step are identical).
"""

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.model import Operator
from nengo_ocl_b200.operators import MultiDotInc
from nengo_ocl_b200.plan import Plan
from nengo_ocl_b200.runtime import to_device, zeros

MAX_NEURONS, SMALL_NEURONS, MAX_INPUT = 4096, 256, 512


class FusedEnsembles(Operator):
    """All fused populations of a model as one operator."""

    def __init__(self, members):
        Operator.__init__(self, tag="fused-%d" % len(members))
        self.members = members
        sets, incs, reads, updates = [], [], [], []
        internal = set()
        for mem in members:
            internal.add(mem["J"])
            sets.append(mem["out"])
            updates.extend(mem["state"])
            reads.append(mem["bias"])
            for A, X in mem["enc_terms"]:
                reads.extend([A, X])
            for c in mem["conns"]:
                sets.append(c["weighted"])
                if c["filtered"] is not None:
                    updates.append(c["filtered"])
                if c["pes"]:
                    reads.append(c["error"])
                    updates.extend([c["pre_filtered"], c["W"]])
                    internal.add(c["delta"])
                    if c.get("error_alias") is not None:
                        internal.add(c["error_alias"])
                else:
                    reads.append(c["W"])
        self.sets, self.incs, self.reads, self.updates = sets, incs, reads, updates
        self.internal = internal


def _is_type(op, name):
    return type(op).__name__ == name


def _dense_rowmajor(view):
    """2-D view whose rows are contiguous and packed."""
    return view.ndim == 2 and (view.shape[1] == 1 or view.elemstrides[1] == 1) and (
        view.shape[0] == 1 or view.elemstrides[0] == view.shape[1])


def _first_order(sim, op):
    """(b0, a0) of a first-order filter process op, or None."""
    try:
        num, den = sim.linear_filter_coefficients(op)
    except Exception:  # not a linear filter we understand
        return None
    if len(num) == 1 and len(den) <= 1:
        return float(np.float32(num[0])), (float(np.float32(den[0])) if len(den) else 0.0)
    return None


def _is_linear_filter(op):
    return _is_type(op, "SimProcess") and any(c.__name__ == "LinearFilter" for c in type(op.process).__mro__)


def _extent(sig):
    lo = sig.elemoffset
    return lo, lo + sum((n - 1) * abs(st) for n, st in zip(sig.shape, sig.elemstrides)) + 1


def _writers_overlapping(writers, cache, sig):
    """Number of writer entries of ``sig.base`` whose element range overlaps ``sig``."""
    base = sig.base
    if base not in cache:
        ext = np.array([_extent(w[2]) for w in writers.get(base, [])], dtype=np.int64).reshape(-1, 2)
        cache[base] = (ext[:, 0], ext[:, 1])
    los, his = cache[base]
    lo, hi = _extent(sig)
    return int(np.count_nonzero((los < hi) & (his > lo)))


def find_fusable(sim, operators):
    """Match the ensemble pattern; returns (members, consumed operators)."""
    writers, readers = {}, {}
    for op in operators:
        for kind in ("sets", "incs", "updates"):
            for s in getattr(op, kind):
                writers.setdefault(s.base, []).append((op, kind, s))
        for s in op.reads:
            readers.setdefault(s.base, []).append((op, s))

    extents = {}  # base -> (lo, hi) arrays of its writers' element ranges, built on demand
    members, consumed = [], set()
    for nop in operators:
        if not _is_type(nop, "SimNeurons") or type(nop.neurons).__name__ != "LIF":
            continue
        if nop.neurons.min_voltage != 0 or nop.J.is_view or nop.output.is_view:
            continue
        n = nop.J.size
        if n > MAX_NEURONS:
            continue
        J, out = nop.J, nop.output
        # --- J: bias copy + one encoder MultiDotInc
        jw = writers.get(J, [])
        bias_ops = [op for op, kind, s in jw if _is_type(op, "Copy") and kind == "sets" and s is J]
        enc_ops = [op for op, kind, s in jw if isinstance(op, MultiDotInc) and kind == "incs" and s is J]
        if len(bias_ops) != 1 or len(enc_ops) > 1 or len(jw) != 1 + len(enc_ops):
            continue
        # (an ensemble whose input is known to be zero has had its encoder product removed)
        bias_op, enc_op = bias_ops[0], (enc_ops[0] if enc_ops else None)
        if bias_op.src_slice is not None or bias_op.dst_slice is not None or bias_op.src.is_view:
            continue
        if [op for op, _ in readers.get(J, [])] != [nop]:
            continue
        A_views = sim._A_views[enc_op] if enc_op is not None else []
        X_views = sim._X_views[enc_op] if enc_op is not None else []
        if not all(_dense_rowmajor(A) and A.shape[0] == n and X.shape == (A.shape[1], 1)
                   for A, X in zip(A_views, X_views)):
            continue
        if sum(A.shape[1] for A in A_views) > MAX_INPUT:
            continue
        member = dict(neurons=nop, J=J, out=out, n=n, bias=bias_op.src, enc_terms=list(zip(A_views, X_views)),
                      state=[nop.state["voltage"], nop.state["refractory_time"]], conns=[],
                      ops=[nop, bias_op] + ([enc_op] if enc_op is not None else []))

        # --- decoded connections reading the spikes
        out_readers = [op for op, s in readers.get(out, []) if s is out]
        for dop in out_readers:
            if not isinstance(dop, MultiDotInc) or len(dop.As) != 1 or dop.Xs[0] is not out:
                continue
            if dop._signal_beta is not None or dop._float_beta != 1 or dop.gamma != 0 or dop.Y_in is not dop.Y:
                continue
            Wv = sim._A_views[dop][0]
            weighted = dop.Y
            if weighted.is_view or not _dense_rowmajor(Wv) or Wv.shape[1] != n or Wv.is_view and Wv.size != Wv.base.size:
                continue
            ww = writers.get(weighted, [])
            resets = [op for op, kind, s in ww if _is_type(op, "Reset") and s is weighted and op.value == 0]
            if len(ww) != 2 or len(resets) != 1:
                continue
            conn = dict(W=Wv.base, W_view=Wv, d=Wv.shape[0], weighted=weighted, filtered=None, b0=0.0, a0=0.0,
                        pes=False, ops=[dop, resets[0]])
            # synapse on the decoded value
            wr = [op for op, s in readers.get(weighted, []) if s is weighted]
            # the filtered value may be a packed slice of a larger signal (an exchange buffer)
            filt = [op for op in wr if _is_linear_filter(op) and op.mode == "update" and op.input is weighted
                    and op.output.ndim == 1 and (op.output.size == 1 or op.output.elemstrides[0] == 1)]
            if len(filt) == 1 and len(wr) == 1:
                coef = _first_order(sim, filt[0])
                if coef is not None and _writers_overlapping(writers, extents, filt[0].output) == 1:
                    conn.update(filtered=filt[0].output, b0=coef[0], a0=coef[1])
                    conn["ops"].append(filt[0])
            # PES on the decoders
            Wbase = Wv.base
            w_writers = writers.get(Wbase, [])
            if len(w_writers) == 1:
                cop = w_writers[0][0]
                if (_is_type(cop, "Copy") and cop.inc and cop.src_slice is None and cop.dst_slice is None
                        and cop.dst is Wbase and not cop.src.is_view):
                    delta = cop.src
                    dw = writers.get(delta, [])
                    dr = [op for op, _ in readers.get(delta, [])]
                    w_readers = [op for op, _ in readers.get(Wbase, [])]
                    if (len(dw) == 1 and _is_type(dw[0][0], "SimPES") and dr == [cop] and w_readers == [dop]):
                        pes_op = dw[0][0]
                        pf = pes_op.pre_filtered
                        pfw = writers.get(pf, [])
                        pfr = [op for op, _ in readers.get(pf, [])]
                        if (len(pfw) == 1 and _is_linear_filter(pfw[0][0]) and pfw[0][0].input is out
                                and pfw[0][0].mode == "update" and pfr == [pes_op] and not pf.is_view
                                and pes_op.delta is delta and pes_op.error.size == conn["d"]):
                            coef = _first_order(sim, pfw[0][0])
                            if coef is not None and coef[1] != 0.0:
                                conn.update(pes=True, delta=delta, error=pes_op.error, pre_filtered=pf,
                                            pf_b0=coef[0], pf_a0=coef[1],
                                            alpha=-pes_op.learning_rate * sim.model.dt / pf.shape[0])
                                conn["ops"] += [pes_op, cop, pfw[0][0]]
                                # An error signal that is only "reset to zero, += one whole signal" and read
                                # by nothing but this rule is that signal (0 + x = x): the kernel reads the
                                # source directly and the reset + copy need no launch of their own.
                                err = pes_op.error
                                ew = writers.get(err.base, [])
                                er = [op for op, _ in readers.get(err.base, [])]
                                e_reset = [op for op, kind, s in ew if _is_type(op, "Reset") and s is err
                                           and op.value == 0]
                                e_copy = [op for op, kind, s in ew if _is_type(op, "Copy") and kind == "incs"
                                          and s is err and op.src_slice is None and op.dst_slice is None
                                          and op.src.size == err.size and _contiguous_1d(op.src)]
                                if (not err.is_view and len(ew) == 2 and len(e_reset) == 1 and len(e_copy) == 1
                                        and er == [pes_op]
                                        and not any(sim.model.sig[p]["in"].base is err for p in sim.model.probes)):
                                    conn.update(error=e_copy[0].src, error_alias=err)
                                    conn["ops"] += [e_reset[0], e_copy[0]]
            if not conn["pes"] and w_writers:
                continue  # somebody else modifies these weights during the step
            member["conns"].append(conn)
            member["ops"].extend(conn["ops"])
        fused_here = set(member["ops"])
        member["store_spikes"] = any(op not in fused_here for op in out_readers) or any(
            sim.model.sig[p]["in"].base is out for p in sim.model.probes)
        members.append(member)
    # The fused kernel runs all members concurrently: a member whose encoder input overlaps a
    # signal that the kernel itself writes (any member's decoded value, filtered value, spikes
    # or activity trace) could read the old or the new value.  The operator order gives it the
    # old one (reads come before updates), so such a member stays un-fused.
    written = {}
    for mem in members:
        sigs = [mem["out"]] + list(mem["state"])
        for c in mem["conns"]:
            sigs += [c["weighted"]] + ([c["filtered"]] if c["filtered"] is not None else [])
            sigs += [c["pre_filtered"], c["W"]] if c["pes"] else []
        for sig in sigs:
            written.setdefault(sig.base, []).append(_extent(sig))
    def reads_own_output(mem):
        for _, X in mem["enc_terms"]:
            lo, hi = _extent(X)
            if any(a < hi and b > lo for a, b in written.get(X.base, [])):
                return True
        return False

    members = [mem for mem in members if not reads_own_output(mem)]
    for mem in members:
        consumed.update(mem["ops"])
    return members, consumed


def fold_resets_into_products(operators):
    """``Reset(y, v)`` followed only by one merged product ``y += sum A_i x_i`` becomes the
    product in "set" form, ``y = v + sum A_i x_i`` (beta 0, gamma v): one launch less.
    The products are changed in place; returns the resets that are no longer needed."""
    writers = {}
    for op in operators:
        for kind in ("sets", "incs", "updates"):
            for s in getattr(op, kind):
                writers.setdefault(s.base, []).append((op, kind, s))
    dropped = set()
    changed = []
    for base, ws in writers.items():
        if base.is_view or len(ws) != 2:
            continue
        resets = [op for op, kind, s in ws if _is_type(op, "Reset") and s is base]
        dots = [op for op, kind, s in ws if isinstance(op, MultiDotInc) and kind == "incs" and s is base
                and op.Y is base and op.Y_in is base and op._signal_beta is None and op._float_beta == 1
                and op.gamma == 0]
        # (only a reset to zero: "0 + terms" is exact, any other value would be added after
        # the terms instead of before them and round differently)
        if len(resets) == 1 and len(dots) == 1 and resets[0].value == 0:
            changed.append((dots[0], dots[0]._float_beta, dots[0].gamma, dots[0]._incs_Y))
            dots[0]._float_beta, dots[0].gamma, dots[0]._incs_Y = 0.0, float(resets[0].value), False
            dropped.add(resets[0])
    fold_resets_into_products.last_changes = changed
    return dropped


def undo_fold(changes):
    """Put the products changed by ``fold_resets_into_products`` back into increment form."""
    for dot, beta, gamma, incs in changes:
        dot._float_beta, dot.gamma, dot._incs_Y = beta, gamma, incs


def fuse_ensemble_groups(sim, groups, planner=None):
    """Replace matched operators by one ``FusedEnsembles`` op and re-plan."""
    from nengo_ocl_b200.planners import greedy_planner

    planner = planner or getattr(sim, "_planner", None) or greedy_planner
    operators = sim.operators
    members, consumed = find_fusable(sim, operators)
    gathers, gathered = find_gather_sums([op for op in operators if op not in consumed])
    consumed = set(consumed) | gathered
    folded = fold_resets_into_products([op for op in operators if op not in consumed])
    if not members and not gathers and not folded:
        return groups
    consumed |= folded
    new_ops = [op for op in operators if op not in consumed] + gathers
    if members:
        new_ops.append(FusedEnsembles(members))
    try:
        new_groups = planner(new_ops)
    except ValueError:
        # merging would create a same-step dependency cycle: stay un-fused, with the products back
        # in the increment form that the kept groups (and their resets) were planned for
        undo_fold(getattr(fold_resets_into_products, "last_changes", []))
        return groups
    sim.operators = new_ops
    sim.fused_groups = [dict(pes=any(c["pes"] for c in mem["conns"]), n=mem["n"],
                             unstored=[mem["J"]] + ([] if mem["store_spikes"] else [mem["out"]])
                             + [c["delta"] for c in mem["conns"] if c["pes"]]
                             + [c["error_alias"] for c in mem["conns"] if c.get("error_alias") is not None])
                        for mem in members]
    return new_groups


def _fbits(x):
    return int(np.float32(x).view(np.int32))


def fused_tables(sim, members):
    """int32 tables of ``nb2_ensemble_step`` (layouts in include/nengo_b200.h)."""
    starts = sim.all_data.starts
    sidx = sim.sidx
    st = lambda sig: int(starts[sidx[sig]])
    ens, terms, conns = [], [], []
    dt32 = np.float32(sim.model.dt)
    for mem in members:
        nt = mem["neurons"].neurons
        # expm1(-dt / tau) of a neuron that integrates over the whole step: the float32 quotient,
        # evaluated in double and rounded once (what the kernels do for any other interval)
        em1_dt = np.float32(np.expm1(np.float64(-dt32 / np.float32(nt.tau_rc))))
        row = [mem["n"], -1, st(mem["state"][0]), st(mem["state"][1]), st(mem["out"]) if mem["store_spikes"] else -1,
               st(mem["bias"]), len(mem["enc_terms"]), len(terms), len(mem["conns"]), len(conns),
               _fbits(nt.tau_rc), _fbits(nt.tau_ref), _fbits(nt.amplitude), 0, _fbits(em1_dt), 0]
        for A, X in mem["enc_terms"]:
            xi = sidx[X]
            terms.append([st(A), A.shape[1], st(X), int(sim.all_data.stride0s[xi])])
        for c in mem["conns"]:
            crow = [st(c["W_view"]), c["d"], st(c["weighted"]), st(c["filtered"]) if c["filtered"] is not None else -1,
                    _fbits(c["b0"]), _fbits(c["a0"]), int(c["pes"]), 0, 0, 0, 0, 0, 0, 0, 0, 0]
            if c["pes"]:
                crow[7] = st(c["error"])
                crow[8] = st(c["pre_filtered"])
                crow[9], crow[10], crow[11] = _fbits(c["pf_b0"]), _fbits(c["pf_a0"]), _fbits(c["alpha"])
            conns.append(crow)
        # 128-bit path when the neuron count, every encoder width and every array start are multiples of 4
        first_conn = row[9]
        offsets = [row[2], row[3], row[5]] + ([row[4]] if row[4] >= 0 else [])
        offsets += [v for trow in terms[row[7]:] for v in (trow[0], trow[1])]
        offsets += [v for crow in conns[first_conn:] for v in (crow[0],) + ((crow[8],) if crow[6] else ())]
        row[13] = int(mem["n"] % 4 == 0 and all(v % 4 == 0 for v in offsets))
        ens.append(row)
    as32 = lambda rows, width: np.asarray(rows, dtype=np.int32).reshape(-1, width)
    return as32(ens, 16), as32(terms, 4), as32(conns, 16)


def fused_bytes_per_step(members):
    """Algorithmic bytes of one fused step: encoders, bias, x, state (V, W read
    and write), decoders and decoded values; with PES also the decoder write,
    the activity trace (read and write) and the error."""
    total = 0
    for mem in members:
        n = mem["n"]
        d_in = sum(A.shape[1] for A, _ in mem["enc_terms"])
        total += 4 * n * d_in + 4 * n + 4 * d_in + 16 * n
        if mem["store_spikes"]:
            total += 4 * n
        for c in mem["conns"]:
            total += 4 * c["d"] * n + 4 * c["d"]
            if c["filtered"] is not None:
                total += 8 * c["d"]
            if c["pes"]:
                total += 4 * c["d"] * n + 8 * n + 4 * c["d"]
    return total


# ---- streamed kernel for large populations (csrc/nb2_fused_stream.cu) ---------------
_STREAM = _capi.header_constants("NB2_STREAM_")
STREAM_STAGE_FLOATS = _STREAM["NB2_STREAM_STAGE_FLOATS"]
STREAM_WARPS = _STREAM["NB2_STREAM_WARPS"]
STREAM_SLOTS = _STREAM["NB2_STREAM_SLOTS"]
STREAM_MAX_NEURONS = _STREAM["NB2_STREAM_MAX_NEURONS"]
STREAM_MAX_INPUT = _STREAM["NB2_STREAM_MAX_INPUT"]
STREAM_MIN_NEURONS = 256
STREAM_REC, STREAM_DITEMS, STREAM_CHUNK = 32, 16, 192


def streamable(ens, terms, conns):
    """Rows of the ensemble table that ``nb2_ensemble_stream`` can take."""
    out = []
    for i, row in enumerate(ens):
        n, nt, t0, nc, c0 = int(row[0]), int(row[6]), int(row[7]), int(row[8]), int(row[9])
        d_total = int(terms[t0:t0 + nt, 1].sum()) if nt else 0
        pes = int(conns[c0:c0 + nc, 6].sum()) if nc else 0
        ok = (row[13] & 1) and STREAM_MIN_NEURONS <= n <= STREAM_MAX_NEURONS and nt <= 4 and pes <= 1
        ok = ok and d_total <= STREAM_MAX_INPUT and 32 * (d_total + 4) <= STREAM_STAGE_FLOATS
        ok = ok and (nt == 0 or bool(np.all(terms[t0:t0 + nt, 1] % 4 == 0)))
        if ok:
            out.append(i)
    return np.asarray(out, dtype=np.int32)


def stream_records(ens, terms, conns, rows, n_ctas_max):
    """Work records and per-CTA record ranges of ``nb2_ensemble_stream``.

    Record layout (32 int32): [0] type (1 = E: a block of neurons, 2 = D: rows of
    one decoder matrix), [1] ensemble table row, [2] shared-memory slot, [5] number
    of copies, [6] the count of finished records of the other type in this slot
    that the record waits for, then per copy 3 ints at 8 + 3q: element index in the
    signal buffer, bytes, float offset in the stage.  E: [3] first neuron, [4]
    neurons, [7] connection table row of the PES connection or -1; copies = encoder
    rows of every term, bias, voltage, refractory time [, PES activity trace].
    D: [3] connection table row, [4] first row, [7] rows (rows x 128-column tiles
    <= 16); one copy; [11..18] neurons, PES flag, alpha, element index of the first
    row's error / decoded / filtered value (filtered: -1 = none), synapse b0, a0
    (float bits).  [31] (both types): total bytes of the copies.
    Ensembles are dealt to CTAs in contiguous runs balanced by bytes; the records
    of a CTA are ordered E(0), E(1), D(0), E(2), D(1), ..., D(last).
    """
    rows = [int(r) for r in rows]
    per_ens = []
    for r in rows:
        row = ens[r]
        n, nt, t0, nc, c0 = int(row[0]), int(row[6]), int(row[7]), int(row[8]), int(row[9])
        ds = [int(terms[t0 + k, 1]) for k in range(nt)]
        pes_conn = next((c0 + k for k in range(nc) if conns[c0 + k, 6]), -1)
        per_neuron = sum(ds) + 3 + (1 if pes_conn >= 0 else 0)
        # E records start on multiples of 32 neurons (one writer per word of the spike bitmap)
        ne_max = min(STREAM_CHUNK, (STREAM_STAGE_FLOATS // per_neuron) & ~31)
        n_chunks = -(-n // ne_max)
        ne_even = min(ne_max, (-(-n // n_chunks) + 31) & ~31)
        E, D = [], []
        for i0 in range(0, n, ne_even):
            ne = min(ne_even, n - i0)
            rec = np.zeros(STREAM_REC, dtype=np.int64)
            rec[0], rec[1], rec[3], rec[4], rec[7] = 1, r, i0, ne, pes_conn
            copies, off = [], 0
            for k, d in enumerate(ds):
                copies.append((int(terms[t0 + k, 0]) + i0 * d, 4 * ne * d, off))
                off += ne * d
            vecs = [int(row[5]), int(row[2]), int(row[3])] + ([int(conns[pes_conn, 8])] if pes_conn >= 0 else [])
            for start in vecs:
                copies.append((start + i0, 4 * ne, off))
                off += ne
            assert off <= STREAM_STAGE_FLOATS and len(copies) <= 8
            rec[5] = len(copies)
            for q, cp in enumerate(copies):
                rec[8 + 3 * q:11 + 3 * q] = cp
            rec[31] = sum(cp[1] for cp in copies)  # bytes the stage's barrier expects
            E.append(rec)
        # a D record holds at most STREAM_DITEMS (row, 128-column tile) pairs: two lanes each
        nr_max = max(1, min(STREAM_DITEMS // (-(-n // 128)), STREAM_STAGE_FLOATS // n))
        for k in range(nc):
            d_c = int(conns[c0 + k, 1])
            for r0 in range(0, d_c, nr_max):
                nr = min(nr_max, d_c - r0)
                rec = np.zeros(STREAM_REC, dtype=np.int64)
                rec[0], rec[1], rec[3], rec[4], rec[5], rec[7] = 2, r, c0 + k, r0, 1, nr
                rec[8:11] = (int(conns[c0 + k, 0]) + r0 * n, 4 * nr * n, 0)
                # what the record needs from the connection table, so that the kernel reads it from
                # shared memory: neurons, PES flag, alpha, error / decoded / filtered element of the
                # first row, synapse coefficients
                crow = conns[c0 + k]
                rec[11:19] = (n, int(crow[6]), int(crow[11]), int(crow[7]) + r0, int(crow[2]) + r0,
                              int(crow[3]) + r0 if crow[3] >= 0 else -1, int(crow[4]), int(crow[5]))
                rec[31] = 4 * nr * n
                D.append(rec)
        nbytes = 4 * n * (sum(ds) + 5) + sum(4 * int(conns[c0 + k, 1]) * n * (2 if conns[c0 + k, 6] else 1)
                                              for k in range(nc))
        per_ens.append((E, D, nbytes))
    if not per_ens:
        return np.zeros((0, STREAM_REC), np.int32), np.zeros((0, 2), np.int32)
    cost = np.array([b for _, _, b in per_ens], dtype=np.float64)
    n_ctas = int(min(len(per_ens), n_ctas_max))
    csum = np.cumsum(cost)
    cut = np.unique(np.concatenate([[0], np.searchsorted(csum, csum[-1] * np.arange(1, n_ctas) / n_ctas) + 1,
                                    [len(per_ens)]]))
    cut = cut[cut <= len(per_ens)]
    blocks, ranges, pos = [], [], 0
    for a, b in zip(cut[:-1], cut[1:]):
        mine = per_ens[a:b]
        e_cum = [0] * STREAM_SLOTS
        d_cum = [0] * STREAM_SLOTS
        seq = []
        for g, (E, D, _) in enumerate(mine):
            slot = g % STREAM_SLOTS
            for rec in E:
                rec[2], rec[6] = slot, d_cum[slot]  # the slot's previous ensemble must be decoded
            e_cum[slot] += len(E)
            for rec in D:
                rec[2], rec[6] = slot, e_cum[slot]  # all spikes of this ensemble must be there
            d_cum[slot] += len(D)
        for g, (E, D, _) in enumerate(mine):  # E(g) goes before D(g - 1)
            seq.extend(E)
            if g > 0:
                seq.extend(mine[g - 1][1])
        seq.extend(mine[-1][1])
        block = np.asarray(seq, dtype=np.int64).reshape(-1, STREAM_REC)
        blocks.append(block)
        ranges.append((pos, pos + len(block)))
        pos += len(block)
    records = np.concatenate(blocks, axis=0)
    assert records.max() < 2 ** 31
    return records.astype(np.int32), np.asarray(ranges, dtype=np.int32)


def stream_push_runs(ens, conns, records, ranges, lo, hi):
    """Per CTA of the streamed kernel, the run {first element, length} of the signal-
    buffer range [lo, hi) that the filtered outputs of its ensembles' connections
    fill, or None unless every CTA's outputs in that range are one contiguous run
    and the runs tile the range (then the kernel can push the range to the other
    GPUs itself, each CTA its own run)."""
    runs = np.zeros((len(ranges), 2), dtype=np.int32)
    covered = np.zeros(max(hi - lo, 0), dtype=bool)
    for b, (r0, r1) in enumerate(ranges):
        spans = []
        for r in np.unique(records[r0:r1, 1]):
            c0, nc = int(ens[r, 9]), int(ens[r, 8])
            for crow in conns[c0:c0 + nc]:
                if crow[3] >= 0:
                    a, e = max(int(crow[3]), lo), min(int(crow[3]) + int(crow[1]), hi)
                    if a < e:
                        spans.append((a, e))
        if not spans:
            runs[b] = (lo, 0)
            continue
        spans.sort()
        if any(e0 != a1 for (_, e0), (a1, _) in zip(spans, spans[1:])):
            return None  # gaps or overlaps inside one CTA's outputs
        first, last = spans[0][0], spans[-1][1]
        if covered[first - lo:last - lo].any():
            return None
        covered[first - lo:last - lo] = True
        runs[b] = (first, last - first)
    return runs if hi > lo and covered.all() else None


def plan_fused_ensembles(sim, ops):
    (fused,) = ops
    members = fused.members
    queue = sim.queue
    ens, terms, conns = fused_tables(sim, members)
    n_all = np.array([mem["n"] for mem in members])
    streamed = streamable(ens, terms, conns) if getattr(sim, "stream_ensembles", True) else np.zeros(0, np.int32)
    rest = np.setdiff1d(np.arange(len(members)), streamed)
    small = rest[n_all[rest] <= SMALL_NEURONS // 2].astype(np.int32)
    large = rest[n_all[rest] > SMALL_NEURONS // 2].astype(np.int32)
    n_ctas_max = getattr(queue.device, "sm_count", 148)
    records, ranges = stream_records(ens, terms, conns, streamed, n_ctas_max)
    d_records = to_device(queue, records) if len(records) else None
    d_ranges = to_device(queue, ranges) if len(ranges) else None
    status = zeros(queue, (1,), np.int32)
    d_ens, d_terms, d_conns = to_device(queue, ens), to_device(queue, terms), to_device(queue, conns)
    if len(terms) == 0:
        d_terms = to_device(queue, np.zeros((1, 4), np.int32))
    if len(conns) == 0:
        d_conns = to_device(queue, np.zeros((1, 16), np.int32))
    d_small = to_device(queue, small) if len(small) else None
    d_large = to_device(queue, large) if len(large) else None
    data = sim.all_data.cl_buf
    fn, check, dt = _capi.lib().nb2_ensemble_step, _capi.check, float(sim.model.dt)
    fn_stream = _capi.lib().nb2_ensemble_stream
    p = lambda a: None if a is None else a.ptr
    args = (len(large), p(d_large), len(small), p(d_small), d_ens.ptr, d_terms.ptr, d_conns.ptr, data.ptr, dt)
    # Multi-GPU: if every element of this rank's segment of the exchange signal is the filtered
    # output of a streamed connection, the streamed kernel pushes it to the peers itself.
    xdesc = None
    exch = getattr(sim, "_exchange", None)
    if exch is not None and exch.world > 1 and len(streamed):
        lo = sim._exchange_start + exch.rank * exch.seg
        runs = stream_push_runs(ens, conns, records, ranges, lo, lo + exch.seg)
        if runs is not None:
            d_runs = to_device(queue, runs)
            xdesc = exch.descriptor(sim._exchange_start, d_runs)
    import ctypes

    stream_args = (p(d_records), len(records), p(d_ranges), len(ranges), d_ens.ptr, d_terms.ptr, d_conns.ptr,
                   data.ptr, dt, status.ptr, ctypes.byref(xdesc) if xdesc is not None else None)
    n_rest, n_streamed = len(large) + len(small), len(streamed)

    def launch(stream):
        if n_streamed:
            check(fn_stream(stream, *stream_args))
        if n_rest:
            check(fn(stream, *args))

    plan = Plan(queue, launch, (256, max(len(large), 1) + (len(small) + 7) // 8), lsize=(256, 1),
                n_launches=int(len(large) > 0) + int(len(small) > 0) + int(n_streamed > 0),
                name="fused_ensemble_step", tag="%d ensembles" % len(members))
    if not n_streamed:  # (the streamed kernel owns its CTAs for a whole step: no phase form)
        plan.phase = _capi.phase("ensemble_step", *args)
    plan.full_args = (d_ens, d_terms, d_conns, d_small, d_large, d_records, d_ranges, status, data, xdesc)
    plan.fused_push = xdesc is not None
    plan.tables = dict(ens=ens, terms=terms, conns=conns, small=small, large=large, streamed=streamed,
                       records=records, ranges=ranges)
    plan.status = status
    plan.bw_per_call = fused_bytes_per_step(members)
    n_neurons = int(n_all.sum())
    plan.flops_per_call = sum(2 * mem["n"] * sum(A.shape[1] for A, _ in mem["enc_terms"])
                              + sum((4 if c["pes"] else 2) * c["d"] * mem["n"] for c in mem["conns"])
                              for mem in members)
    plan.description = "ensembles: %d; neurons: %d; connections: %d (PES: %d)" % (
        len(members), n_neurons, len(conns), int(sum(c[6] for c in conns.tolist())) if len(conns) else 0)
    return [plan]


# ---- reset + whole-signal increments -> one gather-sum ---------------------------
class GatherSum(Operator):
    """``dst[part] = sum(srcs of part)`` for every part of ``dst``: a signal that is
    reset to zero and then only incremented by copies into the whole signal or into
    non-overlapping contiguous slices of it.  ``parts`` = [(offset, size, [srcs])];
    a part without sources is just zeroed."""

    def __init__(self, dst, parts, ops):
        n_src = sum(len(srcs) for _, _, srcs in parts)
        Operator.__init__(self, tag="gather-%d" % n_src)
        self.dst, self.parts, self.ops = dst, list(parts), list(ops)
        self.srcs = [s for _, _, srcs in parts for s in srcs]
        self.sets = [dst]
        self.reads = list(self.srcs)


def _contiguous_1d(sig):
    return sig.ndim <= 1 and (sig.size <= 1 or sig.elemstrides[-1] == 1)


def find_gather_sums(operators):
    """Signals written only by ``Reset(0)`` and un-indexed ``Copy(inc=True)`` ops whose
    targets are the signal itself or contiguous slices of it that do not overlap
    each other partially (several copies into the same slice are summed)."""
    writers = {}
    for op in operators:
        for kind in ("sets", "incs", "updates"):
            for s in getattr(op, kind):
                writers.setdefault(s.base, []).append((op, kind, s))
    order = {op: i for i, op in enumerate(operators)}
    gathers, consumed = [], set()
    for base, ws in writers.items():
        if base.is_view or len(ws) < 2 or base.ndim > 1:
            continue
        resets = [op for op, kind, s in ws if _is_type(op, "Reset") and s is base and op.value == 0]
        copies = [(op, s) for op, kind, s in ws if _is_type(op, "Copy") and kind == "incs"
                  and op.src_slice is None and op.dst_slice is None and op.src.size == s.size
                  and _contiguous_1d(op.src) and _contiguous_1d(s)]
        if len(resets) != 1 or len(resets) + len(copies) != len(ws):
            continue
        by_extent = {}
        for op, s in sorted(copies, key=lambda c: order[c[0]]):  # operator order = summation order
            by_extent.setdefault((s.elemoffset, s.size), []).append(op)
        extents = sorted(by_extent)
        if any(a0 + an > b0 for (a0, an), (b0, _) in zip(extents, extents[1:])):
            continue  # partially overlapping targets
        parts, pos = [], 0
        for off, size in extents:
            if off > pos:
                parts.append((pos, off - pos, []))  # nobody increments this stretch: it is only reset
            parts.append((off, size, [op.src for op in by_extent[(off, size)]]))
            pos = off + size
        if pos < base.size:
            parts.append((pos, base.size - pos, []))
        ops_used = resets + [op for op, _ in copies]
        gathers.append(GatherSum(base, parts, ops_used))
        consumed.update(ops_used)
    return gathers, consumed


def plan_gather_sums(sim, ops):
    """One launch for all gather-sums of a group (csrc: nb2_gather_sum)."""
    starts, sidx = sim.all_data.starts, sim.sidx
    blocks, srcs = [], []
    n_bytes = 0
    for op in ops:
        d0 = int(starts[sidx[op.dst]])
        for part_off, size, part_srcs in op.parts:
            s0 = [int(starts[sidx[s]]) for s in part_srcs]
            for off in range(0, size, 256):
                blocks.append([d0 + part_off + off, min(256, size - off), len(srcs), len(s0)])
                srcs.extend(s + off for s in s0)
            n_bytes += 4 * size * (len(s0) + 1)
    queue = sim.queue
    d_blocks = to_device(queue, np.asarray(blocks, dtype=np.int32).reshape(-1, 4))
    d_srcs = to_device(queue, np.asarray(srcs + [0], dtype=np.int32))
    data = sim.all_data.cl_buf
    fn, check = _capi.lib().nb2_gather_sum, _capi.check
    width = 1  # threads per table block: the next power of two >= the longest block
    while width < max([b[1] for b in blocks] + [1]):
        width *= 2
    args = (len(blocks), width, d_blocks.ptr, d_srcs.ptr, data.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (256, max(len(blocks) * width // 256, 1)), lsize=(256, 1), name="gather_sum",
                tag="%d signals" % len(ops))
    plan.phase = _capi.phase("gather_sum", *args)
    plan.full_args = (d_blocks, d_srcs, data)
    plan.bw_per_call = n_bytes
    plan.description = "signals: %d; sources: %d" % (len(ops), len(srcs))
    return [plan]
