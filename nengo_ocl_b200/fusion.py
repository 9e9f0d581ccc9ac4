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
from nengo_ocl_b200.runtime import to_device

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
            if not conn["pes"] and w_writers:
                continue  # somebody else modifies these weights during the step
            member["conns"].append(conn)
            member["ops"].extend(conn["ops"])
        fused_here = set(member["ops"])
        member["store_spikes"] = any(op not in fused_here for op in out_readers) or any(
            sim.model.sig[p]["in"].base is out for p in sim.model.probes)
        members.append(member)
        consumed.update(member["ops"])
    return members, consumed


def fuse_ensemble_groups(sim, groups, planner=None):
    """Replace matched operators by one ``FusedEnsembles`` op and re-plan."""
    from nengo_ocl_b200.planners import greedy_planner

    planner = planner or getattr(sim, "_planner", None) or greedy_planner
    operators = sim.operators
    members, consumed = find_fusable(sim, operators)
    gathers, gathered = find_gather_sums([op for op in operators if op not in consumed])
    if not members and not gathers:
        return groups
    consumed = set(consumed) | gathered
    new_ops = [op for op in operators if op not in consumed] + gathers
    if members:
        new_ops.append(FusedEnsembles(members))
    try:
        new_groups = planner(new_ops)
    except ValueError:
        return groups  # merging would create a same-step dependency cycle: stay un-fused
    sim.operators = new_ops
    sim.fused_groups = [dict(pes=any(c["pes"] for c in mem["conns"]), n=mem["n"],
                             unstored=[mem["J"]] + ([] if mem["store_spikes"] else [mem["out"]])
                             + [c["delta"] for c in mem["conns"] if c["pes"]]) for mem in members]
    return new_groups


def _fbits(x):
    return int(np.float32(x).view(np.int32))


def fused_tables(sim, members):
    """int32 tables of ``nb2_ensemble_step`` (layouts in include/nengo_b200.h)."""
    starts = sim.all_data.starts
    sidx = sim.sidx
    st = lambda sig: int(starts[sidx[sig]])
    ens, terms, conns = [], [], []
    for mem in members:
        nt = mem["neurons"].neurons
        row = [mem["n"], -1, st(mem["state"][0]), st(mem["state"][1]), st(mem["out"]) if mem["store_spikes"] else -1,
               st(mem["bias"]), len(mem["enc_terms"]), len(terms), len(mem["conns"]), len(conns),
               _fbits(nt.tau_rc), _fbits(nt.tau_ref), _fbits(nt.amplitude), 0, 0, 0]
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


def plan_fused_ensembles(sim, ops):
    (fused,) = ops
    members = fused.members
    queue = sim.queue
    ens, terms, conns = fused_tables(sim, members)
    n_all = np.array([mem["n"] for mem in members])
    small = np.flatnonzero(n_all <= SMALL_NEURONS // 2).astype(np.int32)
    large = np.flatnonzero(n_all > SMALL_NEURONS // 2).astype(np.int32)
    d_ens, d_terms, d_conns = to_device(queue, ens), to_device(queue, terms), to_device(queue, conns)
    if len(terms) == 0:
        d_terms = to_device(queue, np.zeros((1, 4), np.int32))
    if len(conns) == 0:
        d_conns = to_device(queue, np.zeros((1, 16), np.int32))
    d_small = to_device(queue, small) if len(small) else None
    d_large = to_device(queue, large) if len(large) else None
    data = sim.all_data.cl_buf
    fn, check, dt = _capi.lib().nb2_ensemble_step, _capi.check, float(sim.model.dt)
    p = lambda a: None if a is None else a.ptr
    args = (len(large), p(d_large), len(small), p(d_small), d_ens.ptr, d_terms.ptr, d_conns.ptr, data.ptr, dt)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (256, max(len(large), 1) + (len(small) + 7) // 8), lsize=(256, 1),
                n_launches=int(len(large) > 0) + int(len(small) > 0), name="fused_ensemble_step",
                tag="%d ensembles" % len(members))
    plan.full_args = (d_ens, d_terms, d_conns, d_small, d_large, data)
    plan.tables = dict(ens=ens, terms=terms, conns=conns, small=small, large=large)
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
    """``dst = sum(srcs)``: a signal that is reset to zero and then only
    incremented by whole-signal copies."""

    def __init__(self, dst, srcs, ops):
        Operator.__init__(self, tag="gather-%d" % len(srcs))
        self.dst, self.srcs, self.ops = dst, list(srcs), list(ops)
        self.sets = [dst]
        self.reads = list(srcs)


def find_gather_sums(operators):
    """Signals written only by ``Reset(0)`` and un-sliced ``Copy(inc=True)`` ops."""
    writers = {}
    for op in operators:
        for kind in ("sets", "incs", "updates"):
            for s in getattr(op, kind):
                writers.setdefault(s.base, []).append((op, kind, s))
    order = {op: i for i, op in enumerate(operators)}
    gathers, consumed = [], set()
    for base, ws in writers.items():
        if base.is_view or len(ws) < 2:
            continue
        resets = [op for op, kind, s in ws if _is_type(op, "Reset") and s is base and op.value == 0]
        copies = [op for op, kind, s in ws if _is_type(op, "Copy") and kind == "incs" and s is base
                  and op.src_slice is None and op.dst_slice is None and op.src.size == base.size
                  and (op.src.ndim <= 1 and (op.src.size <= 1 or op.src.elemstrides[-1] == 1))]
        if len(resets) != 1 or len(resets) + len(copies) != len(ws) or base.ndim > 1:
            continue
        ordered = sorted(copies, key=order.get)  # operator order = summation order
        gathers.append(GatherSum(base, [op.src for op in ordered], resets + ordered))
        consumed.update(resets + ordered)
    return gathers, consumed


def plan_gather_sums(sim, ops):
    """One launch for all gather-sums of a group (csrc: nb2_gather_sum)."""
    starts, sidx = sim.all_data.starts, sim.sidx
    blocks, srcs = [], []
    n_bytes = 0
    for op in ops:
        d0, size = int(starts[sidx[op.dst]]), op.dst.size
        s0 = [int(starts[sidx[s]]) for s in op.srcs]
        for off in range(0, size, 256):
            blocks.append([d0 + off, min(256, size - off), len(srcs), len(s0)])
            srcs.extend(s + off for s in s0)
        n_bytes += 4 * size * (len(s0) + 1)
    queue = sim.queue
    d_blocks = to_device(queue, np.asarray(blocks, dtype=np.int32).reshape(-1, 4))
    d_srcs = to_device(queue, np.asarray(srcs + [0], dtype=np.int32))
    data = sim.all_data.cl_buf
    fn, check = _capi.lib().nb2_gather_sum, _capi.check
    args = (len(blocks), d_blocks.ptr, d_srcs.ptr, data.ptr)

    def launch(stream):
        check(fn(stream, *args))

    plan = Plan(queue, launch, (256, max(len(blocks), 1)), lsize=(256, 1), name="gather_sum",
                tag="%d signals" % len(ops))
    plan.full_args = (d_blocks, d_srcs, data)
    plan.bw_per_call = n_bytes
    plan.description = "signals: %d; sources: %d" % (len(ops), len(srcs))
    return [plan]
