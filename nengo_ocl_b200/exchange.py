"""Host side of the per-step exchange between the GPUs of one box.

One process per GPU.  The model is sharded by ensemble block; the shards share
one ``exchange`` signal (same layout on every rank) of which each rank owns a
contiguous segment (see ``synth.pes_learning_shard``).  ``Exchange`` allocates
the staging buffers and flags, swaps their IPC handles through a communicator
and provides two plans for the simulator's step list: ``wait`` (first plan of a
step) and ``push`` (last plan of a step), both plain kernel launches that are
captured in the step's CUDA graph (csrc/nb2_exchange.cu).

The communicator only needs ``rank``, ``world``, ``all_gather_object(obj)`` and
``barrier()``; ``TorchComm`` wraps ``torch.distributed`` (NCCL or gloo), and
``LocalComm`` is the single-process case.  The reference has no multi-device
code (nengo_ocl/simulator.py:215-219), so none of this has a counterpart there.
"""

import ctypes

import numpy as np

from nengo_ocl_b200 import _capi
from nengo_ocl_b200.plan import Plan
from nengo_ocl_b200.runtime import DeviceArray, to_device, zeros


class LocalComm:
    rank, world = 0, 1

    def all_gather_object(self, obj):
        return [obj]

    def barrier(self):
        pass


class TorchComm:
    """``torch.distributed`` as the control plane (handles, barriers); the data
    path is the push kernel, not a collective."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_gather_object(self, obj):
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self.group)
        return out

    def barrier(self):
        self.dist.barrier(group=self.group)


def shard_ranges(n_items, world):
    """Contiguous, equal blocks of items per rank (``n_items`` multiple of ``world``)."""
    assert n_items % world == 0
    per = n_items // world
    return [(r * per, (r + 1) * per) for r in range(world)]


class Exchange:
    """Device buffers and plans of the exchange for one rank.

    Parameters
    ----------
    queue : CommandQueue
    comm : communicator (``rank``, ``world``, ``all_gather_object``, ``barrier``)
    replica_ptr : int
        Device address of element 0 of the exchange signal inside the packed
        signal buffer.
    seg : int
        Floats per rank segment (the signal has ``world * seg`` floats).
    timeout_s : float
        Limit of one wait; afterwards ``status()`` is ``NB2_ERR_TIMEOUT``.
    """

    def __init__(self, queue, comm, replica_ptr, seg, timeout_s=2.0):
        self.queue, self.comm = queue, comm
        self.rank, self.world, self.seg = comm.rank, comm.world, int(seg)
        self.replica_ptr = int(replica_ptr)
        self.timeout_s = float(timeout_s)
        self.ctl = zeros(queue, (8,), np.int32)
        self.flags = zeros(queue, (max(self.world, 1),), np.int32)
        self.staging = zeros(queue, (2 * self.world * self.seg,), np.float32)
        self._opened = []
        self.fused_push = False
        self.peer_staging = self.peer_flags = None
        if self.world > 1:
            self._connect()

    def _connect(self):
        def handle(arr):
            buf = ctypes.create_string_buffer(64)
            _capi.call("nb2_ipc_get_handle", arr.ptr, buf)
            return buf.raw

        mine = (handle(self.staging), handle(self.flags))
        everyone = self.comm.all_gather_object(mine)
        staging_ptrs = np.zeros(self.world, dtype=np.uint64)
        flag_ptrs = np.zeros(self.world, dtype=np.uint64)
        for p, (hs, hf) in enumerate(everyone):
            if p == self.rank:
                continue
            ps, pf = ctypes.c_void_p(), ctypes.c_void_p()
            _capi.call("nb2_ipc_open_handle", ctypes.create_string_buffer(hs, 64), ctypes.byref(ps))
            _capi.call("nb2_ipc_open_handle", ctypes.create_string_buffer(hf, 64), ctypes.byref(pf))
            self._opened += [ps, pf]
            staging_ptrs[p], flag_ptrs[p] = ps.value, pf.value
        # device arrays of pointers (uploaded as pairs of int32 words)
        self.peer_staging = to_device(self.queue, staging_ptrs.view(np.int32))
        self.peer_flags = to_device(self.queue, flag_ptrs.view(np.int32))
        self.comm.barrier()

    # -- plans ------------------------------------------------------------------
    def descriptor(self, x_base, cta_runs):
        """``nb2_exchange_desc`` for a compute kernel that pushes this rank's segment
        itself (``x_base``: element index of the exchange signal in the signal buffer;
        ``cta_runs``: device array, per CTA the run it pushes).  After this call
        ``plans()`` leaves the separate push kernel out."""
        assert self.world > 1
        self.fused_push = True
        self._cta_runs = cta_runs  # keep alive
        lo = int(x_base) + self.rank * self.seg
        return _capi.ExchangeDesc(self.peer_staging.ptr.value, self.peer_flags.ptr.value, self.ctl.ptr.value,
                                  cta_runs.ptr.value, int(x_base), lo, lo + self.seg, self.rank, self.world,
                                  self.seg)

    def plans(self):
        """(wait plan, push plan); empty lists for a single rank, no push plan when the
        push is folded into the compute kernel."""
        if self.world == 1:
            return [], []
        lib, check = _capi.lib(), _capi.check
        replica = ctypes.c_void_p(self.replica_ptr)
        wait_args = (self.ctl.ptr, self.flags.ptr, self.staging.ptr, replica, self.rank, self.world, self.seg,
                     self.timeout_s)
        push_args = (self.ctl.ptr, self.peer_staging.ptr, self.peer_flags.ptr, replica, self.rank, self.world,
                     self.seg)

        def wait(stream):
            check(lib.nb2_exchange_wait(stream, *wait_args))

        def push(stream):
            check(lib.nb2_exchange_push(stream, *push_args))

        nbytes = 4 * self.seg * (self.world - 1)
        pw = Plan(self.queue, wait, (256, 1), name="exchange_wait", tag="%d peers" % (self.world - 1),
                  bw_per_call=2 * nbytes)
        pp = Plan(self.queue, push, (256, 1), name="exchange_push", tag="%d peers" % (self.world - 1),
                  bw_per_call=nbytes + 4 * self.seg)
        pw.full_args = pp.full_args = (self.ctl, self.flags, self.staging, self.peer_staging, self.peer_flags)
        return [pw], ([] if self.fused_push else [pp])

    def status(self):
        """0, or NB2_ERR_TIMEOUT if a wait gave up since the last reset."""
        return int(self.ctl.get()[2])

    def epoch(self):
        return int(self.ctl.get()[0])

    def reset(self):
        """Back to step 0 on every rank (collective: all ranks must call it)."""
        self.queue.finish()
        self.comm.barrier()
        for arr in (self.ctl, self.flags, self.staging):
            arr.fill(0)
        self.comm.barrier()

    def close(self):
        """Collective: no rank unmaps or frees while a peer may still push into it."""
        if self.world > 1 and self._opened:
            self.queue.finish()
            self.comm.barrier()
        for p in self._opened:
            try:
                _capi.lib().nb2_ipc_close_handle(p)
            except Exception:
                pass
        self._opened = []
