"""Two ranks on two GPUs: sharded model + peer-push exchange against the
unsharded CPU oracle.  Skipped when fewer than two GPUs are visible.  The
control plane is gloo; the data path is nb2_exchange_push / nb2_exchange_wait."""

import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KW = dict(seed=5, n_ensembles=8, n_neurons=256, dimensions=8, n_templates=2, n_probes=2, sim_time=0.1)
STEPS = 70  # more than two probe-drain batches, and an odd number of graph replays


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, fused_push):
    sys.path.insert(0, ROOT)
    os.environ["LOCAL_RANK"] = str(rank)
    import torch.distributed as dist

    from nengo_ocl_b200 import synth
    from nengo_ocl_b200.exchange import TorchComm
    from nengo_ocl_b200.runtime import create_some_context
    from nengo_ocl_b200.simulator import Simulator

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    mdl = synth.pes_learning_shard(rank=rank, world=world, **KW)
    comm = TorchComm()
    if not fused_push:
        Simulator.stream_ensembles = False  # per-ensemble kernel, then the separate nb2_exchange_push
    with Simulator(None, model=mdl, context=create_some_context(rank), exchange=(mdl.info["exchange"], comm)) as sim:
        assert sim.fused_groups
        assert sim._exchange.fused_push == fused_push
        assert [p.name for p in sim._plans].count("exchange_push") == (0 if fused_push else 1)
        comm.barrier()
        sim.run_steps(STEPS)
        assert sim._exchange.status() == 0 and sim._exchange.epoch() == STEPS
        np.save(os.path.join(out_dir, "exchange_%d.npy" % rank), np.asarray(sim.signals[mdl.info["exchange"]]))
        np.save(os.path.join(out_dir, "probe_%d.npy" % rank), sim.data[mdl.probes[0]])
        # a second run after reset reproduces the first bit for bit
        sim.reset()
        sim.run_steps(STEPS)
        np.save(os.path.join(out_dir, "exchange_again_%d.npy" % rank),
                np.asarray(sim.signals[mdl.info["exchange"]]))
        comm.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fused_push", [True, False], ids=["push_in_step_kernel", "separate_push_kernel"])
def test_two_gpus_match_unsharded_oracle(tmp_path, fused_push):
    from nengo_ocl_b200 import _capi
    import ctypes

    n = ctypes.c_int()
    _capi.call("nb2_device_count", ctypes.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from nengo_ocl_b200 import synth
    from oracle.simulator import OracleSimulator

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), fused_push), nprocs=world, join=True)
    full = synth.pes_learning_shard(rank=0, world=1, **KW)
    ora = OracleSimulator(full)
    ora.run_steps(STEPS)
    ref = ora[full.info["exchange"]]
    seg = ref.size // world
    for r in range(world):
        got = np.load(tmp_path / ("exchange_%d.npy" % r))
        # own segment: state after STEPS steps; peers' segments: what was received before the last
        # step, i.e. the peers' state after STEPS - 1 steps -- compare the own segment
        own = slice(r * seg, (r + 1) * seg)
        assert np.array_equal(got[own], ref[own])  # the sharded run is bit-identical to the oracle
        assert np.array_equal(got, np.load(tmp_path / ("exchange_again_%d.npy" % r)))
    p0 = np.load(tmp_path / "probe_0.npy")
    assert p0.shape == (STEPS, KW["dimensions"])
    assert np.array_equal(p0, np.array(ora.probe_data[full.probes[0]], dtype=p0.dtype))


def test_wait_gives_up_and_reports(queue):
    """A flag that nothing sets: the wait runs out after its limit, records the
    status, leaves the replica untouched and the context usable."""
    import ctypes

    from nengo_ocl_b200 import _capi
    from nengo_ocl_b200.runtime import to_device, zeros

    world, seg = 2, 64
    ctl = to_device(queue, np.array([1, 0, 0, 0, 0, 0, 0, 0], dtype=np.int32))  # epoch 1: one step was pushed
    flags = zeros(queue, (world,), np.int32)
    staging = to_device(queue, np.full(2 * world * seg, 7.0, dtype=np.float32))
    replica = to_device(queue, np.arange(world * seg, dtype=np.float32))
    _capi.call("nb2_exchange_wait", queue.stream, ctl.ptr, flags.ptr, staging.ptr, replica.ptr, 0, world, seg,
               ctypes.c_double(0.05))
    queue.finish()
    assert ctl.get()[2] == _capi.NB2_ERR_TIMEOUT
    assert np.array_equal(replica.get(), np.arange(world * seg, dtype=np.float32))
    # the same call with the flag published copies the peer's segment
    ctl.set(np.array([1, 0, 0, 0, 0, 0, 0, 0], dtype=np.int32))
    flags.set(np.array([0, 1], dtype=np.int32))
    _capi.call("nb2_exchange_wait", queue.stream, ctl.ptr, flags.ptr, staging.ptr, replica.ptr, 0, world, seg,
               ctypes.c_double(0.05))
    queue.finish()
    got = replica.get()
    assert ctl.get()[2] == 0
    assert np.array_equal(got[:seg], np.arange(seg, dtype=np.float32)) and np.all(got[seg:] == 7.0)
