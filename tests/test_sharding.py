"""Sharding by ensemble block and the per-step exchange, on the CPU.

The multi-GPU path partitions the ensembles across ranks and exchanges one
segment of the `exchange` signal per rank and step.  Here the ranks are gloo
processes running the CPU oracle on their shard and exchanging segments with an
all-gather: the union of the shards must reproduce the unsharded model exactly
(the arithmetic of every ensemble is unchanged by sharding)."""

import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KW = dict(seed=5, n_ensembles=8, n_neurons=48, dimensions=4, n_templates=2, n_probes=2, sim_time=0.05)
KW_WS = dict(seed=2, n_ensembles=16, n_neurons=30, k=2, n_templates=3, n_probes=2, max_out=8)
STEPS = 25


def make_shard(kind, rank, world):
    from nengo_ocl_b200 import synth

    if kind == "pes":
        return synth.pes_learning_shard(rank=rank, world=world, **KW)
    return synth.watts_strogatz_shard(rank=rank, world=world, **KW_WS)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, kind):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from nengo_ocl_b200 import synth
    from nengo_ocl_b200.exchange import TorchComm, shard_ranges
    from oracle.simulator import OracleSimulator

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    comm = TorchComm()
    assert (comm.rank, comm.world) == (rank, world)
    assert comm.all_gather_object(("r", rank)) == [("r", r) for r in range(world)]
    mdl = make_shard(kind, rank, world)
    lo, n = mdl.info["segment"]
    if kind == "pes":
        assert (lo // KW["dimensions"], (lo + n) // KW["dimensions"]) == shard_ranges(KW["n_ensembles"], world)[rank]
    ora = OracleSimulator(mdl)
    ex = mdl.info["exchange"]
    for _ in range(STEPS):
        ora.step()
        mine = torch.from_numpy(np.ascontiguousarray(ora[ex][lo:lo + n]))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)  # the push/wait pair of the GPU path
        ora.view(ex)[...] = torch.cat(parts).numpy()
    np.save(os.path.join(out_dir, "exchange_%d.npy" % rank), ora[ex])
    np.save(os.path.join(out_dir, "probe_%d.npy" % rank), np.array(ora.probe_data[mdl.probes[0]]))
    comm.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["pes", "watts_strogatz"])
def test_two_gloo_ranks_reproduce_the_unsharded_model(tmp_path, kind):
    import torch.multiprocessing as mp

    sys.path.insert(0, ROOT)
    from oracle.simulator import OracleSimulator

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), kind), nprocs=world, join=True)
    full = make_shard(kind, 0, 1)
    ora = OracleSimulator(full)
    ora.run_steps(STEPS)
    ref = ora[full.info["exchange"]]
    assert np.abs(ref).max() > 0.01
    for r in range(world):
        got = np.load(tmp_path / ("exchange_%d.npy" % r))
        assert np.array_equal(got, ref)
    # probe 0 of rank 0 is the first probe of the full model too (connection / ensemble 0)
    assert np.array_equal(np.load(tmp_path / "probe_0.npy"), np.array(ora.probe_data[full.probes[0]]))


def test_shard_structure():
    sys.path.insert(0, ROOT)
    from nengo_ocl_b200 import synth

    shards = [synth.pes_learning_shard(rank=r, world=4, **KW) for r in range(4)]
    full = synth.pes_learning_shard(rank=0, world=1, **KW)
    assert sum(s.n_neurons for s in shards) == full.n_neurons
    assert all(np.array_equal(s.info["targets"], full.info["targets"]) for s in shards)
    segs = [s.info["segment"] for s in shards]
    assert [lo for lo, _ in segs] == [0, 8, 16, 24] and all(n == 8 for _, n in segs)
    # every connection is instantiated exactly once across the shards
    labels = sorted(c["label"] for s in shards for c in s.info["connections"])
    assert labels == sorted(c["label"] for c in full.info["connections"])
    with pytest.raises(AssertionError):
        synth.pes_learning_shard(rank=0, world=3, **KW)


def test_stream_push_runs():
    """The streamed kernel may push a rank's segment only if every CTA's outputs are one run
    and the runs tile the segment."""
    from nengo_ocl_b200 import fusion

    ens = np.zeros((3, 16), np.int32)
    conns = np.zeros((4, 16), np.int32)
    # ensemble r has connection r (ensemble 2 has two): conn table row = [W, d, weighted, filtered, ...]
    ens[:, 8], ens[:, 9] = [1, 1, 2], [0, 1, 2]
    conns[:, 1] = 4
    conns[:, 3] = [100, 104, 108, -1]  # the last connection has no synapse output
    rec = lambda rows: np.array([[1, r] + [0] * 30 for r in rows], np.int32)
    two_ctas = (rec([0, 0, 1, 2]), np.array([[0, 3], [3, 4]], np.int32))  # CTA 0: ensembles 0, 1; CTA 1: 2
    runs = fusion.stream_push_runs(ens, conns, *two_ctas, 100, 112)
    assert runs.tolist() == [[100, 8], [108, 4]]
    assert fusion.stream_push_runs(ens, conns, *two_ctas, 100, 116) is None  # 112..115 unwritten
    assert fusion.stream_push_runs(ens, conns, rec([0, 2]), np.array([[0, 2]], np.int32), 100, 112) is None  # gap
    assert fusion.stream_push_runs(ens, conns, rec([1]), np.array([[0, 1]], np.int32), 104, 108).tolist() == [[104, 4]]
    # a CTA whose ensembles write outside the segment pushes nothing
    runs = fusion.stream_push_runs(ens, conns, *two_ctas, 100, 108)
    assert runs.tolist() == [[100, 8], [100, 0]]
