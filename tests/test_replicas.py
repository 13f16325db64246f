"""Multi-rank host logic on CPU: two gloo ranks split a batch, run their shares
independently, and agree on the aggregates.  No collective touches the data
path; the gather only reassembles outputs for the check."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from mlc_compiler_b200 import replicas


def test_shard_bounds_are_contiguous_and_cover_the_batch():
    for world in (1, 2, 4, 8):
        spans = [replicas.shard_bounds(32, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 32
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert {hi - lo for lo, hi in spans} == {32 // world}
    with pytest.raises(ValueError, match="evenly"):
        replicas.shard_bounds(32, 3, 0)
    with pytest.raises(ValueError):
        replicas.shard_bounds(32, 2, 2)


def test_single_process_group_is_a_no_op():
    g = replicas.ReplicaGroup()
    x = torch.arange(6.0).reshape(3, 2)
    assert g.max(1.5) == 1.5 and g.sum(2.0) == 2.0
    assert torch.equal(g.gather_outputs(x), x)
    out = replicas.run_replica(g, [x], lambda t: t * 2)
    assert torch.equal(out, x * 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    group = replicas.ReplicaGroup.from_env(backend="gloo")
    try:
        torch.manual_seed(0)
        ids = torch.randint(0, 1000, (8, 16))
        mask = torch.ones(8, 16)

        def runner(i, m):       # stands in for a compiled replica
            return (i.float() * m).sum(-1, keepdim=True) + 0.0 * group.rank

        out = replicas.run_replica(group, [ids, mask], runner)
        ms = 2.0 + rank         # rank 1 is the slow one
        agg = replicas.split_throughput(group, 8, ms)
        group.barrier()
        results[rank] = {"out": None if out is None else out.clone(), "agg": agg,
                         "want": (ids.float() * mask).sum(-1, keepdim=True)}
    finally:
        group.close()


def test_two_gloo_ranks_split_a_batch_and_aggregate():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        r0, r1 = results[0], results[1]
    assert r1["out"] is None
    assert torch.equal(r0["out"], r0["want"])            # shards reassembled in rank order
    for r in (r0, r1):
        assert r["agg"]["global_batch"] == 8 and r["agg"]["per_gpu_batch"] == 4
        assert r["agg"]["ms_per_forward"] == 3.0          # the slowest rank
        assert abs(r["agg"]["seq_per_s"] - 8 / 3e-3) < 1e-6   # the batch is done with its last shard
