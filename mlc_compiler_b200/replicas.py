"""Multi-GPU execution: independent replicas, batch split across ranks.

The compiled path is a single-device inference graph in which the batch is an
outer, fully independent dimension: no fused kernel reduces across samples and
nothing is exchanged between devices (the reference has no distributed code at
all).  Scaling out therefore means one process per GPU, each with its own
weights, its own schedule compiled for its share of the batch, its own arena
and CUDA graph.  The only cross-rank traffic is control: a barrier, the
max/sum of timings, and -- when the caller wants the full result on one rank --
a gather of output shards.  There is no collective on the data path.

Works with any ``torch.distributed`` backend (``nccl`` on GPUs, ``gloo`` on
CPU hosts) and degenerates to a no-op in a single process.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Sequence

import torch


def shard_bounds(global_batch: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, equal shards.  Shapes are static per compiled schedule, so a
    ragged split would need a second schedule; it is refused instead."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} does not split evenly over {world} replicas")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def shard_inputs(inputs: Sequence[torch.Tensor], world: int, rank: int) -> list[torch.Tensor]:
    """This rank's slice of every batched input (dimension 0)."""
    out = []
    for t in inputs:
        lo, hi = shard_bounds(t.shape[0], world, rank)
        out.append(t[lo:hi])
    return out


@dataclass
class ReplicaGroup:
    rank: int = 0
    world: int = 1
    local_rank: int = 0

    @classmethod
    def from_env(cls, backend: str | None = None, device: torch.device | None = None):
        """Join the process group described by RANK / WORLD_SIZE / LOCAL_RANK /
        MASTER_ADDR / MASTER_PORT (as set by ``torch.distributed.run``)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if world > 1:
            import torch.distributed as dist

            if not dist.is_initialized():
                backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
                kw = {}
                if backend == "nccl" and device is not None:
                    kw["device_id"] = device
                dist.init_process_group(backend, **kw)
        return cls(rank, world, local)

    # -- control-plane reductions ---------------------------------------------
    def _reduce(self, value: float, op: str, device) -> float:
        if self.world == 1:
            return float(value)
        import torch.distributed as dist

        t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM,
                               "min": dist.ReduceOp.MIN}[op])
        return float(t.item())

    def max(self, value: float, device=None) -> float:
        return self._reduce(value, "max", device)

    def sum(self, value: float, device=None) -> float:
        return self._reduce(value, "sum", device)

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()

    def gather_outputs(self, shard: torch.Tensor) -> torch.Tensor | None:
        """Concatenate every rank's output shard on rank 0 in rank order (the
        order the batch was split in); other ranks get ``None``."""
        if self.world == 1:
            return shard
        import torch.distributed as dist

        shard = shard.contiguous()
        parts = [torch.empty_like(shard) for _ in range(self.world)] if self.rank == 0 else None
        if dist.get_backend() == "nccl":
            # gather is a control-plane convenience here, not a data-path step
            all_parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(all_parts, shard)
            parts = all_parts if self.rank == 0 else None
        else:
            dist.gather(shard, parts, dst=0)
        return torch.cat(parts, dim=0) if self.rank == 0 else None

    def close(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()


def split_throughput(group: ReplicaGroup, global_batch: int, ms_per_forward: float,
                     device=None) -> dict:
    """Whole-job figures for one batch split over the replicas: the batch is done
    when the slowest rank is, so sequences/s = global batch / the slowest rank's
    time (not the sum of each rank's own rate, which would credit fast ranks for
    time they spend waiting)."""
    if global_batch % group.world:
        raise ValueError(f"global batch {global_batch} does not split evenly over "
                         f"{group.world} replicas")
    slow = group.max(ms_per_forward, device)
    return {"global_batch": global_batch, "per_gpu_batch": global_batch // group.world,
            "seq_per_s": global_batch / (slow / 1e3), "ms_per_forward": slow}


def run_replica(group: ReplicaGroup, inputs: Sequence[torch.Tensor],
                runner: Callable[..., torch.Tensor]) -> torch.Tensor | None:
    """Split ``inputs`` along the batch, run this rank's share through ``runner``
    and gather the result on rank 0."""
    mine = shard_inputs(inputs, group.world, group.rank)
    return group.gather_outputs(runner(*mine))
