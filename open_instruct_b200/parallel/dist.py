"""Process-group plumbing: one process per GPU, ``torch.distributed`` over NCCL (gloo on CPU).

Replaces the accelerate / DeepSpeed launcher glue of the reference (``open_instruct/finetune.py:396-404``,
``open_instruct/grpo_fast.py:327-329``): ranks come from the ``torchrun`` environment, the rendezvous
address defaults to 127.0.0.1, and every helper degrades to a no-op in a single process.
"""

from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def find_free_port(host: str = "127.0.0.1") -> int:
    """A TCP port that is free right now (bind to port 0, read the number back).  Rendezvous ports are picked this way
    instead of from fixed numbers, which collide on machines shared with other jobs."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return int(s.getsockname()[1])


def env_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def env_world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def env_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def init_distributed(backend: str | None = None, timeout_s: float = 1800.0) -> tuple[int, int, torch.device]:
    """Initialise the default group from the environment.  Returns (rank, world, device)."""
    world = env_world_size()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(env_local_rank())
        device = torch.device("cuda", env_local_rank())
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(backend=backend, rank=env_rank(), world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return env_rank() if world > 1 else 0, world, device


class _SoloGroup:
    """A group of exactly this process: lets one rank of a larger job run a component alone
    (single-process oracles in tests, rank-0-only evaluation)."""


SOLO = _SoloGroup()


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def rank(group=None) -> int:
    return dist.get_rank(group) if is_dist() and group is not SOLO else 0


def world_size(group=None) -> int:
    return dist.get_world_size(group) if is_dist() and group is not SOLO else 1


def barrier(group=None) -> None:
    if is_dist() and group is not SOLO:
        dist.barrier(group)


def all_reduce_(t: torch.Tensor, op=None, group=None) -> torch.Tensor:
    if is_dist() and group is not SOLO:
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
    return t


def max_over_ranks(value: float, device=None) -> float:
    """MAX-reduce a host scalar (device-time measurements are reported as the slowest rank)."""
    if not is_dist():
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def broadcast_object(obj, src: int = 0, group=None):
    if not is_dist():
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def tp_groups(tp: int):
    """Tensor-parallel groups of ``tp`` consecutive ranks and the data-parallel groups across them (ranks with the same
    position inside their TP group).  Returns ``(tp_group, dp_group)`` of this rank; collective."""
    return hsdp_groups(tp)


def hsdp_groups(shard_degree: int):
    """Split the default group into shard groups of ``shard_degree`` consecutive ranks and replica groups of the ranks
    that hold the same slice (hybrid sharding: ``DataParallelType.hsdp`` with ``shard_degree`` / ``num_replicas`` in the
    reference's olmo-core path, ``open_instruct/dpo.py:270-277``).  Returns ``(shard_group, replica_group)`` of this rank;
    every rank must call it (``new_group`` is collective)."""
    world, me = world_size(), rank()
    if shard_degree <= 0 or world % shard_degree:
        raise ValueError(f"shard_degree {shard_degree} must divide the world size {world}")
    shard_group = replica_group = None
    for s0 in range(0, world, shard_degree):
        ranks = list(range(s0, s0 + shard_degree))
        g = dist.new_group(ranks)
        if me in ranks:
            shard_group = g
    for r0 in range(shard_degree):
        ranks = list(range(r0, world, shard_degree))
        g = dist.new_group(ranks)
        if me in ranks:
            replica_group = g
    return shard_group, replica_group


def destroy() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
