"""Process-group plumbing: one process per GPU, ``torch.distributed`` for the
rendezvous and for the NCCL baseline only.

The reference forks one process per GPU itself and exchanges handles through an
anonymous shared mapping (comm_comp/ipc_multiproc.cuh:105-171).  Here the ranks
are started by ``torchrun`` (or ``torch.multiprocessing``) and the store of
``torch.distributed`` carries the handles.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


numa_info: dict = {}       # what :func:`init` found and did about CPU affinity (utils/numa.py)


def env_rank_world() -> tuple[int, int, int]:
    """(rank, world, local_rank) from the launcher's environment (1 process if unset)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def init(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int, int]:
    """Initialise ``torch.distributed`` when WORLD_SIZE > 1; pick the CUDA device.

    Returns (rank, world, local_rank).  With one process nothing is initialised
    and every collective helper in this package degenerates to a no-op.
    """
    rank, world, local = env_rank_world()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % max(1, torch.cuda.device_count()))
        # host buffers this rank pins from here on land on its GPU's NUMA node (no-op where unknown)
        global numa_info
        from ..utils.numa import bind_to_gpu_node
        numa_info = bind_to_gpu_node(torch.cuda.current_device())
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if use_cuda else "gloo"
        kwargs = {}
        if backend == "nccl" and use_cuda:
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, local


def world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def all_gather_object(obj, group=None) -> list:
    if not dist.is_initialized():
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def host_barrier(group=None) -> None:
    if dist.is_initialized():
        dist.barrier(group=group)


def max_over_ranks(value: float, group=None) -> float:
    """Max of a host float over all ranks (device-timed numbers are reported as this)."""
    if not dist.is_initialized():
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


_holds = 0


def hold() -> None:
    """Keeps the process group alive across several experiments run in one process per rank: until the
    matching :func:`release`, :func:`shutdown` does nothing (and :func:`init` finds the group still up)."""
    global _holds
    _holds += 1


def release() -> None:
    global _holds
    _holds = max(0, _holds - 1)


def shutdown() -> None:
    if _holds == 0 and dist.is_initialized():
        dist.destroy_process_group()
