"""Rank bootstrap for multi-GPU sessions: one process per GPU over torch.distributed.

Replaces the reference's ``NcclContext`` bootstrap (MPI ``MPI_Bcast`` of the NCCL
unique id or a hand-rolled TCP rendezvous, onnxruntime/contrib_ops/cuda/collective/
nccl_kernels.cc:59-245).  The environment contract is kept: ``LOCAL_RANK`` /
``LOCAL_WORLD_SIZE`` (the reference's names) as well as torchrun's ``RANK`` /
``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT`` are honoured.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistInfo:
    """What a session needs to know about its process group."""
    group_name: str
    rank: int
    world_size: int
    local_rank: int = 0


def env_rank_world() -> tuple:
    rank = int(os.environ.get("RANK", os.environ.get("LOCAL_RANK", "0")))
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("LOCAL_WORLD_SIZE", "1")))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def init_distributed(backend: Optional[str] = None, timeout_s: int = 600) -> DistInfo:
    """Join (or create) the default process group and return its description.

    ``backend`` defaults to ``nccl`` when CUDA is available and ``gloo`` otherwise (CPU ranks)."""
    rank, world, local = env_rank_world()
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", os.environ.get("RANK0_IP", "127.0.0.1"))
        os.environ.setdefault("MASTER_PORT", os.environ.get("RANK0_PORT", "18888"))
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return DistInfo(dist.group.WORLD.group_name, dist.get_rank(), dist.get_world_size(), local)


def single_process() -> DistInfo:
    return DistInfo("", 0, 1, 0)
