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


class RankLeft(RuntimeError):
    """A peer announced that it is leaving (or stopped refreshing its heartbeat): no further collective may start."""


class RankMonitor:
    """Host-side failure detection between steps, over a key-value store every rank can reach.

    The reference has nothing of the kind: its custom all-reduce barriers spin for ever
    (onnxruntime/contrib_ops/cuda/collective/custom_reduce_impl.cu:113-135), so a dead peer hangs the GPU.  Here the
    device-side waits are bounded, and this class keeps a rank from launching into a group that is no longer complete:
    a rank calls ``leave()`` between steps (never with kernels or collectives in flight), and every rank calls
    ``check()`` before its next launch.  ``beat()`` / ``max_silence_s`` add a heartbeat for ranks that die without
    saying so.  The store is the one torch.distributed was initialised with, or any ``torch.distributed.Store``.
    """

    def __init__(self, rank: int, world_size: int, store=None, max_silence_s: float = 0.0, prefix: str = "ortb200/monitor"):
        import time
        self.rank, self.world, self.prefix, self.max_silence_s = rank, world_size, prefix, max_silence_s
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self._time = time
        self.beat()

    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def beat(self) -> None:
        self.store.set(self._key("beat", self.rank), repr(self._time.time()))

    def leave(self, reason: str = "") -> None:
        """Announce an orderly exit.  Call it between steps, after the device is idle."""
        self.store.set(self._key("left", self.rank), reason or "left")

    def departed(self):
        """Ranks that left or have been silent for longer than ``max_silence_s`` (0 = heartbeats are not checked)."""
        gone = []
        now = self._time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([self._key("left", r)]):
                gone.append((r, self.store.get(self._key("left", r)).decode()))
            elif self.max_silence_s > 0 and self.store.check([self._key("beat", r)]):
                last = float(self.store.get(self._key("beat", r)).decode())
                if now - last > self.max_silence_s:
                    gone.append((r, f"silent for {now - last:.1f} s"))
        return gone

    def check(self) -> None:
        self.beat()
        gone = self.departed()
        if gone:
            raise RankLeft("; ".join(f"rank {r}: {why}" for r, why in gone))
