"""Timing helpers shared by the benchmark scripts: CUDA events, warm-up, max over ranks."""
from __future__ import annotations

import json
import os
from typing import Callable

import torch
import torch.distributed as dist


def setup():
    """(rank, world, device); initialises NCCL when launched by torch.distributed.run."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    info = None
    if world > 1:
        from onnxruntime_b200.parallel.dist import init_distributed
        info = init_distributed("nccl")
        local = info.local_rank
    else:
        local = 0
    torch.cuda.set_device(local)
    return (info.rank if info else 0), world, torch.device("cuda", local), info


def timed_ms(fn: Callable[[], None], steps: int, warmup: int, world: int, device) -> float:
    """Milliseconds per call: ``warmup`` untimed calls, then ``steps`` calls between CUDA events, max over ranks."""
    for _ in range(max(warmup, 3)):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return ms


def report(rank: int, **fields) -> None:
    if rank == 0:
        print(json.dumps(fields))


def finish(world: int) -> None:
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
