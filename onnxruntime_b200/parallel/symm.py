"""Symmetric peer-mapped workspace for the fused compute+collective kernels.

Every rank allocates one buffer through ``torch.distributed._symmetric_memory``;
after the rendezvous each rank holds the address at which every peer's buffer is
mapped into its own address space (NVLink peer access inside one node).  The
kernels write partial results straight into peers' buffers and signal with
flags in the same buffer, so the transfer overlaps the tensor-core work tile by
tile.  The reference has a much smaller relative of this for its custom
all-reduce (CUDA-IPC handles exchanged over MPI,
onnxruntime/contrib_ops/cuda/collective/ipc_utils.cc:30-112).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

DEFAULT_BYTES = 64 << 20


@dataclass
class SymmetricWorkspace:
    tensor: torch.Tensor          # local buffer (kept alive here)
    handle: object                # torch symmetric-memory handle
    peer_ptrs: List[int]          # peer_ptrs[r] = address of rank r's buffer in this process
    nbytes: int
    multicast_ptr: int = 0        # NVLS multicast address of the buffer, 0 when unavailable


def create_workspace(nbytes: int = DEFAULT_BYTES, group: Optional[dist.ProcessGroup] = None) -> SymmetricWorkspace:
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    dev = torch.device("cuda", torch.cuda.current_device())
    t = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
    t.zero_()
    hdl = symm_mem.rendezvous(t, group.group_name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    mc = 0
    try:
        mc = int(hdl.multicast_ptr or 0)
    except Exception:
        mc = 0
    torch.cuda.synchronize()
    dist.barrier(group)
    return SymmetricWorkspace(t, hdl, ptrs, nbytes, mc)


def attach(session, ws: SymmetricWorkspace) -> None:
    """Give a session the peer addresses; its row-parallel GEMMs then reduce across ranks inside the kernel.  With an
    NVLS multicast address the prompt-sized all-reduces are summed and replicated by the switch (session config
    ``ortb200.nvls`` = "0" keeps them on peer loads and stores)."""
    session._sess.set_symmetric_workspace(ws.peer_ptrs, ws.nbytes, ws.multicast_ptr)
    session._symm_ws = ws  # keep the mapping alive as long as the session
