"""All-gather -> GEMM kernel against all-gather followed by a GEMM, and against the plain GEMMs.

One process: `python -m onnxruntime_b200.benchmarks.allgather_gemm` times the kernel with a single rank (no peers: a
plain GEMM in the kernel's tile order) beside `ortb200_gemm` and torch.matmul (cuBLAS).  Several ranks:
`python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m onnxruntime_b200.benchmarks.allgather_gemm`
shards `--tokens` rows over the ranks and compares the fused kernel with the process group's all-gather + `ortb200_gemm`.
Timing: CUDA events around one call, a buffer larger than L2 written between calls, barrier before each call, max
over ranks.  The counterpart in the reference is AllGather (onnxruntime/contrib_ops/cuda/collective/nccl_kernels.cc:430)
followed by MatMul.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--features", type=int, default=4096, help="output features of this rank's weight")
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    from onnxruntime_b200.ops import _kernels as K

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rows = args.tokens // world
    need = 8 * world * rows * args.hidden * 2            # the gather areas are an eighth of the workspace
    nbytes = max(64 << 20, 1 << (need - 1).bit_length())
    if world > 1:
        from onnxruntime_b200.parallel import symm
        dist.init_process_group("nccl")
        ws = symm.create_workspace(nbytes)
        peers, nbytes = ws.peer_ptrs, ws.nbytes
    else:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        peers = [buf.data_ptr()]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    x = (torch.randn(rows, args.hidden, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(args.features, args.hidden, device="cuda") * 0.05).bfloat16()
    full = torch.empty(world * rows, args.hidden, dtype=torch.bfloat16, device="cuda")

    def timed(fn) -> float:
        for _ in range(args.warmup):
            fn()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / args.iters], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def library():
        if world > 1:
            dist.all_gather_into_tensor(full, x)
            return K.gemm(full, w)
        return K.gemm(x, w)

    res = {"ranks": world, "tokens": world * rows, "features": args.features, "hidden": args.hidden,
           "ms_fused": timed(lambda: K.allgather_gemm(x, w, peers, rank, nbytes, status=status)),
           "ms_allgather_then_gemm": timed(library),
           "ms_gemm_alone": timed(lambda: K.gemm(full if world > 1 else x, w)),
           "ms_cublas_alone": timed(lambda: torch.matmul(full if world > 1 else x, w.t()))}
    res["tflops_fused"] = 2.0 * world * rows * args.features * args.hidden / res["ms_fused"] / 1e9
    res["status"] = int(status.item())
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
