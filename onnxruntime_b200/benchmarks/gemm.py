"""GEMM micro-benchmark: one problem through this library's tcgen05 kernels and through cuBLAS (torch.matmul).

    python -m onnxruntime_b200.benchmarks.gemm --m 8192 --n 6144 --k 4096 [--act gelu --residual --dtype bf16 --steps 20]

Inputs are rotated through several buffers so that every timed launch reads operands that are not in the L2.  Prints
one JSON line with microseconds, TFLOP/s and (for small M) the weight-streaming rate.  Also the driver for profiler
captures of the GEMM kernels (one kernel family per shape: M <= 64 decode kernel, larger M CTA-pair kernel)."""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--act", default="none")
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skip-cublas", action="store_true")
    a = ap.parse_args(argv)
    from onnxruntime_b200.ops import _kernels as K
    K.lib()
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    dev = torch.device("cuda")
    bytes_per_set = (a.m * a.k + a.n * a.k + a.m * a.n) * 2
    sets = max(2, min(8, int(300e6 // max(bytes_per_set, 1)) + 1))   # together larger than the 126 MB L2
    xs = [(torch.randn(a.m, a.k, device=dev) * 0.5).to(dt) for _ in range(sets)]
    ws = [(torch.randn(a.n, a.k, device=dev) * 0.05).to(dt) for _ in range(sets)]
    res = (torch.randn(a.m, a.n, device=dev)).to(dt) if a.residual else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def timed(fn):
        for i in range(max(a.warmup, 3)):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / a.steps

    ours = timed(lambda i: K.gemm(xs[i % sets], ws[i % sets], residual=res, act=a.act, status=status))
    y = K.gemm(xs[0], ws[0], residual=res, act=a.act, status=status)
    ref = xs[0].float() @ ws[0].float().t()
    if a.act == "gelu":
        ref = torch.nn.functional.gelu(ref)
    elif a.act == "relu":
        ref = torch.relu(ref)
    if res is not None:
        ref = ref + res.float()
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    flops = 2.0 * a.m * a.n * a.k
    out = {"metric": "gemm_us", "shape": [a.m, a.n, a.k], "dtype": a.dtype, "act": a.act, "residual": a.residual,
           "ours_us": round(ours, 2), "ours_tflops": round(flops / ours / 1e6, 1), "weight_gbs": round(a.n * a.k * 2 / ours / 1e3, 1),
           "kernel_config": dict(zip(("tile", "split_or_cluster", "stages"), K.gemm_last_config())), "rel_err": err, "status": int(status.item())}
    if not a.skip_cublas:
        cub = timed(lambda i: torch.matmul(xs[i % sets], ws[i % sets].t()))
        out["cublas_us"] = round(cub, 2)
        out["cublas_tflops"] = round(flops / cub / 1e6, 1)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
