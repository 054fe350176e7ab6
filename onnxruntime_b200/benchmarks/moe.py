"""Mixtral-8x7B-shaped MoE layer, prefill: tokens x hidden through top-2 of 8 SwiGLU experts.

    python -m onnxruntime_b200.benchmarks.moe [--tokens 8192 --hidden 4096 --inter 14336 --experts 8 --steps 10 --baseline torch]

One GPU runs ``com.microsoft.MoE`` over all experts; N GPUs run ``ShardedMoE`` with experts/N local experts per rank
(expert parallelism, replicated tokens, outputs summed over ranks)."""
from __future__ import annotations

import argparse

import numpy as np
import torch

from .common import finish, report, setup, timed_ms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16 * 512)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--baseline", default="", choices=["", "torch"])
    ap.add_argument("--combine", default="fused", choices=["fused", "allreduce"],
                    help="N > 1: fused = one kernel un-permutes, scales, sums across ranks over peer memory and replicates; "
                         "allreduce = local combine, then a library all-reduce of the whole output (baseline)")
    a = ap.parse_args(argv)
    rank, world, device, info = setup()
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    E, H, I, k = a.experts, a.hidden, a.inter, a.topk
    assert E % world == 0
    el = E // world
    g = torch.Generator(device="cpu").manual_seed(0)
    x = (torch.randn(a.tokens, H, generator=g) * 0.5).to(torch.bfloat16).to(device)
    logits = torch.randn(a.tokens, E, generator=g).to(torch.bfloat16).to(device)

    def expert_weights(e):
        ge = torch.Generator(device="cpu").manual_seed(100 + e)
        return [(torch.randn(I, H, generator=ge) * 0.02).to(torch.bfloat16), (torch.randn(H, I, generator=ge) * 0.02).to(torch.bfloat16),
                (torch.randn(I, H, generator=ge) * 0.02).to(torch.bfloat16)]
    mine = [expert_weights(e) for e in range(rank * el, (rank + 1) * el)]
    fc1 = torch.stack([w[0] for w in mine]).to(device)   # [el, I, H]
    fc2 = torch.stack([w[1] for w in mine]).to(device)   # [el, H, I]
    fc3 = torch.stack([w[2] for w in mine]).to(device)

    if a.baseline == "torch":
        import torch.distributed as dist

        def step():
            p = torch.softmax(logits.float(), -1)
            w, idx = torch.topk(p, k, -1)
            w = (w / w.sum(-1, keepdim=True)).to(x.dtype)
            out = torch.zeros_like(x)
            for le in range(el):
                e = rank * el + le
                tok, slot = (idx == e).nonzero(as_tuple=True)
                if tok.numel() == 0:
                    continue
                xe = x[tok]
                h = torch.nn.functional.silu(xe @ fc1[le].T) * (xe @ fc3[le].T)
                out.index_add_(0, tok, (h @ fc2[le].T) * w[tok, slot].unsqueeze(-1))
            if world > 1:
                dist.all_reduce(out)
            return out
        with torch.no_grad():
            ms = timed_ms(step, a.steps, a.warmup, world, device)
        launches = None
    else:
        so = ort.SessionOptions()
        names = ["fc1", "fc2", "fc3"]
        so.add_external_initializers(names, [fc1 if world == 1 else fc1.transpose(1, 2).contiguous(),
                                             fc2 if world == 1 else fc2.transpose(1, 2).contiguous(),
                                             fc3 if world == 1 else fc3.transpose(1, 2).contiguous()])
        # ShardedMoE keeps the older [E, in, out] weight layout of the reference's op
        shapes = {"fc1": [el, I, H] if world == 1 else [el, H, I], "fc2": [el, H, I] if world == 1 else [el, I, H],
                  "fc3": [el, I, H] if world == 1 else [el, H, I]}
        op = "MoE" if world == 1 else "ShardedMoE"
        attrs = dict(k=k, activation_type="silu", normalize_routing_weights=1)
        if world > 1:
            attrs["local_experts_start_index"] = rank * el
        node = ol.make_node(op, ["x", "router", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", **attrs)
        graph = ol.make_graph([node], "moe", [ol.make_tensor_value_info("x", T.BFLOAT16, [a.tokens, H]),
                                              ol.make_tensor_value_info("router", T.BFLOAT16, [a.tokens, E])],
                              [ol.make_tensor_value_info("y", T.BFLOAT16, [a.tokens, H])],
                              [ol.make_external_tensor(n, T.BFLOAT16, shapes[n]) for n in names])
        sess = ort.InferenceSession(ol.make_model(graph).serialize(), so, providers=[("CUDAExecutionProvider", {"device_id": str(device.index)})],
                                    dist=info, enable_fallback=False)
        del fc1, fc2, fc3
        if world > 1 and a.combine == "fused":
            from onnxruntime_b200.parallel import symm
            need = 8 * a.tokens * H * 2 * max(1, (k + world - 1) // world + 1)   # scatter and result areas, two parities
            symm.attach(sess, symm.create_workspace(max(64 << 20, (need + (1 << 20)) // 256 * 256)))
        out = torch.empty(a.tokens, H, dtype=torch.bfloat16, device=device)
        b = sess.io_binding()
        b.bind_torch_input("x", x)
        b.bind_torch_input("router", logits)
        b.bind_torch_output("y", out)
        ms = timed_ms(lambda: sess.run_with_iobinding(b), a.steps, a.warmup, world, device)
        launches = sess.last_run_launch_count()
        sess.check_device_status()
    flops = a.tokens * k * 6 * H * I  # three GEMMs per routed token
    report(rank, metric="mixtral_moe_prefill_tokens_per_s", value=round(a.tokens / (ms * 1e-3), 1), unit="tokens/s", n_gpus=world,
           ms_per_step=round(ms, 3), tflops_total=round(flops / (ms * 1e-3) / 1e12, 1), dtype="bf16", impl=a.baseline or "ours",
           config={"tokens": a.tokens, "hidden": H, "intermediate": I, "experts": E, "top_k": k, "parallelism": f"ep{world}",
                   "combine": (a.combine if world > 1 and not a.baseline else None)},
           launches_per_step=launches, data="synthetic")
    finish(world)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
