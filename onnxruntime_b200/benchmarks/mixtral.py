"""Mixtral-8x7B-shaped decoder, prefill: batch x seq prompt tokens through every layer (GroupQueryAttention + top-2 of 8
SwiGLU experts) on 1 GPU (``MoE``) or expert-parallel over N GPUs (``ShardedMoE``; attention replicated, every rank sees all
tokens, expert outputs combined across ranks).

    python -m onnxruntime_b200.benchmarks.mixtral [--batch 16 --seq 512 --layers 32 --steps 5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m onnxruntime_b200.benchmarks.mixtral

``--combine fused`` (default) uses the one-kernel cross-rank combine over peer memory; ``allreduce`` the library
all-reduce of the whole output (the baseline).  Random-init weights N(0, 0.02), random token ids.  Timed on the device
with CUDA events, max over ranks; the value is prompt tokens per second of the whole job."""
from __future__ import annotations

import argparse

import torch

from .common import finish, report, setup, timed_ms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--combine", default="fused", choices=["fused", "allreduce"])
    a = ap.parse_args(argv)
    rank, world, device, info = setup()
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.generation import DecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama

    cfg = LlamaConfig(vocab_size=32000, hidden_size=4096, num_layers=a.layers, num_heads=32, num_kv_heads=8, head_dim=128, ffn_size=14336,
                      max_seq_len=(a.seq + 127) // 128 * 128, rope_theta=1e6)
    model, weights = build_llama(cfg, external_weights=True, device=str(device), moe_experts=a.experts, moe_top_k=a.topk, ep_rank=rank,
                                 ep_size=world)
    so = ort.SessionOptions()
    so.add_external_initializers(list(weights.keys()), list(weights.values()))
    so.add_session_config_entry("ortb200.fused_moe_combine", "1" if a.combine == "fused" else "0")
    sess = ort.InferenceSession(model, so, providers=[("CUDAExecutionProvider", {"device_id": str(device.index)})], dist=info,
                                enable_fallback=False)
    del weights
    torch.cuda.empty_cache()
    tokens = a.batch * a.seq
    if world > 1 and a.combine == "fused":
        from onnxruntime_b200.parallel import symm
        need = 8 * tokens * cfg.hidden_size * 2 * max(1, (a.topk + world - 1) // world + 1)
        symm.attach(sess, symm.create_workspace(max(64 << 20, (need + (1 << 20)) // 256 * 256)))
    runner = DecoderRunner(sess, cfg, batch=a.batch, max_len=cfg.max_seq_len, device=device)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=torch.Generator().manual_seed(1)).to(device)
    ms = timed_ms(lambda: runner.prefill(ids), a.steps, a.warmup, world, device)
    sess.check_device_status()
    flops = tokens * a.layers * (a.topk * 6 * cfg.hidden_size * cfg.ffn_size + 2 * cfg.hidden_size * (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
                                 + 2 * cfg.hidden_size * cfg.num_heads * cfg.head_dim)
    report(rank, metric="mixtral_prefill_tokens_per_s", value=round(tokens / (ms * 1e-3), 1), unit="tokens/s", n_gpus=world,
           ms_per_step=round(ms, 3), tflops_total=round(flops / (ms * 1e-3) / 1e12, 1), dtype="bf16", impl="ours",
           config={"model": f"Mixtral-8x7B-shaped/{a.layers}L", "batch": a.batch, "seq": a.seq, "experts": a.experts, "top_k": a.topk,
                   "parallelism": f"ep{world}", "combine": a.combine if world > 1 else None},
           launches_per_step=sess.last_run_launch_count(), data="synthetic (random token ids, random-init N(0,0.02) weights)")
    finish(world)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
