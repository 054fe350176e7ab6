"""BERT-large encoder throughput, data parallel: every rank runs batch x seq tokens through the same model.

    python -m onnxruntime_b200.benchmarks.bert [--batch 64 --seq 384 --layers 24 --steps 10 --baseline torch --dtype fp8]

The session path loads the exporter-style (unfused) graph and lets the optimizer find Attention,
SkipLayerNormalization, EmbedLayerNormalization and the GEMM epilogues; inputs are bound on the device."""
from __future__ import annotations

import argparse

import numpy as np
import torch

from .common import finish, report, setup, timed_ms


def torch_bert(cfg, weights, ids, mask):
    """The same encoder through PyTorch library kernels (cuBLAS GEMMs, SDPA attention, separate LayerNorm / GELU)."""
    import torch.nn.functional as F
    H, N = cfg.hidden_size, cfg.num_heads
    B, S = ids.shape
    x = weights["embeddings.word"][ids] + weights["embeddings.position"][:S].unsqueeze(0)
    x = F.layer_norm(x, (H,), weights["embeddings.ln.gamma"], weights["embeddings.ln.beta"], cfg.layer_norm_eps)
    amask = mask.bool().view(B, 1, 1, S)
    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        q = (x @ weights[f"{p}.attn.q.weight"] + weights[f"{p}.attn.q.bias"]).view(B, S, N, -1).transpose(1, 2)
        k = (x @ weights[f"{p}.attn.k.weight"] + weights[f"{p}.attn.k.bias"]).view(B, S, N, -1).transpose(1, 2)
        v = (x @ weights[f"{p}.attn.v.weight"] + weights[f"{p}.attn.v.bias"]).view(B, S, N, -1).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=amask).transpose(1, 2).reshape(B, S, H)
        a = a @ weights[f"{p}.attn.o.weight"] + weights[f"{p}.attn.o.bias"]
        x = F.layer_norm(x + a, (H,), weights[f"{p}.attn.ln.gamma"], weights[f"{p}.attn.ln.beta"], cfg.layer_norm_eps)
        h = F.gelu(x @ weights[f"{p}.ffn.fc1.weight"] + weights[f"{p}.ffn.fc1.bias"])
        h = h @ weights[f"{p}.ffn.fc2.weight"] + weights[f"{p}.ffn.fc2.bias"]
        x = F.layer_norm(x + h, (H,), weights[f"{p}.ffn.ln.gamma"], weights[f"{p}.ffn.ln.beta"], cfg.layer_norm_eps)
    return x


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=384)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--baseline", default="", choices=["", "torch"])
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "fp8"], help="fp8: dense layers as GemmFloat8 (e4m3 weights and activations)")
    a = ap.parse_args(argv)
    rank, world, device, info = setup()

    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.bert import BertConfig, build_bert, build_bert_fp8, init_weights
    cfg = BertConfig.bert_large(num_layers=a.layers, max_position=max(512, a.seq))
    weights = init_weights(cfg)
    rng = np.random.RandomState(rank)
    ids = torch.from_numpy(rng.randint(0, cfg.vocab_size, (a.batch, a.seq))).to(device)
    lens = rng.randint(a.seq // 2, a.seq + 1, a.batch)
    mask = torch.from_numpy((np.arange(a.seq)[None, :] < lens[:, None]).astype(np.int64)).to(device)

    if a.baseline == "torch":
        tw = {k: torch.from_numpy(v).to(device) for k, v in weights.items()}
        with torch.no_grad():
            ms = timed_ms(lambda: torch_bert(cfg, tw, ids, mask), a.steps, a.warmup, world, device)
        launches = None
        fused = {}
    else:
        model = build_bert_fp8(cfg, weights) if a.dtype == "fp8" else build_bert(cfg, weights)
        sess = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"device_id": str(device.index)})], enable_fallback=False)
        out_name = sess.get_outputs()[0].name
        out = torch.empty(a.batch, a.seq, cfg.hidden_size, dtype=torch.float16, device=device)
        b = sess.io_binding()
        b.bind_torch_input("input_ids", ids)
        b.bind_torch_input("attention_mask", mask)
        b.bind_torch_output(out_name, out)
        ms = timed_ms(lambda: sess.run_with_iobinding(b), a.steps, a.warmup, world, device)
        launches = sess.last_run_launch_count()
        fused = {}
        for n in sess.graph_nodes():
            if n["op_type"] in ("Attention", "MultiHeadAttention", "SkipLayerNormalization", "EmbedLayerNormalization", "FusedGemm", "BiasGelu", "GemmFloat8"):
                fused[n["op_type"]] = fused.get(n["op_type"], 0) + 1
        sess.check_device_status()
    tokens = a.batch * a.seq * world
    flops = a.layers * (8 * cfg.hidden_size ** 2 + 4 * cfg.hidden_size * cfg.ffn_size + 4 * a.seq * cfg.hidden_size) * a.batch * a.seq
    report(rank, metric="bert_large_sequences_per_s", value=round(a.batch * world / (ms * 1e-3), 2), unit="sequences/s", n_gpus=world,
           ms_per_step=round(ms, 3), tokens_per_s=round(tokens / (ms * 1e-3), 1), tflops_per_gpu=round(flops / (ms * 1e-3) / 1e12, 1),
           dtype=a.dtype, impl=a.baseline or "ours", config={"batch_per_gpu": a.batch, "seq_len": a.seq, "layers": a.layers,
                                                            "parallelism": f"dp{world}"},
           launches_per_step=launches, fused_ops=fused, data="synthetic (random ids, right-padded to random lengths)")
    finish(world)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
