"""Llama-3-70B-shaped decoder with 4-bit weights (MatMulNBits, blocks of 32) over a paged KV cache, decode.

    python -m onnxruntime_b200.benchmarks.llama_int4 [--layers 80 --batch 8 --context 1024 --steps 32 --block-size 256]
    python -m torch.distributed.run --nproc-per-node 8 ... -m onnxruntime_b200.benchmarks.llama_int4   # TP = world

Every projection of every layer is ``com.microsoft.MatMulNBits`` on packed weights that stay packed in device
memory (the decode kernel expands them tile by tile in shared memory); attention is
``com.microsoft.PagedAttention`` over one pool of cache blocks addressed through a block table; with N ranks the
heads and FFN columns are split N ways and the two row-parallel projections of a layer are all-reduced.  The timed
region is one decode step (one new token for each of ``batch`` sequences that already hold ``context`` tokens),
replayed as a CUDA graph.  Weights are random; the cache holds zeros (attention cost does not depend on values)."""
from __future__ import annotations

import argparse

import torch

from .common import finish, report, setup, timed_ms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--batch", default="8", help="decode batch size, or a comma-separated list measured on one loaded model")
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="70b", choices=["70b", "8b"])
    ap.add_argument("--dense", action="store_true", help="bf16 MatMul weights instead of 4-bit (for comparison)")
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args(argv)
    rank, world, device, info = setup()
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.generation import PagedDecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama

    batches = [int(b) for b in str(a.batch).split(",")]
    max_len = (a.context + a.steps + max(a.warmup, 3) + 8 + a.block_size - 1) // a.block_size * a.block_size
    make = LlamaConfig.llama3_70b if a.model == "70b" else LlamaConfig.llama3_8b
    cfg = make(max_seq_len=max_len, num_layers=a.layers)
    model, weights = build_llama(cfg, tp_rank=rank, tp_size=world, external_weights=True, device=str(device),
                                 quant_bits=0 if a.dense else 4, paged=True)
    weight_bytes = sum(w.numel() * w.element_size() for n, w in weights.items() if "layers." in n or n == "lm_head.weight")
    so = ort.SessionOptions()
    so.add_external_initializers(list(weights.keys()), list(weights.values()))
    providers = [("CUDAExecutionProvider", {"device_id": str(device.index), "enable_cuda_graph": "0" if a.no_graph else "1"})]
    sess = ort.InferenceSession(model, so, providers=providers, dist=info if world > 1 else None, enable_fallback=False)
    del weights
    torch.cuda.empty_cache()
    if world > 1:
        from onnxruntime_b200.parallel import symm
        symm.attach(sess, symm.create_workspace(256 << 20))
    for gi, batch in enumerate(batches):
        runner = PagedDecoderRunner(sess, cfg, batch=batch, max_len=max_len, block_size=a.block_size, tp_size=world, device=device,
                                    graph_id=1 + gi)
        runner.assume_context(a.context)
        tokens = torch.randint(0, cfg.vocab_size, (batch,), device=device)
        before = sess.kernel_launch_count()
        runner.decode_step(tokens)     # the first step runs eagerly (the session captures its graph afterwards): count it
        launches = sess.kernel_launch_count() - before
        runner.decode_step()
        ms = timed_ms(lambda: runner.decode_step(), a.steps, a.warmup, world, device)
        sess.check_device_status()
        report(rank, metric="llama3_70b_int4_paged_decode_tokens_per_s" if a.model == "70b" and not a.dense else "paged_decode_tokens_per_s",
               value=round(batch / ms * 1e3, 1), unit="tokens/s", n_gpus=world, ms_per_step=round(ms, 4),
               weight_gb_per_rank=round(weight_bytes / 1e9, 2), weight_stream_gbs=round(weight_bytes / ms / 1e6, 1),
               launches_per_step=launches, dtype="int4 weights (block 32, bf16 scales), bf16 activations" if not a.dense else "bf16",
               impl="ours", data="synthetic",
               config={"model": f"Llama-3-{a.model.upper()}", "layers": a.layers, "batch": batch, "context": a.context,
                       "kv_block_size": a.block_size, "parallelism": f"tp{world}", "cuda_graph": not a.no_graph})
        del runner
        torch.cuda.empty_cache()
    finish(world)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
