"""Tiny BERT-style encoder on the CPU provider, fp32: latency of the exporter-style graph, of the fused graph
(Attention / SkipLayerNormalization / BiasGelu / EmbedLayerNormalization), and of a plain numpy restatement of the
same math as the timed CPU baseline; outputs are compared element by element.

    python -m onnxruntime_b200.benchmarks.tiny_bert_cpu [--batch 2 --seq 32 --runs 200 --threads 1]

Model: 2 layers, hidden 128, 2 heads, FFN 512 (erf GELU), post-LayerNorm, vocabulary 1000, 64 positions; token ids
uniform in [0, 1000), mask all ones, weights N(0, 0.02), LayerNorm gamma 1 / beta 0, seed 0."""
from __future__ import annotations

import argparse
import json
import time

import numpy as np


def _latency_ms(fn, runs: int, warmup: int = 10):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(runs):
        t0 = time.perf_counter()
        fn()
        ts.append((time.perf_counter() - t0) * 1e3)
    ts.sort()
    return {"p50": round(ts[len(ts) // 2], 4), "p90": round(ts[int(len(ts) * 0.9)], 4), "min": round(ts[0], 4)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--runs", type=int, default=200)
    ap.add_argument("--threads", type=int, default=1, help="intra-op threads of the sessions and of the numpy baseline's BLAS")
    a = ap.parse_args(argv)
    import torch
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.bert import BertConfig, build_bert, init_weights, reference_forward
    cfg = BertConfig.tiny()
    w = init_weights(cfg, 0)
    model = build_bert(cfg, w)
    rng = np.random.RandomState(0)
    ids = rng.randint(0, cfg.vocab_size, (a.batch, a.seq)).astype(np.int64)
    mask = np.ones((a.batch, a.seq), np.int64)
    feeds = {"input_ids": ids, "attention_mask": mask}

    def session(level):
        so = ort.SessionOptions()
        so.graph_optimization_level = level
        so.intra_op_num_threads = a.threads
        return ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    plain, fused = session(ort.GraphOptimizationLevel.ORT_DISABLE_ALL), session(ort.GraphOptimizationLevel.ORT_ENABLE_ALL)
    torch.set_num_threads(a.threads)
    ref = reference_forward(cfg, w, ids, mask, None)
    out_plain, out_fused = plain.run(None, feeds)[0], fused.run(None, feeds)[0]
    res = {
        "metric": "tiny_bert_cpu_latency_ms", "unit": "ms", "dtype": "fp32", "threads": a.threads,
        "config": {"layers": cfg.num_layers, "hidden": cfg.hidden_size, "heads": cfg.num_heads, "ffn": cfg.ffn_size, "batch": a.batch, "seq": a.seq},
        "session_unfused": _latency_ms(lambda: plain.run(None, feeds), a.runs),
        "session_fused": _latency_ms(lambda: fused.run(None, feeds), a.runs),
        "numpy_baseline": _latency_ms(lambda: reference_forward(cfg, w, ids, mask, None), max(a.runs // 4, 10)),
        "nodes": {"unfused": len(plain.graph_nodes()), "fused": len(fused.graph_nodes())},
        "max_abs_diff": {"unfused_vs_numpy": float(np.abs(out_plain - ref).max()), "fused_vs_numpy": float(np.abs(out_fused - ref).max()),
                         "fused_vs_unfused": float(np.abs(out_fused - out_plain).max())},
        "data": "synthetic (token ids uniform in [0, 1000), all-ones mask, weights N(0, 0.02), seed 0)",
    }
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
