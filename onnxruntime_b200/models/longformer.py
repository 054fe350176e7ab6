"""Longformer-style encoder as an ONNX graph, plus a numpy restatement.

Post-LayerNorm BERT blocks whose self attention is ``com.microsoft.LongformerAttention`` (sliding window of ``window``
tokens to either side, plus tokens marked global that attend to, and are attended by, every token through their own
projection weights), the form the reference's Longformer tooling emits
(onnxruntime/python/tools/transformers/models/longformer/convert_to_onnx.py).
Inputs: input_ids [B, S] int64, attention_mask [B, S] float (0 keep, -10000 padding), global_attention_mask [B, S] int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class LongformerConfig:
    vocab_size: int = 120
    hidden_size: int = 32
    num_layers: int = 2
    num_heads: int = 4
    ffn_size: int = 64
    window: int = 2               # one-sided
    max_position: int = 64
    layer_norm_eps: float = 1e-5


def init_weights(cfg: LongformerConfig, seed: int = 0, scale: float = 0.08) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    H, F = cfg.hidden_size, cfg.ffn_size
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape):
        w[name] = (rng.randn(*shape) * scale).astype(np.float32)

    def ln(name):
        w[name + ".gamma"] = (1.0 + rng.randn(H) * 0.02).astype(np.float32)
        w[name + ".beta"] = (rng.randn(H) * 0.02).astype(np.float32)

    n("embed", cfg.vocab_size, H), n("pos", cfg.max_position, H), ln("embed_ln")
    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        n(p + ".qkv.weight", H, 3 * H), n(p + ".qkv.bias", 3 * H), n(p + ".global_qkv.weight", H, 3 * H), n(p + ".global_qkv.bias", 3 * H)
        n(p + ".dense.weight", H, H), n(p + ".dense.bias", H), ln(p + ".ln1")
        n(p + ".fc1.weight", H, F), n(p + ".fc1.bias", F), n(p + ".fc2.weight", F, H), n(p + ".fc2.bias", H), ln(p + ".ln2")
    return w


def build_longformer(cfg: LongformerConfig, weights: Optional[Dict[str, np.ndarray]] = None, seed: int = 0, opset: int = 17) -> bytes:
    w = weights if weights is not None else init_weights(cfg, seed)
    inits = [ol.make_tensor(k, v) for k, v in w.items()]
    nodes: List[ol.Node] = []
    count = [0]

    def const(value, dtype):
        count[0] += 1
        inits.append(ol.make_tensor(f"c_{count[0]}", np.asarray(value, dtype=dtype)))
        return f"c_{count[0]}"

    def op(op_type, inputs, outputs=None, domain="", **attrs):
        count[0] += 1
        outs = outputs or [f"{op_type.lower()}_{count[0]}"]
        nodes.append(ol.make_node(op_type, inputs, outs, name=f"{op_type}_{count[0]}", domain=domain, **attrs))
        return outs[0]

    def ln(x, name):
        return op("LayerNormalization", [x, name + ".gamma", name + ".beta"], axis=-1, epsilon=cfg.layer_norm_eps)

    seq = op("Gather", [op("Shape", ["input_ids"]), const(1, np.int64)], axis=0)
    pos = op("Range", [const(0, np.int64), seq, const(1, np.int64)])
    x = ln(op("Add", [op("Gather", ["embed", "input_ids"], axis=0), op("Gather", ["pos", pos], axis=0)]), "embed_ln")
    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        a = op("LongformerAttention", [x, p + ".qkv.weight", p + ".qkv.bias", "attention_mask", p + ".global_qkv.weight", p + ".global_qkv.bias",
                                       "global_attention_mask"], domain="com.microsoft", num_heads=cfg.num_heads, window=cfg.window)
        x = ln(op("Add", [x, op("Add", [op("MatMul", [a, p + ".dense.weight"]), p + ".dense.bias"])]), p + ".ln1")
        h = op("Gelu", [op("Add", [op("MatMul", [x, p + ".fc1.weight"]), p + ".fc1.bias"])], domain="com.microsoft")
        x = ln(op("Add", [x, op("Add", [op("MatMul", [h, p + ".fc2.weight"]), p + ".fc2.bias"])]), p + ".ln2")
    op("Identity", [x], ["last_hidden_state"])
    vi = ol.make_tensor_value_info
    model = ol.make_model(ol.make_graph(nodes, "longformer", [vi("input_ids", T.INT64, ["batch", "seq"]), vi("attention_mask", T.FLOAT, ["batch", "seq"]),
                                                              vi("global_attention_mask", T.INT32, ["batch", "seq"])],
                                        [vi("last_hidden_state", T.FLOAT, ["batch", "seq", cfg.hidden_size])], inits), opset=opset)
    model.opset_imports["com.microsoft"] = 1
    return model.serialize()


def reference_forward(cfg: LongformerConfig, w: Dict[str, np.ndarray], input_ids: np.ndarray, attention_mask: np.ndarray,
                      global_attention_mask: np.ndarray) -> np.ndarray:
    import math
    f = {k: v.astype(np.float64) for k, v in w.items()}
    B, S = input_ids.shape
    H, N = cfg.hidden_size, cfg.num_heads
    hd = H // N
    erf = np.vectorize(math.erf)

    def ln(x, name):
        mu = x.mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(((x - mu) ** 2).mean(-1, keepdims=True) + cfg.layer_norm_eps) * f[name + ".gamma"] + f[name + ".beta"]

    def heads(t, part):
        return t[:, :, part * H:(part + 1) * H].reshape(B, S, N, hd).transpose(0, 2, 1, 3)

    def attend(qkv, allowed):
        s = heads(qkv, 0) @ heads(qkv, 1).transpose(0, 1, 3, 2) / math.sqrt(hd) + attention_mask.astype(np.float64)[:, None, None, :]
        s = np.where(allowed, s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        return (p / p.sum(-1, keepdims=True)) @ heads(qkv, 2)

    pos = np.arange(S)
    is_global = global_attention_mask != 0
    allowed = (np.abs(pos[:, None] - pos[None, :]) <= cfg.window)[None, None] | is_global[:, None, None, :]
    x = ln(f["embed"][input_ids] + f["pos"][pos][None], "embed_ln")
    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        local = attend(x @ f[p + ".qkv.weight"] + f[p + ".qkv.bias"], allowed)
        glob = attend(x @ f[p + ".global_qkv.weight"] + f[p + ".global_qkv.bias"], np.ones_like(allowed))
        a = np.where(is_global[:, None, :, None], glob, local).transpose(0, 2, 1, 3).reshape(B, S, H)
        x = ln(x + a @ f[p + ".dense.weight"] + f[p + ".dense.bias"], p + ".ln1")
        h = x @ f[p + ".fc1.weight"] + f[p + ".fc1.bias"]
        h = 0.5 * h * (1.0 + erf(h / math.sqrt(2.0)))
        x = ln(x + h @ f[p + ".fc2.weight"] + f[p + ".fc2.bias"], p + ".ln2")
    return x
