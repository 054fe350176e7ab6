"""GPT-2-style decoder as an ONNX graph with past / present key-value state, plus a numpy restatement.

The graph has the form the reference's GPT-2 tooling produces after fusion (onnxruntime/python/tools/transformers/models/
gpt2/gpt2_helper.py, onnx_model_gpt2.py): per layer LayerNormalization -> com.microsoft Attention (unidirectional, merged
QKV weight, past_i -> present_i of shape [2, batch, heads, sequence, head]) -> residual -> LayerNormalization -> MatMul +
FastGelu (tanh form) -> MatMul -> residual; learned position embeddings indexed by position_ids; the output projection
shares the token embedding.  Inputs (int32, as the generation operators feed them): input_ids, position_ids, attention_mask
(over past + new tokens), past_0 .. past_{L-1};
outputs: logits, present_0 .. present_{L-1} - the interface the GreedySearch / BeamSearch operators drive (model_type 0).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class Gpt2Config:
    vocab_size: int = 1000
    hidden_size: int = 64
    num_layers: int = 2
    num_heads: int = 4
    max_position: int = 128
    layer_norm_eps: float = 1e-5
    dtype: str = "fp32"      # fp32 | fp16

    @staticmethod
    def gpt2_small(**kw) -> "Gpt2Config":
        base = dict(vocab_size=50257, hidden_size=768, num_layers=12, num_heads=12, max_position=1024)
        base.update(kw)
        return Gpt2Config(**base)


def init_weights(cfg: Gpt2Config, seed: int = 0) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    dt = np.float16 if cfg.dtype == "fp16" else np.float32
    H = cfg.hidden_size
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape):
        w[name] = (rng.randn(*shape) * 0.02).astype(dt)

    n("wte", cfg.vocab_size, H)
    n("wpe", cfg.max_position, H)
    for i in range(cfg.num_layers):
        p = f"h.{i}"
        for ln in ("ln_1", "ln_2"):
            w[f"{p}.{ln}.gamma"] = (1.0 + rng.randn(H) * 0.02).astype(dt)
            w[f"{p}.{ln}.beta"] = (rng.randn(H) * 0.02).astype(dt)
        n(f"{p}.attn.qkv.weight", H, 3 * H)
        n(f"{p}.attn.qkv.bias", 3 * H)
        n(f"{p}.attn.proj.weight", H, H)
        n(f"{p}.attn.proj.bias", H)
        n(f"{p}.mlp.fc.weight", H, 4 * H)
        n(f"{p}.mlp.fc.bias", 4 * H)
        n(f"{p}.mlp.proj.weight", 4 * H, H)
        n(f"{p}.mlp.proj.bias", H)
    w["ln_f.gamma"] = (1.0 + rng.randn(H) * 0.02).astype(dt)
    w["ln_f.beta"] = (rng.randn(H) * 0.02).astype(dt)
    return w


def build_gpt2(cfg: Gpt2Config, weights: Optional[Dict[str, np.ndarray]] = None, seed: int = 0, opset: int = 17) -> bytes:
    w = weights if weights is not None else init_weights(cfg, seed)
    odt = T.FLOAT16 if cfg.dtype == "fp16" else T.FLOAT
    H, N, L = cfg.hidden_size, cfg.num_heads, cfg.num_layers
    nodes: List[ol.Node] = []
    inits = [ol.make_tensor(k, v) for k, v in w.items()]
    inits.append(ol.make_tensor("wte_t", np.ascontiguousarray(w["wte"].T)))
    count = [0]

    def op(op_type, inputs, outputs=None, domain="", **attrs):
        count[0] += 1
        outs = outputs or [f"{op_type.lower()}_{count[0]}"]
        nodes.append(ol.make_node(op_type, inputs, outs, name=f"{op_type}_{count[0]}", domain=domain, **attrs))
        return outs[0]

    inputs = [ol.make_tensor_value_info("input_ids", T.INT32, ["batch", "seq"]), ol.make_tensor_value_info("position_ids", T.INT32, ["batch", "seq"]),
              ol.make_tensor_value_info("attention_mask", T.INT32, ["batch", "total"])]
    outputs = [ol.make_tensor_value_info("logits", odt, ["batch", "seq", cfg.vocab_size])]
    x = op("Add", [op("Gather", ["wte", "input_ids"], axis=0), op("Gather", ["wpe", "position_ids"], axis=0)])
    for i in range(L):
        p = f"h.{i}"
        inputs.append(ol.make_tensor_value_info(f"past_{i}", odt, [2, "batch", N, "past", H // N]))
        outputs.append(ol.make_tensor_value_info(f"present_{i}", odt, [2, "batch", N, "total", H // N]))
        ln1 = op("LayerNormalization", [x, f"{p}.ln_1.gamma", f"{p}.ln_1.beta"], axis=-1, epsilon=cfg.layer_norm_eps)
        count[0] += 1
        attn = f"attn_{count[0]}"
        nodes.append(ol.make_node("Attention", [ln1, f"{p}.attn.qkv.weight", f"{p}.attn.qkv.bias", "attention_mask", f"past_{i}"], [attn, f"present_{i}"],
                                  name=f"Attention_{i}", domain="com.microsoft", num_heads=N, unidirectional=1))
        x = op("Add", [x, op("Add", [op("MatMul", [attn, f"{p}.attn.proj.weight"]), f"{p}.attn.proj.bias"])])
        ln2 = op("LayerNormalization", [x, f"{p}.ln_2.gamma", f"{p}.ln_2.beta"], axis=-1, epsilon=cfg.layer_norm_eps)
        h = op("FastGelu", [op("MatMul", [ln2, f"{p}.mlp.fc.weight"]), f"{p}.mlp.fc.bias"], domain="com.microsoft")
        x = op("Add", [x, op("Add", [op("MatMul", [h, f"{p}.mlp.proj.weight"]), f"{p}.mlp.proj.bias"])])
    xf = op("LayerNormalization", [x, "ln_f.gamma", "ln_f.beta"], axis=-1, epsilon=cfg.layer_norm_eps)
    op("MatMul", [xf, "wte_t"], ["logits"])
    model = ol.make_model(ol.make_graph(nodes, "gpt2", inputs, outputs, inits), opset=opset)
    model.opset_imports["com.microsoft"] = 1
    return model.serialize()


def empty_past(cfg: Gpt2Config, batch: int) -> Dict[str, np.ndarray]:
    dt = np.float16 if cfg.dtype == "fp16" else np.float32
    return {f"past_{i}": np.zeros((2, batch, cfg.num_heads, 0, cfg.hidden_size // cfg.num_heads), dt) for i in range(cfg.num_layers)}


def reference_forward(cfg: Gpt2Config, w: Dict[str, np.ndarray], input_ids: np.ndarray, attention_mask: Optional[np.ndarray] = None) -> np.ndarray:
    """Logits of the whole sequence in one pass (float64), causal mask plus an optional [batch, seq] padding mask."""
    B, S = input_ids.shape
    H, N = cfg.hidden_size, cfg.num_heads
    hd = H // N
    f = {k: v.astype(np.float64) for k, v in w.items()}

    def ln(x, g, b):
        mu = x.mean(-1, keepdims=True)
        var = ((x - mu) ** 2).mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(var + cfg.layer_norm_eps) * g + b

    x = f["wte"][input_ids] + f["wpe"][np.arange(S)][None]
    bias = np.where(np.tril(np.ones((S, S), bool)), 0.0, -np.inf)[None, None]
    if attention_mask is not None:
        bias = bias + np.where(attention_mask[:, None, None, :] != 0, 0.0, -10000.0)
    for i in range(cfg.num_layers):
        p = f"h.{i}"
        qkv = ln(x, f[f"{p}.ln_1.gamma"], f[f"{p}.ln_1.beta"]) @ f[f"{p}.attn.qkv.weight"] + f[f"{p}.attn.qkv.bias"]
        q, k, v = (t.reshape(B, S, N, hd).transpose(0, 2, 1, 3) for t in np.split(qkv, 3, -1))
        s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(hd) + bias
        pr = np.exp(s - s.max(-1, keepdims=True))
        pr = pr / pr.sum(-1, keepdims=True)
        a = (pr @ v).transpose(0, 2, 1, 3).reshape(B, S, H)
        x = x + a @ f[f"{p}.attn.proj.weight"] + f[f"{p}.attn.proj.bias"]
        h = ln(x, f[f"{p}.ln_2.gamma"], f[f"{p}.ln_2.beta"]) @ f[f"{p}.mlp.fc.weight"] + f[f"{p}.mlp.fc.bias"]
        h = 0.5 * h * (1.0 + np.tanh(0.7978845608028654 * (h + 0.044715 * h ** 3)))
        x = x + h @ f[f"{p}.mlp.proj.weight"] + f[f"{p}.mlp.proj.bias"]
    return ln(x, f["ln_f.gamma"], f["ln_f.beta"]) @ f["wte"].T


def step_feeds(cfg: Gpt2Config, input_ids: np.ndarray, past: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """Feeds of one call: `input_ids` are the new tokens that follow the tokens already in `past`."""
    B, S = input_ids.shape
    P = next(iter(past.values())).shape[3]
    feeds = {"input_ids": input_ids.astype(np.int32), "position_ids": np.tile(np.arange(P, P + S, dtype=np.int32), (B, 1)),
             "attention_mask": np.ones((B, P + S), np.int32)}
    feeds.update(past)
    return feeds
