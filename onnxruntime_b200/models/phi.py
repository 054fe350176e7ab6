"""Phi-2-style decoder as an ONNX graph, plus a numpy restatement.

The block shape of the reference's Phi-2 export (onnxruntime/python/tools/transformers/models/phi2/convert_to_onnx.py,
fusion_options for ``phi``): one LayerNormalization per layer feeding BOTH the attention and the MLP, whose outputs are added
to the residual together (parallel block); linear layers with bias; rotary embedding on the first ``rotary_dim`` channels of
every head only, done inside ``GroupQueryAttention`` (cos / sin caches of rotary_dim / 2 columns); tanh-form GELU
(``FastGelu``); a final LayerNormalization and an output projection with bias.  KV caches are the operator's
past / present pairs [batch, heads, sequence, head].

Inputs: input_ids [B, S] int64, seqlens_k [B] int32 (tokens in the cache after this call, minus one),
total_sequence_length (int32 scalar), past_key_values.{i}.key / .value; outputs: logits, present.{i}.key / .value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class PhiConfig:
    vocab_size: int = 300
    hidden_size: int = 64
    num_layers: int = 2
    num_heads: int = 4
    rotary_dim: int = 8           # of head_dim = hidden_size / num_heads channels
    ffn_size: int = 256
    max_seq_len: int = 64
    rope_theta: float = 10000.0
    layer_norm_eps: float = 1e-5

    @staticmethod
    def phi2(**kw) -> "PhiConfig":
        base = dict(vocab_size=51200, hidden_size=2560, num_layers=32, num_heads=32, rotary_dim=32, ffn_size=10240, max_seq_len=2048)
        base.update(kw)
        return PhiConfig(**base)


def init_weights(cfg: PhiConfig, seed: int = 0, scale: float = 0.05) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    H, F = cfg.hidden_size, cfg.ffn_size
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape):
        w[name] = (rng.randn(*shape) * scale).astype(np.float32)

    n("embed", cfg.vocab_size, H)
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        w[p + ".ln.gamma"] = (1.0 + rng.randn(H) * 0.02).astype(np.float32)
        w[p + ".ln.beta"] = (rng.randn(H) * 0.02).astype(np.float32)
        n(p + ".qkv.weight", H, 3 * H), n(p + ".qkv.bias", 3 * H), n(p + ".dense.weight", H, H), n(p + ".dense.bias", H)
        n(p + ".fc1.weight", H, F), n(p + ".fc1.bias", F), n(p + ".fc2.weight", F, H), n(p + ".fc2.bias", H)
    w["final_ln.gamma"] = (1.0 + rng.randn(H) * 0.02).astype(np.float32)
    w["final_ln.beta"] = (rng.randn(H) * 0.02).astype(np.float32)
    n("lm_head.weight", H, cfg.vocab_size), n("lm_head.bias", cfg.vocab_size)
    return w


def rope_caches(cfg: PhiConfig):
    half = cfg.rotary_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (np.arange(half, dtype=np.float64) / half))
    ang = np.outer(np.arange(cfg.max_seq_len, dtype=np.float64), inv)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def build_phi(cfg: PhiConfig, weights: Optional[Dict[str, np.ndarray]] = None, seed: int = 0, opset: int = 17) -> bytes:
    w = weights if weights is not None else init_weights(cfg, seed)
    N, hd = cfg.num_heads, cfg.hidden_size // cfg.num_heads
    cos, sin = rope_caches(cfg)
    inits = [ol.make_tensor(k, v) for k, v in w.items()] + [ol.make_tensor("cos_cache", cos), ol.make_tensor("sin_cache", sin)]
    nodes: List[ol.Node] = []
    count = [0]

    def op(op_type, inputs, outputs=None, domain="", **attrs):
        count[0] += 1
        outs = outputs or [f"{op_type.lower()}_{count[0]}"]
        nodes.append(ol.make_node(op_type, inputs, outs, name=f"{op_type}_{count[0]}", domain=domain, **attrs))
        return outs[0]

    vi = ol.make_tensor_value_info
    inputs = [vi("input_ids", T.INT64, ["batch", "seq"]), vi("seqlens_k", T.INT32, ["batch"]), vi("total_sequence_length", T.INT32, [])]
    outputs = [vi("logits", T.FLOAT, ["batch", "seq", cfg.vocab_size])]
    x = op("Gather", ["embed", "input_ids"], axis=0)
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        inputs += [vi(f"past_key_values.{i}.key", T.FLOAT, ["batch", N, "past", hd]), vi(f"past_key_values.{i}.value", T.FLOAT, ["batch", N, "past", hd])]
        outputs += [vi(f"present.{i}.key", T.FLOAT, ["batch", N, "total", hd]), vi(f"present.{i}.value", T.FLOAT, ["batch", N, "total", hd])]
        h = op("LayerNormalization", [x, p + ".ln.gamma", p + ".ln.beta"], axis=-1, epsilon=cfg.layer_norm_eps)
        qkv = op("Add", [op("MatMul", [h, p + ".qkv.weight"]), p + ".qkv.bias"])
        count[0] += 1
        attn = f"attn_{count[0]}"
        nodes.append(ol.make_node("GroupQueryAttention", [qkv, "", "", f"past_key_values.{i}.key", f"past_key_values.{i}.value", "seqlens_k",
                                                          "total_sequence_length", "cos_cache", "sin_cache"],
                                  [attn, f"present.{i}.key", f"present.{i}.value"], name=f"{p}.attn", domain="com.microsoft", num_heads=N, kv_num_heads=N,
                                  do_rotary=1, rotary_interleaved=0))
        a = op("Add", [op("MatMul", [attn, p + ".dense.weight"]), p + ".dense.bias"])
        m = op("FastGelu", [op("MatMul", [h, p + ".fc1.weight"]), p + ".fc1.bias"], domain="com.microsoft")
        m = op("Add", [op("MatMul", [m, p + ".fc2.weight"]), p + ".fc2.bias"])
        x = op("Add", [x, op("Add", [a, m])])
    xf = op("LayerNormalization", [x, "final_ln.gamma", "final_ln.beta"], axis=-1, epsilon=cfg.layer_norm_eps)
    op("Add", [op("MatMul", [xf, "lm_head.weight"]), "lm_head.bias"], ["logits"])
    model = ol.make_model(ol.make_graph(nodes, "phi", inputs, outputs, inits), opset=opset)
    model.opset_imports["com.microsoft"] = 1
    return model.serialize()


def empty_past(cfg: PhiConfig, batch: int) -> Dict[str, np.ndarray]:
    hd = cfg.hidden_size // cfg.num_heads
    out = {}
    for i in range(cfg.num_layers):
        out[f"past_key_values.{i}.key"] = np.zeros((batch, cfg.num_heads, 0, hd), np.float32)
        out[f"past_key_values.{i}.value"] = np.zeros((batch, cfg.num_heads, 0, hd), np.float32)
    return out


def step_feeds(cfg: PhiConfig, input_ids: np.ndarray, past: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    B, S = input_ids.shape
    P = past["past_key_values.0.key"].shape[2]
    feeds = {"input_ids": input_ids.astype(np.int64), "seqlens_k": np.full(B, P + S - 1, np.int32), "total_sequence_length": np.array(P + S, np.int32)}
    feeds.update(past)
    return feeds


def reference_forward(cfg: PhiConfig, w: Dict[str, np.ndarray], input_ids: np.ndarray) -> np.ndarray:
    """Logits of a whole sequence in one causal pass (float64)."""
    f = {k: v.astype(np.float64) for k, v in w.items()}
    B, S = input_ids.shape
    H, N = cfg.hidden_size, cfg.num_heads
    hd, rd = H // N, cfg.rotary_dim
    cos, sin = (c.astype(np.float64)[:S] for c in rope_caches(cfg))

    def ln(x, g, b):
        mu = x.mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(((x - mu) ** 2).mean(-1, keepdims=True) + cfg.layer_norm_eps) * g + b

    def rope(t):  # [B, N, S, hd]: rotate-half on the first rd channels
        r, rest = t[..., :rd], t[..., rd:]
        x1, x2 = r[..., :rd // 2], r[..., rd // 2:]
        c, s = cos[None, None], sin[None, None]
        return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s, rest], -1)

    x = f["embed"][input_ids]
    causal = np.where(np.tril(np.ones((S, S), bool)), 0.0, -np.inf)[None, None]
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        h = ln(x, f[p + ".ln.gamma"], f[p + ".ln.beta"])
        qkv = h @ f[p + ".qkv.weight"] + f[p + ".qkv.bias"]
        q, k, v = (t.reshape(B, S, N, hd).transpose(0, 2, 1, 3) for t in np.split(qkv, 3, -1))
        q, k = rope(q), rope(k)
        s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(hd) + causal
        pr = np.exp(s - s.max(-1, keepdims=True))
        pr = pr / pr.sum(-1, keepdims=True)
        a = (pr @ v).transpose(0, 2, 1, 3).reshape(B, S, H) @ f[p + ".dense.weight"] + f[p + ".dense.bias"]
        m = h @ f[p + ".fc1.weight"] + f[p + ".fc1.bias"]
        m = 0.5 * m * (1.0 + np.tanh(0.7978845608028654 * (m + 0.044715 * m ** 3)))
        x = x + a + m @ f[p + ".fc2.weight"] + f[p + ".fc2.bias"]
    return ln(x, f["final_ln.gamma"], f["final_ln.beta"]) @ f["lm_head.weight"] + f["lm_head.bias"]
