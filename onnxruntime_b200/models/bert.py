"""BERT-style encoder as an (unfused) ONNX graph, plus an independent numpy restatement.

The graph is emitted the way a framework exporter emits it: LayerNorm as
ReduceMean/Sub/Pow/Sqrt/Div, GELU as the erf formula, attention as separate
Q/K/V MatMul+Add, Reshape, Transpose, scaled QK^T, additive mask, Softmax.  The
session's optimizer is expected to rediscover ``EmbedLayerNormalization``,
``Attention``, ``SkipLayerNormalization`` and ``BiasGelu`` in it (the reference's
fusion tests build their inputs the same way:
onnxruntime/test/python/transformers/bert_model_generator.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class BertConfig:
    vocab_size: int = 1000
    hidden_size: int = 128
    num_layers: int = 2
    num_heads: int = 2
    ffn_size: int = 512
    max_position: int = 64
    type_vocab_size: int = 0       # 0 = no segment embedding
    layer_norm_eps: float = 1e-12
    dtype: str = "fp32"            # fp32 | fp16
    gelu: str = "erf"              # erf | tanh

    @staticmethod
    def tiny() -> "BertConfig":
        return BertConfig()

    @staticmethod
    def bert_large(**kw) -> "BertConfig":
        base = dict(vocab_size=30522, hidden_size=1024, num_layers=24, num_heads=16, ffn_size=4096, max_position=512,
                    dtype="fp16")
        base.update(kw)
        return BertConfig(**base)


def init_weights(cfg: BertConfig, seed: int = 0) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    dt = np.float16 if cfg.dtype == "fp16" else np.float32
    H, F = cfg.hidden_size, cfg.ffn_size
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape):
        w[name] = (rng.randn(*shape) * 0.02).astype(dt)

    n("embeddings.word", cfg.vocab_size, H)
    n("embeddings.position", cfg.max_position, H)
    if cfg.type_vocab_size:
        n("embeddings.token_type", cfg.type_vocab_size, H)
    w["embeddings.ln.gamma"] = np.ones(H, dt)
    w["embeddings.ln.beta"] = np.zeros(H, dt)
    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        for nm in ("q", "k", "v", "o"):
            n(f"{p}.attn.{nm}.weight", H, H)
            w[f"{p}.attn.{nm}.bias"] = (rng.randn(H) * 0.02).astype(dt)
        w[f"{p}.attn.ln.gamma"] = np.ones(H, dt)
        w[f"{p}.attn.ln.beta"] = np.zeros(H, dt)
        n(f"{p}.ffn.fc1.weight", H, F)
        w[f"{p}.ffn.fc1.bias"] = (rng.randn(F) * 0.02).astype(dt)
        n(f"{p}.ffn.fc2.weight", F, H)
        w[f"{p}.ffn.fc2.bias"] = (rng.randn(H) * 0.02).astype(dt)
        w[f"{p}.ffn.ln.gamma"] = np.ones(H, dt)
        w[f"{p}.ffn.ln.beta"] = np.zeros(H, dt)
    return w


class _Builder:
    def __init__(self, dt):
        self.nodes: List[ol.Node] = []
        self.inits: List[ol.Tensor] = []
        self.count = 0
        self.dt = dt

    def name(self, prefix: str) -> str:
        self.count += 1
        return f"{prefix}_{self.count}"

    def const(self, value, dtype=None) -> str:
        nm = self.name("const")
        self.inits.append(ol.make_tensor(nm, np.asarray(value, dtype=dtype if dtype is not None else self.dt)))
        return nm

    def op(self, op_type: str, inputs, n_out: int = 1, domain: str = "", **attrs):
        outs = [self.name(op_type.lower()) for _ in range(n_out)]
        self.nodes.append(ol.make_node(op_type, inputs, outs, name=self.name(op_type + "_node"), domain=domain, **attrs))
        return outs[0] if n_out == 1 else outs

    def layer_norm(self, x: str, gamma: str, beta: str, eps: float) -> str:
        mean = self.op("ReduceMean", [x], axes=[-1], keepdims=1)
        d = self.op("Sub", [x, mean])
        sq = self.op("Pow", [d, self.const(2.0)])
        var = self.op("ReduceMean", [sq], axes=[-1], keepdims=1)
        std = self.op("Sqrt", [self.op("Add", [var, self.const(eps)])])
        return self.op("Add", [self.op("Mul", [self.op("Div", [d, std]), gamma]), beta])

    def gelu(self, x: str, kind: str) -> str:
        if kind == "erf":
            e = self.op("Erf", [self.op("Div", [x, self.const(math.sqrt(2.0))])])
            return self.op("Mul", [self.op("Mul", [x, self.op("Add", [e, self.const(1.0)])]), self.const(0.5)])
        x3 = self.op("Pow", [x, self.const(3.0)])
        inner = self.op("Mul", [self.const(math.sqrt(2.0 / math.pi)), self.op("Add", [x, self.op("Mul", [self.const(0.044715), x3])])])
        t = self.op("Add", [self.const(1.0), self.op("Tanh", [inner])])
        return self.op("Mul", [self.op("Mul", [x, self.const(0.5)]), t])


def build_bert(cfg: BertConfig, weights: Dict[str, np.ndarray] = None, seed: int = 0, opset: int = 17) -> bytes:
    dt = np.float16 if cfg.dtype == "fp16" else np.float32
    odt = T.FLOAT16 if cfg.dtype == "fp16" else T.FLOAT
    w = weights if weights is not None else init_weights(cfg, seed)
    b = _Builder(dt)
    for k, v in w.items():
        b.inits.append(ol.make_tensor(k, v))
    H, N = cfg.hidden_size, cfg.num_heads
    hd = H // N
    inputs = [ol.make_tensor_value_info("input_ids", T.INT64, ["batch", "seq"]),
              ol.make_tensor_value_info("attention_mask", T.INT64, ["batch", "seq"])]
    if cfg.type_vocab_size:
        inputs.append(ol.make_tensor_value_info("token_type_ids", T.INT64, ["batch", "seq"]))

    # embeddings: word + position (ids 0..S-1 sliced from a constant row) (+ segment), LayerNorm
    word = b.op("Gather", ["embeddings.word", "input_ids"], axis=0)
    shape = b.op("Shape", ["input_ids"])
    seq = b.op("Gather", [shape, b.const(1, np.int64)], axis=0)
    pos_row = b.const(np.arange(cfg.max_position, dtype=np.int64).reshape(1, -1), np.int64)
    pos_ids = b.op("Slice", [pos_row, b.const([0], np.int64), b.op("Unsqueeze", [seq, b.const([0], np.int64)]),
                             b.const([1], np.int64)])
    pos = b.op("Gather", ["embeddings.position", pos_ids], axis=0)
    emb = b.op("Add", [word, pos])
    if cfg.type_vocab_size:
        emb = b.op("Add", [emb, b.op("Gather", ["embeddings.token_type", "token_type_ids"], axis=0)])
    x = b.layer_norm(emb, "embeddings.ln.gamma", "embeddings.ln.beta", cfg.layer_norm_eps)

    # additive mask [B,1,1,S]: (1 - mask) * -10000
    m = b.op("Unsqueeze", [b.op("Unsqueeze", ["attention_mask", b.const([1], np.int64)]), b.const([2], np.int64)])
    mf = b.op("Cast", [m], to=odt)
    add_mask = b.op("Mul", [b.op("Sub", [b.const(1.0), mf]), b.const(-10000.0)])

    shape4 = b.const([0, 0, N, hd], np.int64)
    shape3 = b.const([0, 0, H], np.int64)
    for i in range(cfg.num_layers):
        p = f"layer.{i}"

        def proj(nm: str, src: str) -> str:
            return b.op("Add", [b.op("MatMul", [src, f"{p}.attn.{nm}.weight"]), f"{p}.attn.{nm}.bias"])
        q = b.op("Transpose", [b.op("Reshape", [proj("q", x), shape4])], perm=[0, 2, 1, 3])
        k = b.op("Transpose", [b.op("Reshape", [proj("k", x), shape4])], perm=[0, 2, 3, 1])
        v = b.op("Transpose", [b.op("Reshape", [proj("v", x), shape4])], perm=[0, 2, 1, 3])
        scores = b.op("Div", [b.op("MatMul", [q, k]), b.const(math.sqrt(hd))])
        probs = b.op("Softmax", [b.op("Add", [scores, add_mask])], axis=-1)
        ctx = b.op("Reshape", [b.op("Transpose", [b.op("MatMul", [probs, v])], perm=[0, 2, 1, 3]), shape3])
        attn_out = b.op("Add", [b.op("MatMul", [ctx, f"{p}.attn.o.weight"]), f"{p}.attn.o.bias"])
        x = b.layer_norm(b.op("Add", [attn_out, x]), f"{p}.attn.ln.gamma", f"{p}.attn.ln.beta", cfg.layer_norm_eps)
        h = b.gelu(b.op("Add", [b.op("MatMul", [x, f"{p}.ffn.fc1.weight"]), f"{p}.ffn.fc1.bias"]), cfg.gelu)
        ffn_out = b.op("Add", [b.op("MatMul", [h, f"{p}.ffn.fc2.weight"]), f"{p}.ffn.fc2.bias"])
        x = b.layer_norm(b.op("Add", [ffn_out, x]), f"{p}.ffn.ln.gamma", f"{p}.ffn.ln.beta", cfg.layer_norm_eps)
    b.nodes.append(ol.make_node("Identity", [x], ["last_hidden_state"], name="output"))
    graph = ol.make_graph(b.nodes, "bert", inputs, [ol.make_tensor_value_info("last_hidden_state", odt, ["batch", "seq", H])],
                          b.inits)
    return ol.make_model(graph, opset=opset).serialize()


def build_bert_fp8(cfg: BertConfig, weights: Dict[str, np.ndarray] = None, seed: int = 0, opset: int = 17) -> bytes:
    """The same encoder as a quantisation tool would emit it for fp8 serving (the reference serves fp8 through
    com.microsoft GemmFloat8, onnxruntime/contrib_ops/cuda/math/gemm_float8.cc): every dense layer is
    ``GemmFloat8(Cast_e4m3(activation), W_e4m3, bias, scaleA = 1, scaleB)`` with a per-tensor weight scale, the merged QKV
    projection feeds ``MultiHeadAttention`` in its packed form, residual + LayerNorm are ``SkipLayerNormalization`` and
    the GELU rides in the first FFN GEMM.  Activations (LayerNorm / GELU outputs, O(1) magnitudes) are cast to e4m3
    directly, so scaleA is 1.  Hidden states stay fp16."""
    import torch
    assert cfg.dtype == "fp16", "the fp8 graph keeps fp16 hidden states"
    w = weights if weights is not None else init_weights(cfg, seed)
    b = _Builder(np.float16)
    H, N, F = cfg.hidden_size, cfg.num_heads, cfg.ffn_size
    hd = H // N

    def add(name, arr):
        b.inits.append(ol.make_tensor(name, arr))
        return name

    def fp8_weight(name: str, mat: np.ndarray):
        """[K, N] fp16 -> e4m3 initializer + fp32 scale (amax mapped to 448)"""
        m = torch.from_numpy(mat.astype(np.float32))
        scale = float(m.abs().max()) / 448.0 or 1.0
        add(name, (m / scale).to(torch.float8_e4m3fn))
        add(name + ".scale", np.array([scale], np.float32))
        return name, name + ".scale"

    for k in ("embeddings.word", "embeddings.position", "embeddings.ln.gamma", "embeddings.ln.beta"):
        add(k, w[k])
    one = add("unit_scale", np.array([1.0], np.float32))
    inputs = [ol.make_tensor_value_info("input_ids", T.INT64, ["batch", "seq"]), ol.make_tensor_value_info("attention_mask", T.INT64, ["batch", "seq"])]
    mask32 = b.op("Cast", ["attention_mask"], to=T.INT32)
    x3 = b.op("EmbedLayerNormalization", ["input_ids", "", "embeddings.word", "embeddings.position", "", "embeddings.ln.gamma", "embeddings.ln.beta"],
              n_out=2, domain="com.microsoft", epsilon=cfg.layer_norm_eps)[0]
    flat = b.const([-1, H], np.int64)
    x = b.op("Reshape", [x3, flat])                                     # [T, H] from here on
    shape_in = b.op("Shape", ["input_ids"])
    packed_shape = b.op("Concat", [shape_in, b.const([N, 3, hd], np.int64)], axis=0)

    def gemm8(src: str, wname: str, sname: str, bias: str, act: str = "NONE") -> str:
        q = b.op("Cast", [src], to=T.FLOAT8E4M3FN, saturate=1)
        return b.op("GemmFloat8", [q, wname, bias, one, sname], domain="com.microsoft", dtype=T.FLOAT16, beta=1.0, activation=act)

    for i in range(cfg.num_layers):
        p = f"layer.{i}"
        # merged QKV with columns ordered [head, (q, k, v), head_dim]: the product is MultiHeadAttention's packed input
        cols = np.stack([w[f"{p}.attn.{nm}.weight"].reshape(H, N, hd) for nm in ("q", "k", "v")], 2).reshape(H, 3 * H)
        bias = np.stack([w[f"{p}.attn.{nm}.bias"].reshape(N, hd) for nm in ("q", "k", "v")], 1).reshape(3 * H)
        wq, sq = fp8_weight(f"{p}.attn.qkv.weight", cols)
        qkv = gemm8(x, wq, sq, add(f"{p}.attn.qkv.bias", bias.astype(np.float16)))
        packed = b.op("Reshape", [qkv, packed_shape])
        ctx = b.op("MultiHeadAttention", [packed, "", "", "", mask32], domain="com.microsoft", num_heads=N)
        wo, so = fp8_weight(f"{p}.attn.o.weight", w[f"{p}.attn.o.weight"])
        attn_out = gemm8(b.op("Reshape", [ctx, flat]), wo, so, add(f"{p}.attn.o.bias", w[f"{p}.attn.o.bias"]))
        x = b.op("SkipLayerNormalization", [attn_out, x, add(f"{p}.attn.ln.gamma", w[f"{p}.attn.ln.gamma"]), add(f"{p}.attn.ln.beta", w[f"{p}.attn.ln.beta"])],
                 domain="com.microsoft", epsilon=cfg.layer_norm_eps)
        w1, s1 = fp8_weight(f"{p}.ffn.fc1.weight", w[f"{p}.ffn.fc1.weight"])
        h = gemm8(x, w1, s1, add(f"{p}.ffn.fc1.bias", w[f"{p}.ffn.fc1.bias"]), act="GELU")
        w2, s2 = fp8_weight(f"{p}.ffn.fc2.weight", w[f"{p}.ffn.fc2.weight"])
        ffn_out = gemm8(h, w2, s2, add(f"{p}.ffn.fc2.bias", w[f"{p}.ffn.fc2.bias"]))
        x = b.op("SkipLayerNormalization", [ffn_out, x, add(f"{p}.ffn.ln.gamma", w[f"{p}.ffn.ln.gamma"]), add(f"{p}.ffn.ln.beta", w[f"{p}.ffn.ln.beta"])],
                 domain="com.microsoft", epsilon=cfg.layer_norm_eps)
    out_shape = b.op("Concat", [shape_in, b.const([H], np.int64)], axis=0)
    b.nodes.append(ol.make_node("Reshape", [x, out_shape], ["last_hidden_state"], name="output"))
    graph = ol.make_graph(b.nodes, "bert_fp8", inputs, [ol.make_tensor_value_info("last_hidden_state", T.FLOAT16, ["batch", "seq", H])], b.inits)
    return ol.make_model(graph, opset=opset).serialize()


def reference_forward(cfg: BertConfig, w: Dict[str, np.ndarray], input_ids: np.ndarray, attention_mask: np.ndarray,
                      token_type_ids: np.ndarray = None) -> np.ndarray:
    """Plain numpy fp32 restatement of the encoder math (the oracle for the session's output)."""
    f = {k: v.astype(np.float64) for k, v in w.items()}
    H, N = cfg.hidden_size, cfg.num_heads
    hd = H // N
    B, S = input_ids.shape

    def ln(x, g, bta):
        mu = x.mean(-1, keepdims=True)
        var = ((x - mu) ** 2).mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(var + cfg.layer_norm_eps) * g + bta

    def gelu(x):
        if cfg.gelu == "erf":
            from math import erf
            return 0.5 * x * (1.0 + np.vectorize(erf)(x / math.sqrt(2.0)))
        return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))

    x = f["embeddings.word"][input_ids] + f["embeddings.position"][np.arange(S)][None]
    if cfg.type_vocab_size:
        x = x + f["embeddings.token_type"][token_type_ids]
    x = ln(x, f["embeddings.ln.gamma"], f["embeddings.ln.beta"])
    add_mask = (1.0 - attention_mask.astype(np.float64))[:, None, None, :] * -10000.0
    for i in range(cfg.num_layers):
        p = f"layer.{i}"

        def heads(t):
            return t.reshape(B, S, N, hd).transpose(0, 2, 1, 3)
        q = heads(x @ f[f"{p}.attn.q.weight"] + f[f"{p}.attn.q.bias"])
        k = heads(x @ f[f"{p}.attn.k.weight"] + f[f"{p}.attn.k.bias"])
        v = heads(x @ f[f"{p}.attn.v.weight"] + f[f"{p}.attn.v.bias"])
        s = q @ k.transpose(0, 1, 3, 2) / math.sqrt(hd) + add_mask
        s = s - s.max(-1, keepdims=True)
        pr = np.exp(s)
        pr = pr / pr.sum(-1, keepdims=True)
        ctx = (pr @ v).transpose(0, 2, 1, 3).reshape(B, S, H)
        x = ln(ctx @ f[f"{p}.attn.o.weight"] + f[f"{p}.attn.o.bias"] + x, f[f"{p}.attn.ln.gamma"], f[f"{p}.attn.ln.beta"])
        h = gelu(x @ f[f"{p}.ffn.fc1.weight"] + f[f"{p}.ffn.fc1.bias"])
        x = ln(h @ f[f"{p}.ffn.fc2.weight"] + f[f"{p}.ffn.fc2.bias"] + x, f[f"{p}.ffn.ln.gamma"], f[f"{p}.ffn.ln.beta"])
    return x.astype(np.float32)
