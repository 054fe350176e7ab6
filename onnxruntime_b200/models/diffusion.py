"""A latent-diffusion UNet stage (ResNet block + spatial transformer block) in the operators the reference's Stable
Diffusion optimisation produces (onnxruntime/python/tools/transformers/onnx_model_unet.py, fusion_group_norm.py,
fusion_nhwc_conv.py, fusion_bias_split_gelu.py, fusion_bias_add.py, fusion_attention_unet.py): channels-last tensors
between ``GroupNorm`` (with fused SiLU) and ``NhwcConv``, ``MultiHeadAttention`` for the self and the text cross
attention, ``BiasSplitGelu`` for the GEGLU feed-forward and ``BiasAdd`` for projection bias + residual.

Inputs: sample [N, C, H, W], time_embedding [N, T], encoder_hidden_states [N, S_text, D_text]; output [N, C, H, W].
``reference_forward`` restates the stage in plain torch (float64).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class UNetStageConfig:
    channels: int = 32
    groups: int = 8
    heads: int = 4
    time_dim: int = 24
    text_dim: int = 20
    eps: float = 1e-5


def init_weights(cfg: UNetStageConfig, seed: int = 0) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    C = cfg.channels
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape, scale=0.08):
        w[name] = (rng.randn(*shape) * scale).astype(np.float32)

    for gn in ("res.gn1", "res.gn2", "attn.gn"):
        w[gn + ".gamma"] = (1.0 + rng.randn(C) * 0.05).astype(np.float32)
        w[gn + ".beta"] = (rng.randn(C) * 0.05).astype(np.float32)
    n("res.conv1.weight", C, C, 3, 3), n("res.conv1.bias", C), n("res.conv2.weight", C, C, 3, 3), n("res.conv2.bias", C)
    n("res.time.weight", cfg.time_dim, C), n("res.time.bias", C)
    n("attn.proj_in.weight", C, C), n("attn.proj_in.bias", C), n("attn.proj_out.weight", C, C), n("attn.proj_out.bias", C)
    for ln in ("attn.ln1", "attn.ln2", "attn.ln3"):
        w[ln + ".gamma"] = (1.0 + rng.randn(C) * 0.05).astype(np.float32)
        w[ln + ".beta"] = (rng.randn(C) * 0.05).astype(np.float32)
    for p in ("q", "k", "v"):
        n(f"attn.self.{p}.weight", C, C)
    n("attn.self.o.weight", C, C), n("attn.self.o.bias", C)
    n("attn.cross.q.weight", C, C), n("attn.cross.k.weight", cfg.text_dim, C), n("attn.cross.v.weight", cfg.text_dim, C)
    n("attn.cross.o.weight", C, C), n("attn.cross.o.bias", C)
    n("attn.ff.in.weight", C, 8 * C), n("attn.ff.in.bias", 8 * C), n("attn.ff.out.weight", 4 * C, C), n("attn.ff.out.bias", C)
    return w


def build_unet_stage(cfg: UNetStageConfig, weights: Optional[Dict[str, np.ndarray]] = None, seed: int = 0, opset: int = 17) -> bytes:
    w = weights if weights is not None else init_weights(cfg, seed)
    C = cfg.channels
    nodes: List[ol.Node] = []
    inits: Dict[str, ol.Tensor] = {}
    count = [0]

    def wt(name, value=None):
        if name not in inits:
            inits[name] = ol.make_tensor(name, w[name] if value is None else value)
        return name

    def const(value, dtype):
        count[0] += 1
        name = f"c_{count[0]}"
        inits[name] = ol.make_tensor(name, np.asarray(value, dtype=dtype))
        return name

    def op(op_type, inputs, domain="", outputs=None, **attrs):
        count[0] += 1
        outs = outputs or [f"{op_type.lower()}_{count[0]}"]
        nodes.append(ol.make_node(op_type, inputs, outs, name=f"{op_type}_{count[0]}", domain=domain, **attrs))
        return outs[0]

    MS = "com.microsoft"

    def group_norm(x, name, silu):
        return op("GroupNorm", [x, wt(name + ".gamma"), wt(name + ".beta")], MS, activation=int(silu), channels_last=1, epsilon=cfg.eps, groups=cfg.groups)

    def nhwc_conv(x, name):
        # filters channels-last as well: (M, kH, kW, C)
        return op("NhwcConv", [x, wt(name + ".weight_nhwc", np.ascontiguousarray(w[name + ".weight"].transpose(0, 2, 3, 1))), wt(name + ".bias")], MS,
                  kernel_shape=[3, 3], pads=[1, 1, 1, 1])

    def layer_norm(x, name):
        return op("LayerNormalization", [x, wt(name + ".gamma"), wt(name + ".beta")], axis=-1, epsilon=cfg.eps)

    # ---- ResNet block, channels-last inside
    x = op("Transpose", ["sample"], perm=[0, 2, 3, 1])
    h = nhwc_conv(group_norm(x, "res.gn1", True), "res.conv1")
    t = op("Add", [op("MatMul", [op("Mul", ["time_embedding", op("Sigmoid", ["time_embedding"])]), wt("res.time.weight")]), wt("res.time.bias")])
    h = op("Add", [h, op("Unsqueeze", [t, const([1, 2], np.int64)])])
    h = nhwc_conv(group_norm(h, "res.gn2", True), "res.conv2")
    x = op("Add", [x, h])
    # ---- spatial transformer: tokens = pixels
    res = x
    tokens = op("Reshape", [group_norm(x, "attn.gn", False), const([0, -1, C], np.int64)])
    hs = op("Add", [op("MatMul", [tokens, wt("attn.proj_in.weight")]), wt("attn.proj_in.bias")])
    n1 = layer_norm(hs, "attn.ln1")
    q, k, v = (op("MatMul", [n1, wt(f"attn.self.{p}.weight")]) for p in "qkv")
    sa = op("MultiHeadAttention", [q, k, v], MS, num_heads=cfg.heads)
    hs = op("BiasAdd", [op("MatMul", [sa, wt("attn.self.o.weight")]), wt("attn.self.o.bias"), hs], MS)
    n2 = layer_norm(hs, "attn.ln2")
    ca = op("MultiHeadAttention", [op("MatMul", [n2, wt("attn.cross.q.weight")]), op("MatMul", ["encoder_hidden_states", wt("attn.cross.k.weight")]),
                                   op("MatMul", ["encoder_hidden_states", wt("attn.cross.v.weight")])], MS, num_heads=cfg.heads)
    hs = op("BiasAdd", [op("MatMul", [ca, wt("attn.cross.o.weight")]), wt("attn.cross.o.bias"), hs], MS)
    n3 = layer_norm(hs, "attn.ln3")
    ff = op("BiasSplitGelu", [op("MatMul", [n3, wt("attn.ff.in.weight")]), wt("attn.ff.in.bias")], MS)
    hs = op("BiasAdd", [op("MatMul", [ff, wt("attn.ff.out.weight")]), wt("attn.ff.out.bias"), hs], MS)
    out_tokens = op("Add", [op("MatMul", [hs, wt("attn.proj_out.weight")]), wt("attn.proj_out.bias")])
    y = op("Add", [op("Reshape", [out_tokens, op("Shape", [res])]), res])
    op("Transpose", [y], outputs=["out_sample"], perm=[0, 3, 1, 2])
    vi = ol.make_tensor_value_info
    graph = ol.make_graph(nodes, "unet_stage", [vi("sample", T.FLOAT, ["n", C, "h", "w"]), vi("time_embedding", T.FLOAT, ["n", cfg.time_dim]),
                                                vi("encoder_hidden_states", T.FLOAT, ["n", "text", cfg.text_dim])],
                          [vi("out_sample", T.FLOAT, ["n", C, "h", "w"])], list(inits.values()))
    model = ol.make_model(graph, opset=opset)
    model.opset_imports["com.microsoft"] = 1
    return model.serialize()


def reference_forward(cfg: UNetStageConfig, w: Dict[str, np.ndarray], sample: np.ndarray, time_embedding: np.ndarray,
                      encoder_hidden_states: np.ndarray) -> np.ndarray:
    import torch
    import torch.nn.functional as F
    f = {k: torch.from_numpy(v).double() for k, v in w.items()}
    x, temb, text = (torch.from_numpy(a).double() for a in (sample, time_embedding, encoder_hidden_states))
    C, Hh = cfg.channels, cfg.heads

    def gn(t, name):
        return F.group_norm(t, cfg.groups, f[name + ".gamma"], f[name + ".beta"], cfg.eps)

    def ln(t, name):
        return F.layer_norm(t, (C,), f[name + ".gamma"], f[name + ".beta"], cfg.eps)

    def mha(q, k, v):
        B, S, _ = q.shape
        split = lambda t: t.reshape(B, t.shape[1], Hh, C // Hh).transpose(1, 2)
        a = torch.softmax(split(q) @ split(k).transpose(-1, -2) / (C // Hh) ** 0.5, -1) @ split(v)
        return a.transpose(1, 2).reshape(B, S, C)

    h = F.conv2d(F.silu(gn(x, "res.gn1")), f["res.conv1.weight"], f["res.conv1.bias"], padding=1)
    h = h + (F.silu(temb) @ f["res.time.weight"] + f["res.time.bias"])[:, :, None, None]
    h = F.conv2d(F.silu(gn(h, "res.gn2")), f["res.conv2.weight"], f["res.conv2.bias"], padding=1)
    x = x + h
    res = x
    N, _, H, W = x.shape
    hs = gn(x, "attn.gn").permute(0, 2, 3, 1).reshape(N, H * W, C) @ f["attn.proj_in.weight"] + f["attn.proj_in.bias"]
    n1 = ln(hs, "attn.ln1")
    hs = hs + mha(n1 @ f["attn.self.q.weight"], n1 @ f["attn.self.k.weight"], n1 @ f["attn.self.v.weight"]) @ f["attn.self.o.weight"] + f["attn.self.o.bias"]
    n2 = ln(hs, "attn.ln2")
    hs = hs + mha(n2 @ f["attn.cross.q.weight"], text @ f["attn.cross.k.weight"], text @ f["attn.cross.v.weight"]) @ f["attn.cross.o.weight"] + f["attn.cross.o.bias"]
    ff = ln(hs, "attn.ln3") @ f["attn.ff.in.weight"] + f["attn.ff.in.bias"]
    left, right = ff.chunk(2, -1)
    hs = hs + (left * F.gelu(right)) @ f["attn.ff.out.weight"] + f["attn.ff.out.bias"]
    out = (hs @ f["attn.proj_out.weight"] + f["attn.proj_out.bias"]).reshape(N, H, W, C).permute(0, 3, 1, 2)
    return (out + res).numpy()
