"""Encoder-decoder transformer (the T5 / BART shape) as the two ONNX graphs the generation operators drive, plus a numpy
restatement.

``build_encoder_decoder`` returns (encoder, decoder) in the form of the reference's T5 export
(onnxruntime/python/tools/transformers/models/t5/t5_encoder_decoder_init.py, t5_decoder.py):
  encoder (run once): encoder_input_ids [B, Se], encoder_attention_mask [B, Se], decoder_input_ids [B, Sd] (all int32) ->
      logits [B, Sd, V], encoder_hidden_states [B, Se, H] and per layer present_key_self, present_value_self
      [B, N, Sd, hd], present_key_cross, present_value_cross [B, N, Se, hd];
  decoder (per token): input_ids [R, 1], encoder_attention_mask [R, Se], then past_key_self / past_value_self of every
      layer, then past_key_cross / past_value_cross of every layer -> logits [R, 1, V] and the new self states.
Pre-LayerNorm blocks, learned position embeddings, ReLU feed-forward, tied output embedding.  ``convert_generation.convert(
decoder, op="beam" | "greedy", encoder=encoder, model_type=1, ...)`` wraps the pair into a BeamSearch / GreedySearch model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class EncoderDecoderConfig:
    vocab_size: int = 200
    hidden_size: int = 32
    num_heads: int = 4
    ffn_size: int = 64
    encoder_layers: int = 2
    decoder_layers: int = 2
    max_position: int = 64
    layer_norm_eps: float = 1e-5
    audio_features: int = 0        # > 0: Whisper shape - the encoder reads [batch, audio_features, frames] through two
                                   # Conv1d + GELU layers (the second with stride 2) instead of token ids, and has no mask


def init_weights(cfg: EncoderDecoderConfig, seed: int = 0, scale: float = 0.05) -> Dict[str, np.ndarray]:
    rng = np.random.RandomState(seed)
    H, F = cfg.hidden_size, cfg.ffn_size
    w: Dict[str, np.ndarray] = {}

    def n(name, *shape):
        w[name] = (rng.randn(*shape) * scale).astype(np.float32)

    def ln(name):
        w[name + ".gamma"] = (1.0 + rng.randn(H) * 0.02).astype(np.float32)
        w[name + ".beta"] = (rng.randn(H) * 0.02).astype(np.float32)

    def attn(name):
        for p in ("q", "k", "v", "o"):
            n(f"{name}.{p}.weight", H, H)
            n(f"{name}.{p}.bias", H)

    n("embed", cfg.vocab_size, H)
    if cfg.audio_features:
        n("enc.conv1.weight", H, cfg.audio_features, 3), n("enc.conv1.bias", H)
        n("enc.conv2.weight", H, H, 3), n("enc.conv2.bias", H)
    n("enc.pos", cfg.max_position, H)
    n("dec.pos", cfg.max_position, H)
    for i in range(cfg.encoder_layers):
        p = f"enc.{i}"
        ln(p + ".ln1"), attn(p + ".self"), ln(p + ".ln2")
        n(p + ".fc1.weight", H, F), n(p + ".fc1.bias", F), n(p + ".fc2.weight", F, H), n(p + ".fc2.bias", H)
    ln("enc.ln_f")
    for i in range(cfg.decoder_layers):
        p = f"dec.{i}"
        ln(p + ".ln1"), attn(p + ".self"), ln(p + ".ln2"), attn(p + ".cross"), ln(p + ".ln3")
        n(p + ".fc1.weight", H, F), n(p + ".fc1.bias", F), n(p + ".fc2.weight", F, H), n(p + ".fc2.bias", H)
    ln("dec.ln_f")
    return w


class _G:
    """Graph under construction; weights are added as initializers on first use."""

    def __init__(self, cfg: EncoderDecoderConfig, w: Dict[str, np.ndarray]):
        self.cfg, self.w = cfg, w
        self.nodes: List[ol.Node] = []
        self.inits: Dict[str, ol.Tensor] = {}
        self.count = 0

    def wt(self, name: str) -> str:
        if name not in self.inits:
            self.inits[name] = ol.make_tensor(name, self.w[name])
        return name

    def const(self, value, dtype) -> str:
        self.count += 1
        name = f"c_{self.count}"
        self.inits[name] = ol.make_tensor(name, np.asarray(value, dtype=dtype))
        return name

    def op(self, op_type, inputs, outputs=None, domain="", **attrs) -> str:
        self.count += 1
        outs = outputs or [f"{op_type.lower()}_{self.count}"]
        self.nodes.append(ol.make_node(op_type, inputs, outs, name=f"{op_type}_{self.count}", domain=domain, **attrs))
        return outs[0]

    def linear(self, x, name):
        return self.op("Add", [self.op("MatMul", [x, self.wt(name + ".weight")]), self.wt(name + ".bias")])

    def ln(self, x, name):
        return self.op("LayerNormalization", [x, self.wt(name + ".gamma"), self.wt(name + ".beta")], axis=-1, epsilon=self.cfg.layer_norm_eps)

    def heads(self, x):  # [B, S, H] -> [B, N, S, hd]
        N, hd = self.cfg.num_heads, self.cfg.hidden_size // self.cfg.num_heads
        return self.op("Transpose", [self.op("Reshape", [x, self.const([0, 0, N, hd], np.int64)])], perm=[0, 2, 1, 3])

    def attend(self, q, k, v, bias, name):  # q [B,N,Sq,hd], k / v [B,N,Sk,hd], bias broadcastable to [B,N,Sq,Sk] or None
        hd = self.cfg.hidden_size // self.cfg.num_heads
        s = self.op("Mul", [self.op("MatMul", [q, self.op("Transpose", [k], perm=[0, 1, 3, 2])]), self.const(1.0 / math.sqrt(hd), np.float32)])
        if bias is not None:
            s = self.op("Add", [s, bias])
        ctx = self.op("MatMul", [self.op("Softmax", [s], axis=-1), v])
        merged = self.op("Reshape", [self.op("Transpose", [ctx], perm=[0, 2, 1, 3]), self.const([0, 0, self.cfg.hidden_size], np.int64)])
        return self.linear(merged, name + ".o")

    def key_mask_bias(self, mask):  # [B, Sk] int32 -> additive [B, 1, 1, Sk]
        m = self.op("Cast", [self.op("Unsqueeze", [mask, self.const([1, 2], np.int64)])], to=T.FLOAT)
        return self.op("Mul", [self.op("Sub", [self.const(1.0, np.float32), m]), self.const(-10000.0, np.float32)])

    def embed(self, ids, pos_table, offset=None):  # token + position embedding; positions offset .. offset + S - 1
        tok = self.op("Gather", [self.wt("embed"), ids], axis=0)
        seq = self.op("Gather", [self.op("Shape", [ids]), self.const(1, np.int64)], axis=0)
        start = offset if offset is not None else self.const(0, np.int64)
        pos = self.op("Range", [start, self.op("Add", [start, seq]), self.const(1, np.int64)])
        return self.op("Add", [tok, self.op("Gather", [self.wt(pos_table), pos], axis=0)])

    def ffn(self, x, p):
        return self.linear(self.op("Relu", [self.linear(x, p + ".fc1")]), p + ".fc2")

    def audio_stem(self, features):  # [B, mels, frames] -> [B, frames / 2, H] + positions
        c1 = self.op("Gelu", [self.op("Conv", [features, self.wt("enc.conv1.weight"), self.wt("enc.conv1.bias")], kernel_shape=[3], pads=[1, 1])], domain="com.microsoft")
        c2 = self.op("Gelu", [self.op("Conv", [c1, self.wt("enc.conv2.weight"), self.wt("enc.conv2.bias")], kernel_shape=[3], pads=[1, 1], strides=[2])], domain="com.microsoft")
        x = self.op("Transpose", [c2], perm=[0, 2, 1])
        seq = self.op("Gather", [self.op("Shape", [x]), self.const(1, np.int64)], axis=0)
        pos = self.op("Range", [self.const(0, np.int64), seq, self.const(1, np.int64)])
        return self.op("Add", [x, self.op("Gather", [self.wt("enc.pos"), pos], axis=0)])

    def encoder(self, ids, mask):
        x = self.audio_stem(ids) if self.cfg.audio_features else self.embed(ids, "enc.pos")
        bias = self.key_mask_bias(mask) if mask is not None else None
        for i in range(self.cfg.encoder_layers):
            p = f"enc.{i}"
            h = self.ln(x, p + ".ln1")
            q, k, v = (self.heads(self.linear(h, f"{p}.self.{n}")) for n in "qkv")
            x = self.op("Add", [x, self.attend(q, k, v, bias, p + ".self")])
            x = self.op("Add", [x, self.ffn(self.ln(x, p + ".ln2"), p)])
        return self.ln(x, "enc.ln_f"), bias

    def logits(self, x):
        wt = "embed_t"
        if wt not in self.inits:
            self.inits[wt] = ol.make_tensor(wt, np.ascontiguousarray(self.w["embed"].T))
        return self.op("MatMul", [self.ln(x, "dec.ln_f"), wt], ["logits"])


def build_encoder_decoder(cfg: EncoderDecoderConfig, weights: Optional[Dict[str, np.ndarray]] = None, seed: int = 0,
                          opset: int = 17) -> Tuple[ol.Model, ol.Model]:
    w = weights if weights is not None else init_weights(cfg, seed)
    N, hd, L = cfg.num_heads, cfg.hidden_size // cfg.num_heads, cfg.decoder_layers
    vi = ol.make_tensor_value_info

    # ---- encoder + first decoder pass
    g = _G(cfg, w)
    audio = cfg.audio_features > 0
    enc, enc_bias = g.encoder("encoder_input_features" if audio else "encoder_input_ids", None if audio else "encoder_attention_mask")
    g.op("Identity", [enc], ["encoder_hidden_states"])
    x = g.embed("decoder_input_ids", "dec.pos")
    sd = g.op("Gather", [g.op("Shape", ["decoder_input_ids"]), g.const(1, np.int64)], axis=0)
    causal = g.op("Mul", [g.op("Sub", [g.const(1.0, np.float32), g.op("Trilu", [g.op("Expand", [g.const(1.0, np.float32), g.op("Concat", [g.op("Unsqueeze", [sd, g.const([0], np.int64)])] * 2, axis=0)])], upper=0)]),
                          g.const(-10000.0, np.float32)])
    outs = [vi("logits", T.FLOAT, ["batch", "dec_seq", cfg.vocab_size]), vi("encoder_hidden_states", T.FLOAT, ["batch", "enc_seq", cfg.hidden_size])]
    for i in range(L):
        p = f"dec.{i}"
        h = g.ln(x, p + ".ln1")
        q, k, v = (g.heads(g.linear(h, f"{p}.self.{n}")) for n in "qkv")
        g.op("Identity", [k], [f"present_key_self_{i}"]), g.op("Identity", [v], [f"present_value_self_{i}"])
        x = g.op("Add", [x, g.attend(q, k, v, causal, p + ".self")])
        h = g.ln(x, p + ".ln2")
        ck, cv = g.heads(g.linear(enc, p + ".cross.k")), g.heads(g.linear(enc, p + ".cross.v"))
        g.op("Identity", [ck], [f"present_key_cross_{i}"]), g.op("Identity", [cv], [f"present_value_cross_{i}"])
        x = g.op("Add", [x, g.attend(g.heads(g.linear(h, p + ".cross.q")), ck, cv, enc_bias, p + ".cross")])
        x = g.op("Add", [x, g.ffn(g.ln(x, p + ".ln3"), p)])
        outs += [vi(f"present_key_self_{i}", T.FLOAT, ["batch", N, "dec_seq", hd]), vi(f"present_value_self_{i}", T.FLOAT, ["batch", N, "dec_seq", hd]),
                 vi(f"present_key_cross_{i}", T.FLOAT, ["batch", N, "enc_seq", hd]), vi(f"present_value_cross_{i}", T.FLOAT, ["batch", N, "enc_seq", hd])]
    g.logits(x)
    ins = [vi("encoder_input_ids", T.INT32, ["batch", "enc_seq"]), vi("encoder_attention_mask", T.INT32, ["batch", "enc_seq"]),
           vi("decoder_input_ids", T.INT32, ["batch", "dec_seq"])]
    if audio:
        ins = [vi("encoder_input_features", T.FLOAT, ["batch", cfg.audio_features, "frames"]), vi("decoder_input_ids", T.INT32, ["batch", "dec_seq"])]
    encoder = ol.make_model(ol.make_graph(g.nodes, "encoder_decoder_init", ins, outs, list(g.inits.values())), opset=opset)
    encoder.opset_imports["com.microsoft"] = 1

    # ---- decoder step
    d = _G(cfg, w)
    ins = [vi("input_ids", T.INT32, ["rows", 1])] + ([] if audio else [vi("encoder_attention_mask", T.INT32, ["rows", "enc_seq"])])
    for i in range(L):
        ins += [vi(f"past_key_self_{i}", T.FLOAT, ["rows", N, "past", hd]), vi(f"past_value_self_{i}", T.FLOAT, ["rows", N, "past", hd])]
    for i in range(L):
        ins += [vi(f"past_key_cross_{i}", T.FLOAT, ["rows", N, "enc_seq", hd]), vi(f"past_value_cross_{i}", T.FLOAT, ["rows", N, "enc_seq", hd])]
    past_len = d.op("Gather", [d.op("Shape", ["past_key_self_0"]), d.const(2, np.int64)], axis=0)
    x = d.embed("input_ids", "dec.pos", offset=past_len)
    enc_bias = None if audio else d.key_mask_bias("encoder_attention_mask")
    outs = [vi("logits", T.FLOAT, ["rows", 1, cfg.vocab_size])]
    for i in range(L):
        p = f"dec.{i}"
        h = d.ln(x, p + ".ln1")
        q, k, v = (d.heads(d.linear(h, f"{p}.self.{n}")) for n in "qkv")
        k_all = d.op("Concat", [f"past_key_self_{i}", k], [f"present_key_self_{i}"], axis=2)
        v_all = d.op("Concat", [f"past_value_self_{i}", v], [f"present_value_self_{i}"], axis=2)
        x = d.op("Add", [x, d.attend(q, k_all, v_all, None, p + ".self")])
        h = d.ln(x, p + ".ln2")
        x = d.op("Add", [x, d.attend(d.heads(d.linear(h, p + ".cross.q")), f"past_key_cross_{i}", f"past_value_cross_{i}", enc_bias, p + ".cross")])
        x = d.op("Add", [x, d.ffn(d.ln(x, p + ".ln3"), p)])
        outs += [vi(f"present_key_self_{i}", T.FLOAT, ["rows", N, "total", hd]), vi(f"present_value_self_{i}", T.FLOAT, ["rows", N, "total", hd])]
    d.logits(x)
    decoder = ol.make_model(ol.make_graph(d.nodes, "decoder", ins, outs, list(d.inits.values())), opset=opset)
    return encoder, decoder


def reference_logits(cfg: EncoderDecoderConfig, w: Dict[str, np.ndarray], enc_ids: np.ndarray, enc_mask: Optional[np.ndarray], dec_ids: np.ndarray) -> np.ndarray:
    """Decoder logits [B, Sd, V] of one full pass (float64).  With cfg.audio_features, `enc_ids` holds the features
    [B, audio_features, frames] and `enc_mask` is None."""
    f = {k: v.astype(np.float64) for k, v in w.items()}
    H, N = cfg.hidden_size, cfg.num_heads
    hd = H // N

    def ln(x, name):
        mu = x.mean(-1, keepdims=True)
        return (x - mu) / np.sqrt(((x - mu) ** 2).mean(-1, keepdims=True) + cfg.layer_norm_eps) * f[name + ".gamma"] + f[name + ".beta"]

    def lin(x, name):
        return x @ f[name + ".weight"] + f[name + ".bias"]

    def heads(x):
        return x.reshape(x.shape[0], x.shape[1], N, hd).transpose(0, 2, 1, 3)

    def attend(xq, xkv, bias, name):
        q, k, v = heads(lin(xq, name + ".q")), heads(lin(xkv, name + ".k")), heads(lin(xkv, name + ".v"))
        s = q @ k.transpose(0, 1, 3, 2) / math.sqrt(hd) + bias
        p = np.exp(s - s.max(-1, keepdims=True))
        p = p / p.sum(-1, keepdims=True)
        return lin((p @ v).transpose(0, 2, 1, 3).reshape(xq.shape[0], xq.shape[1], H), name + ".o")

    def ffn(x, p):
        return lin(np.maximum(lin(x, p + ".fc1"), 0), p + ".fc2")

    def conv1d(x, name, stride):  # x [B, C, L], kernel 3, padding 1
        wt, b = f[name + ".weight"], f[name + ".bias"]
        xp = np.pad(x, ((0, 0), (0, 0), (1, 1)))
        cols = np.stack([xp[:, :, k:k + x.shape[2]] for k in range(3)], -1)          # [B, C, L, 3]
        y = np.einsum("bclk,ock->bol", cols, wt) + b[None, :, None]
        return y[:, :, ::stride]

    def gelu(x):
        from math import sqrt
        erf = np.vectorize(math.erf)
        return 0.5 * x * (1.0 + erf(x / sqrt(2.0)))

    if cfg.audio_features:
        x = gelu(conv1d(gelu(conv1d(enc_ids.astype(np.float64), "enc.conv1", 1)), "enc.conv2", 2)).transpose(0, 2, 1)
        enc_bias = 0.0
        x = x + f["enc.pos"][np.arange(x.shape[1])]
    else:
        enc_bias = np.where(enc_mask[:, None, None, :] != 0, 0.0, -10000.0)
        x = f["embed"][enc_ids] + f["enc.pos"][np.arange(enc_ids.shape[1])]
    for i in range(cfg.encoder_layers):
        p = f"enc.{i}"
        h = ln(x, p + ".ln1")
        x = x + attend(h, h, enc_bias, p + ".self")
        x = x + ffn(ln(x, p + ".ln2"), p)
    enc = ln(x, "enc.ln_f")
    Sd = dec_ids.shape[1]
    causal = np.where(np.tril(np.ones((Sd, Sd), bool)), 0.0, -10000.0)[None, None]
    x = f["embed"][dec_ids] + f["dec.pos"][np.arange(Sd)]
    for i in range(cfg.decoder_layers):
        p = f"dec.{i}"
        h = ln(x, p + ".ln1")
        x = x + attend(h, h, causal, p + ".self")
        x = x + attend(ln(x, p + ".ln2"), enc, enc_bias, p + ".cross")
        x = x + ffn(ln(x, p + ".ln3"), p)
    return ln(x, "dec.ln_f") @ f["embed"].T
