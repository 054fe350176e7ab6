"""Llama-family decoder as an ONNX graph (random-init exporter).

Produces the graph shape the reference's LLM tooling produces after its fusion
passes (onnxruntime/python/tools/transformers/models/llama/convert_to_onnx.py:
``GroupQueryAttention`` with packed QKV and in-op rotary embedding,
``SkipSimplifiedLayerNormalization`` carrying the residual stream, one
``past_key_values.{i}.key/value`` -> ``present.{i}.key/value`` pair per layer
bound to the same buffer) and, for tensor parallelism, one graph per rank with
heads / FFN columns divided by the world size and ``com.microsoft.AllReduce``
after the two row-parallel projections (the ``rank_{r}_*.onnx`` convention of
that exporter).

Weights are either embedded (tests) or declared as session-supplied external
initializers and returned separately as torch tensors (large models).
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import onnx_lite as ol

T = ol.TensorProto


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rope_theta: float = 500000.0
    max_seq_len: int = 2048
    rms_eps: float = 1e-5
    dtype: str = "bf16"  # bf16 | fp16 | fp32

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def llama3_70b(**kw) -> "LlamaConfig":
        base = dict(hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8, ffn_size=28672)
        base.update(kw)
        return LlamaConfig(**base)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                    ffn_size=512, max_seq_len=128)
        base.update(kw)
        return LlamaConfig(**base)


_TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
_ONNX_DT = {"bf16": T.BFLOAT16, "fp16": T.FLOAT16, "fp32": T.FLOAT}


def rope_caches(cfg: LlamaConfig, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    half = cfg.head_dim // 2
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float64, device=device) / half))
    t = torch.arange(cfg.max_seq_len, dtype=torch.float64, device=device)
    freqs = torch.outer(t, inv_freq)
    dt = _TORCH_DT[cfg.dtype]
    return freqs.cos().to(dt), freqs.sin().to(dt)


def build_llama(cfg: LlamaConfig, tp_rank: int = 0, tp_size: int = 1, external_weights: bool = False, seed: int = 0,
                device: str = "cpu", with_argmax: bool = True, last_token_logits: bool = True,
                weight_std: float = 0.02, shard_lm_head: bool = True, quant_bits: int = 0,
                quant_block: int = 32, paged: bool = False, moe_experts: int = 0, moe_top_k: int = 2, ep_rank: int = 0,
                ep_size: int = 1) -> Tuple[bytes, Dict[str, torch.Tensor]]:
    """Returns (ModelProto bytes, weights).  With ``external_weights`` the dict holds every weight (on
    ``device``) to pass to ``SessionOptions.add_external_initializers``; otherwise it is empty and the
    weights are embedded in the model.

    ``quant_bits=4`` emits the seven projections of every layer as ``com.microsoft.MatMulNBits`` (symmetric
    blocks of ``quant_block`` weights along K, packed two per byte, one scale per block: the layout of
    onnxruntime/contrib_ops/cpu/quantization/matmul_nbits.cc) the way the reference's 4-bit exporters do;
    the embedding and the LM head stay in the compute type.

    ``paged=True`` builds the serving form: tokens of all sequences packed along one axis (``input_ids``
    [tokens]), ``com.microsoft.PagedAttention`` over block caches ``key_cache.{i}`` / ``value_cache.{i}``
    [num_blocks, block_size, kv_heads, head_dim] shared by all sequences through ``block_table``, with
    ``cumulative_sequence_length`` and ``past_seqlens`` describing the packing (input order of
    onnxruntime/core/graph/contrib_ops/bert_defs.cc, PagedAttention); ``logits_indices`` [rows] picks the
    packed positions whose logits are wanted (the last token of every sequence), so the LM head runs on those
    rows only.

    ``moe_experts > 0`` replaces the dense SwiGLU block of every layer by a top-``moe_top_k`` softmax-routed mixture of
    that many SwiGLU experts (the Mixtral shape): ``com.microsoft.MoE`` on one device, or ``com.microsoft.ShardedMoE``
    holding experts ``[ep_rank * E / ep_size, (ep_rank + 1) * E / ep_size)`` when ``ep_size > 1`` (expert parallelism:
    attention and router weights are replicated, every rank sees all tokens, as the operator's contract has it,
    onnxruntime/contrib_ops/cuda/collective/sharded_moe.cc:54-189)."""
    assert not (moe_experts and (tp_size > 1 or quant_bits)), "the mixture-of-experts form is dense and expert-parallel only"
    assert moe_experts % max(ep_size, 1) == 0
    if paged:
        last_token_logits = False
    assert quant_bits in (0, 4)
    assert cfg.num_heads % tp_size == 0 and cfg.num_kv_heads % tp_size == 0 and cfg.ffn_size % tp_size == 0
    dt, odt = _TORCH_DT[cfg.dtype], _ONNX_DT[cfg.dtype]
    N, Nk, H = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.head_dim
    hidden, ffn = cfg.hidden_size, cfg.ffn_size // tp_size
    gen = torch.Generator(device=device)
    weights: Dict[str, torch.Tensor] = {}
    inits: List[ol.Tensor] = []
    nodes: List[ol.Node] = []

    def randn(name: str, shape, std: float = weight_std, shard: Optional[Tuple[int, int]] = None) -> str:
        """Full-size tensor from a per-name seed, then the rank's shard (so ranks agree on the full model)."""
        gen.manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
        full = tuple(shape)
        if shard is not None:
            axis, parts = shard
            full = list(shape)
            full[axis] *= parts
        w = (torch.randn(full, generator=gen, device=device, dtype=torch.float32) * std).to(dt)
        if shard is not None:
            axis, parts = shard
            w = w.chunk(parts, dim=axis)[tp_rank].contiguous()
        add_weight(name, w)
        return name

    def add_weight(name: str, w: torch.Tensor) -> None:
        if external_weights:
            weights[name] = w
            onnx_type = odt if w.dtype == dt else (T.UINT8 if w.dtype == torch.uint8 else T.FLOAT)
            inits.append(ol.make_external_tensor(name, onnx_type, w.shape))
        else:
            inits.append(ol.make_tensor(name, w))

    def linear(x: str, weight: str, k: int, n: int, out: str, node_name: str, shard: Optional[Tuple[int, int]] = None,
               dense: Optional[torch.Tensor] = None, full_n: Optional[int] = None,
               columns: Optional[torch.Tensor] = None) -> None:
        """out = x @ W with W [k, n] (this rank's shard; ``shard`` = (axis, parts) of the full matrix, or the
        already sharded ``dense`` matrix, which is columns ``columns`` of a ``full_n`` wide one), as MatMul or as
        MatMulNBits over randomly drawn 4-bit blocks."""
        if not quant_bits:
            if dense is not None:
                add_weight(weight, dense)
            else:
                randn(weight, (k, n), shard=shard)
            nodes.append(ol.make_node("MatMul", [x, weight], [out], name=node_name))
            return
        assert k % quant_block == 0
        gen.manual_seed(seed * 1000003 + zlib.crc32(weight.encode()))
        full_n, full_k = full_n or n, k
        if shard is not None:
            full_k, full_n = (k * shard[1], n) if shard[0] == 0 else (k, n * shard[1])
        # packed [N, K/block, block/2] bytes and [N, K/block] scales; scale so that a dequantised weight has
        # about the standard deviation of the dense initialisation (a uniform nibble minus 8 has sigma 4.6)
        packed = torch.randint(0, 256, (full_n, full_k // quant_block, quant_block // 2), generator=gen, device=device,
                               dtype=torch.uint8)
        scales = ((torch.rand((full_n, full_k // quant_block), generator=gen, device=device) * 0.5 + 0.75)
                  * (weight_std / 4.6)).to(dt)
        if shard is not None:
            axis = 1 if shard[0] == 0 else 0          # K shards are block ranges, N shards are row ranges
            packed = packed.chunk(shard[1], dim=axis)[tp_rank].contiguous()
            scales = scales.chunk(shard[1], dim=axis)[tp_rank].contiguous()
        if columns is not None:
            packed, scales = packed[columns].contiguous(), scales[columns].contiguous()
        add_weight(weight + ".q4", packed)
        add_weight(weight + ".scales", scales)
        nodes.append(ol.make_node("MatMulNBits", [x, weight + ".q4", weight + ".scales"], [out], name=node_name,
                                  domain="com.microsoft", K=k, N=n, bits=quant_bits, block_size=quant_block))

    def ones(name: str, n: int) -> str:
        add_weight(name, torch.ones(n, dtype=dt, device=device))
        return name

    cos, sin = rope_caches(cfg, device)
    add_weight("cos_cache", cos)
    add_weight("sin_cache", sin)

    randn("model.embed_tokens.weight", (cfg.vocab_size, hidden))
    nodes.append(ol.make_node("Gather", ["model.embed_tokens.weight", "input_ids"], ["hidden_0"], name="embed", axis=0))

    residual = "hidden_0"   # running residual stream
    pending = None          # output of the previous block still to be added to the residual
    if paged:
        inputs = [
            ol.make_tensor_value_info("input_ids", T.INT64, ["tokens"]),
            ol.make_tensor_value_info("cumulative_sequence_length", T.INT32, ["batch_plus_1"]),
            ol.make_tensor_value_info("past_seqlens", T.INT32, ["batch"]),
            ol.make_tensor_value_info("block_table", T.INT32, ["batch", "max_blocks"]),
            ol.make_tensor_value_info("logits_indices", T.INT64, ["rows"]),
        ]
    else:
        inputs = [
            ol.make_tensor_value_info("input_ids", T.INT64, ["batch", "seq"]),
            ol.make_tensor_value_info("seqlens_k", T.INT32, ["batch"]),
            ol.make_tensor_value_info("total_sequence_length", T.INT32, []),
        ]
    outputs = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}"
        ln1 = ones(f"{p}.input_layernorm.weight", hidden)
        if pending is None:
            nodes.append(ol.make_node("SimplifiedLayerNormalization", [residual, ln1], [f"{p}.ln1_out"], name=f"{p}.ln1",
                                      axis=-1, epsilon=cfg.rms_eps))
        else:
            nodes.append(ol.make_node("SkipSimplifiedLayerNormalization", [pending, residual, ln1],
                                      [f"{p}.ln1_out", "", "", f"{p}.res1"], name=f"{p}.ln1", domain="com.microsoft",
                                      epsilon=cfg.rms_eps))
            residual = f"{p}.res1"
        # packed QKV projection: column-parallel, columns ordered [q heads | k heads | v heads] of this rank
        gen.manual_seed(seed * 1000003 + zlib.crc32(f"{p}.qkv".encode()))
        full = (torch.randn((hidden, (cfg.num_heads + 2 * cfg.num_kv_heads) * H), generator=gen, device=device,
                            dtype=torch.float32) * weight_std).to(dt)
        q_full, k_full, v_full = full.split([cfg.num_heads * H, cfg.num_kv_heads * H, cfg.num_kv_heads * H], dim=1)
        wqkv = torch.cat([q_full.chunk(tp_size, 1)[tp_rank], k_full.chunk(tp_size, 1)[tp_rank],
                          v_full.chunk(tp_size, 1)[tp_rank]], dim=1).contiguous()
        del full, q_full, k_full, v_full
        nq, nkv = cfg.num_heads * H, cfg.num_kv_heads * H
        cols = torch.cat([torch.arange(nq, device=device).chunk(tp_size)[tp_rank],
                          nq + torch.arange(nkv, device=device).chunk(tp_size)[tp_rank],
                          nq + nkv + torch.arange(nkv, device=device).chunk(tp_size)[tp_rank]])
        linear(f"{p}.ln1_out", f"{p}.attn.qkv_proj.weight", hidden, wqkv.shape[1], f"{p}.qkv", f"{p}.qkv_proj", dense=wqkv,
               full_n=nq + 2 * nkv, columns=cols)
        if paged:
            for kv in ("key", "value"):
                inputs.append(ol.make_tensor_value_info(f"{kv}_cache.{i}", odt, ["num_blocks", "block_size", Nk, H]))
                outputs.append(ol.make_tensor_value_info(f"{kv}_cache_out.{i}", odt, ["num_blocks", "block_size", Nk, H]))
            nodes.append(ol.make_node(
                "PagedAttention",
                [f"{p}.qkv", "", "", f"key_cache.{i}", f"value_cache.{i}", "cumulative_sequence_length", "past_seqlens",
                 "block_table", "cos_cache", "sin_cache"],
                [f"{p}.attn_out", f"key_cache_out.{i}", f"value_cache_out.{i}"], name=f"{p}.attn", domain="com.microsoft",
                num_heads=N, kv_num_heads=Nk, do_rotary=1, rotary_interleaved=0))
        else:
            inputs.append(ol.make_tensor_value_info(f"past_key_values.{i}.key", odt, ["batch", Nk, "past_seq", H]))
            inputs.append(ol.make_tensor_value_info(f"past_key_values.{i}.value", odt, ["batch", Nk, "past_seq", H]))
            outputs.append(ol.make_tensor_value_info(f"present.{i}.key", odt, ["batch", Nk, "present_seq", H]))
            outputs.append(ol.make_tensor_value_info(f"present.{i}.value", odt, ["batch", Nk, "present_seq", H]))
            nodes.append(ol.make_node(
                "GroupQueryAttention",
                [f"{p}.qkv", "", "", f"past_key_values.{i}.key", f"past_key_values.{i}.value", "seqlens_k",
                 "total_sequence_length", "cos_cache", "sin_cache"],
                [f"{p}.attn_out", f"present.{i}.key", f"present.{i}.value"], name=f"{p}.attn", domain="com.microsoft",
                num_heads=N, kv_num_heads=Nk, do_rotary=1, rotary_interleaved=0))
        linear(f"{p}.attn_out", f"{p}.attn.o_proj.weight", N * H, hidden, f"{p}.o_partial" if tp_size > 1 else f"{p}.o",
               f"{p}.o_proj", shard=(0, tp_size))
        if tp_size > 1:
            nodes.append(ol.make_node("AllReduce", [f"{p}.o_partial"], [f"{p}.o"], name=f"{p}.o_allreduce", domain="com.microsoft"))
        ln2 = ones(f"{p}.post_attention_layernorm.weight", hidden)
        nodes.append(ol.make_node("SkipSimplifiedLayerNormalization", [f"{p}.o", residual, ln2],
                                  [f"{p}.ln2_out", "", "", f"{p}.res2"], name=f"{p}.ln2", domain="com.microsoft",
                                  epsilon=cfg.rms_eps))
        residual = f"{p}.res2"
        if moe_experts:
            el = moe_experts // ep_size
            randn(f"{p}.moe.router.weight", (hidden, moe_experts))
            nodes.append(ol.make_node("MatMul", [f"{p}.ln2_out", f"{p}.moe.router.weight"], [f"{p}.router_logits"], name=f"{p}.router"))
            names = []
            for nm, shape in (("fc1", (ffn, hidden)), ("fc2", (hidden, ffn)), ("fc3", (ffn, hidden))):
                per_expert = []
                for e in range(ep_rank * el, (ep_rank + 1) * el):
                    gen.manual_seed(seed * 1000003 + zlib.crc32(f"{p}.moe.{nm}.{e}".encode()))
                    w = (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * weight_std).to(dt)
                    # MoE stores [out, in] per expert, ShardedMoE the older [in, out]
                    per_expert.append(w if ep_size == 1 else w.t().contiguous())
                add_weight(f"{p}.moe.{nm}", torch.stack(per_expert))
                names.append(f"{p}.moe.{nm}")
            attrs = dict(k=moe_top_k, activation_type="silu", normalize_routing_weights=1)
            if ep_size > 1:
                attrs["local_experts_start_index"] = ep_rank * el
            nodes.append(ol.make_node("MoE" if ep_size == 1 else "ShardedMoE", [f"{p}.ln2_out", f"{p}.router_logits", names[0], "", names[1], "", names[2]],
                                      [f"{p}.down"], name=f"{p}.moe", domain="com.microsoft", **attrs))
        else:
            linear(f"{p}.ln2_out", f"{p}.mlp.gate_proj.weight", hidden, ffn, f"{p}.gate", f"{p}.gate_proj", shard=(1, tp_size))
            linear(f"{p}.ln2_out", f"{p}.mlp.up_proj.weight", hidden, ffn, f"{p}.up", f"{p}.up_proj", shard=(1, tp_size))
            nodes += [
                ol.make_node("Sigmoid", [f"{p}.gate"], [f"{p}.gate_sig"], name=f"{p}.sigmoid"),
                ol.make_node("Mul", [f"{p}.gate", f"{p}.gate_sig"], [f"{p}.gate_act"], name=f"{p}.silu"),
                ol.make_node("Mul", [f"{p}.gate_act", f"{p}.up"], [f"{p}.mlp_h"], name=f"{p}.gate_mul"),
            ]
            linear(f"{p}.mlp_h", f"{p}.mlp.down_proj.weight", ffn, hidden, f"{p}.down_partial" if tp_size > 1 else f"{p}.down",
                   f"{p}.down_proj", shard=(0, tp_size))
            if tp_size > 1:
                nodes.append(ol.make_node("AllReduce", [f"{p}.down_partial"], [f"{p}.down"], name=f"{p}.down_allreduce",
                                          domain="com.microsoft"))
        pending = f"{p}.down"

    lnf = ones("model.norm.weight", hidden)
    nodes.append(ol.make_node("SkipSimplifiedLayerNormalization", [pending, residual, lnf], ["final_norm"],
                              name="final_norm", domain="com.microsoft", epsilon=cfg.rms_eps))
    head_in = "final_norm"
    if last_token_logits:
        inits.append(ol.make_tensor("last_index", np.array([-1], dtype=np.int64)))
        nodes.append(ol.make_node("Gather", ["final_norm", "last_index"], ["final_last"], name="last_token", axis=1))
        head_in = "final_last"
    if paged:
        nodes.append(ol.make_node("Gather", ["final_norm", "logits_indices"], ["final_rows"], name="logit_rows", axis=0))
        head_in = "final_rows"
    if tp_size > 1 and shard_lm_head and cfg.vocab_size % tp_size == 0:
        # vocabulary-parallel head: every rank computes its slice of the logits, an all-gather along the last axis
        # puts them together (the full-vocabulary product would otherwise be repeated on every rank)
        randn("lm_head.weight", (hidden, cfg.vocab_size // tp_size), shard=(1, tp_size))
        nodes.append(ol.make_node("MatMul", [head_in, "lm_head.weight"], ["logits_shard"], name="lm_head"))
        nodes.append(ol.make_node("AllGather", ["logits_shard"], ["logits"], name="lm_head_allgather", domain="com.microsoft",
                                  axis=1 if paged else 2, group_size=tp_size))
    else:
        randn("lm_head.weight", (hidden, cfg.vocab_size))
        nodes.append(ol.make_node("MatMul", [head_in, "lm_head.weight"], ["logits"], name="lm_head"))
    logits_shape = ["rows"] if paged else ["batch", 1 if last_token_logits else "seq"]
    outputs.insert(0, ol.make_tensor_value_info("logits", odt, logits_shape + [cfg.vocab_size]))
    if with_argmax:
        nodes.append(ol.make_node("ArgMax", ["logits"], ["next_tokens"], name="greedy", axis=-1, keepdims=0))
        outputs.insert(1, ol.make_tensor_value_info("next_tokens", T.INT64, logits_shape))
    graph = ol.make_graph(nodes, "llama", inputs, outputs, inits)
    meta = {"tp_rank": str(tp_rank), "tp_size": str(tp_size), "architecture": "mixtral" if moe_experts else "llama"}
    model = ol.make_model(graph, opset=17, metadata=meta)
    return model.serialize(), weights


def empty_paged_cache(cfg: LlamaConfig, num_blocks: int, block_size: int, device,
                      tp_size: int = 1) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """Per layer (key_cache, value_cache) of shape [num_blocks, block_size, kv_heads / tp, head_dim]."""
    dt = _TORCH_DT[cfg.dtype]
    nk = cfg.num_kv_heads // tp_size
    return [(torch.zeros(num_blocks, block_size, nk, cfg.head_dim, dtype=dt, device=device),
             torch.zeros(num_blocks, block_size, nk, cfg.head_dim, dtype=dt, device=device)) for _ in range(cfg.num_layers)]


def empty_kv_cache(cfg: LlamaConfig, batch: int, max_len: int, device, tp_size: int = 1) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    dt = _TORCH_DT[cfg.dtype]
    nk = cfg.num_kv_heads // tp_size
    return [(torch.zeros(batch, nk, max_len, cfg.head_dim, dtype=dt, device=device),
             torch.zeros(batch, nk, max_len, cfg.head_dim, dtype=dt, device=device)) for _ in range(cfg.num_layers)]
