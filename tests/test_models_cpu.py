"""Model builders and generation drivers on the CPU provider."""
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200.models.generation import DecoderRunner, PagedDecoderRunner
from onnxruntime_b200.models.llama import LlamaConfig, build_llama


@pytest.mark.parametrize("quant_bits", [0, 4])
def test_paged_decoder_matches_contiguous_cache(quant_bits):
    """The PagedAttention form of the decoder (packed tokens, shared block pool, scattered block table) must
    generate the same tokens as the GroupQueryAttention form with one contiguous cache per sequence."""
    cfg = LlamaConfig.tiny(dtype="fp32")
    dense, _ = build_llama(cfg, weight_std=0.05, quant_bits=quant_bits)
    paged, _ = build_llama(cfg, weight_std=0.05, quant_bits=quant_bits, paged=True)
    s1 = ort.InferenceSession(dense, providers=["CPUExecutionProvider"])
    s2 = ort.InferenceSession(paged, providers=["CPUExecutionProvider"])
    ops = {n["op_type"] for n in s2.graph_nodes()}
    assert "PagedAttention" in ops and ("MatMulNBits" in ops) == (quant_bits == 4)
    torch.manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (3, 21))
    a = DecoderRunner(s1, cfg, 3, 64).generate(ids, 8)
    b = PagedDecoderRunner(s2, cfg, 3, 64, block_size=8).generate(ids, 8)
    assert torch.equal(a, b)


def test_int4_model_dequantises_to_the_dense_model():
    """MatMulNBits projections with the exporter's packing equal MatMul on the expanded weights."""
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    cfg = LlamaConfig.tiny(dtype="fp32", num_layers=1)
    q, _ = build_llama(cfg, weight_std=0.05, quant_bits=4)
    m = ol.load_model(q)
    inits = {t.name: ol.to_array(t) for t in m.graph.initializers}
    node = next(n for n in m.graph.nodes if n.op_type == "MatMulNBits")
    packed, scales = inits[node.inputs[1]], inits[node.inputs[2]]
    n_, blocks, half = packed.shape
    lo, hi = (packed & 15).astype(np.float32) - 8, (packed >> 4).astype(np.float32) - 8
    w = np.stack([lo, hi], -1).reshape(n_, blocks, half * 2) * scales[..., None]
    w = w.reshape(n_, -1).T   # [K, N]
    x = np.random.default_rng(0).standard_normal((5, w.shape[0])).astype(np.float32)
    g = ol.make_graph([ol.make_node("MatMulNBits", ["x", "b", "s"], ["y"], domain="com.microsoft", K=w.shape[0], N=n_,
                                    bits=4, block_size=32)], "g",
                      [ol.make_tensor_value_info("x", ol.TensorProto.FLOAT, [5, w.shape[0]])],
                      [ol.make_tensor_value_info("y", ol.TensorProto.FLOAT, [5, n_])],
                      [ol.make_tensor("b", packed), ol.make_tensor("s", scales)])
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), providers=["CPUExecutionProvider"])
    (y,) = sess.run(None, {"x": x})
    np.testing.assert_allclose(y, x @ w, rtol=1e-4, atol=1e-4)
