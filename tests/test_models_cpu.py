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


def _tiny_runner(batch, with_argmax=False):
    cfg = LlamaConfig.tiny(dtype="fp32", vocab_size=64, num_layers=1)
    model, _ = build_llama(cfg, weight_std=0.3, with_argmax=with_argmax)
    sess = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    return cfg, sess, DecoderRunner(sess, cfg, batch, 64)


def test_generate_greedy_sampling_and_processors():
    from onnxruntime_b200.models.generation import GenerationConfig, generate, process_logits, top_k_top_p_filter
    cfg, sess, runner = _tiny_runner(2)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (2, 6))
    greedy = generate(runner, ids, GenerationConfig(max_new_tokens=6))
    ref = DecoderRunner(sess, cfg, 2, 64).generate(ids, 6)
    assert torch.equal(greedy[:, 6:], ref)
    # sampling is reproducible under a seed and stays inside the top-k set
    a = generate(DecoderRunner(sess, cfg, 2, 64), ids, GenerationConfig(max_new_tokens=5, top_k=3, seed=7))
    b = generate(DecoderRunner(sess, cfg, 2, 64), ids, GenerationConfig(max_new_tokens=5, top_k=3, seed=7))
    assert torch.equal(a, b)
    # processors
    logits = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    seq = torch.tensor([[3, 1, 3]])
    out = process_logits(logits, seq, 0, GenerationConfig(repetition_penalty=2.0))
    assert out.tolist() == [[1.0, 1.0, 3.0, 2.0]]
    out = process_logits(logits, seq, 0, GenerationConfig(no_repeat_ngram_size=2))   # (3, 1) seen: 1 after 3 is banned
    assert out[0, 1] == float("-inf") and torch.isfinite(out[0, [0, 2, 3]]).all()
    out = process_logits(logits, seq, 0, GenerationConfig(eos_token_id=2, min_new_tokens=1))
    assert out[0, 2] == float("-inf")
    f = top_k_top_p_filter(torch.tensor([[0.0, 1.0, 2.0, 3.0]]), top_k=2, top_p=1.0)
    assert torch.isinf(f[0, :2]).all() and torch.isfinite(f[0, 2:]).all()
    f = top_k_top_p_filter(torch.log(torch.tensor([[0.1, 0.2, 0.3, 0.4]])), top_k=0, top_p=0.5)
    assert torch.isinf(f[0, :2]).all() and torch.isfinite(f[0, 2:]).all()


def test_beam_search_finds_a_sequence_at_least_as_likely_as_greedy():
    from onnxruntime_b200.models.generation import GenerationConfig, generate
    cfg, sess, _ = _tiny_runner(1)
    torch.manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (2, 5))
    steps, K = 5, 3
    beams = generate(DecoderRunner(sess, cfg, 2 * K, 64), ids, GenerationConfig(max_new_tokens=steps, num_beams=K, length_penalty=0.0))
    greedy = generate(DecoderRunner(sess, cfg, 2, 64), ids, GenerationConfig(max_new_tokens=steps))
    assert beams.shape == greedy.shape and torch.equal(beams[:, :5], ids)

    def logprob(seq):   # score a full sequence with a fresh pass
        r = DecoderRunner(sess, cfg, 2, 64)
        r.prefill(seq[:, :5])
        total = torch.zeros(2)
        logits = r.prefill_logits.reshape(2, -1).float()
        for t in range(steps):
            lp = torch.log_softmax(logits, -1)
            total += lp.gather(1, seq[:, 5 + t].view(-1, 1)).squeeze(1)
            if t + 1 < steps:
                r.decode_step(seq[:, 5 + t].view(-1, 1))
                logits = r.step_logits.reshape(2, -1).float()
        return total
    assert (logprob(beams) >= logprob(greedy) - 1e-4).all()


def test_fp8_bert_graph_tracks_the_fp16_graph():
    """build_bert_fp8 (GemmFloat8 dense layers, packed MultiHeadAttention, SkipLayerNormalization) against the exporter-style
    fp16 graph on the same weights: fp8 rounding only."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.bert import BertConfig, build_bert, build_bert_fp8, init_weights
    cfg = BertConfig(vocab_size=100, hidden_size=64, num_layers=2, num_heads=2, ffn_size=128, max_position=32, dtype="fp16")
    w = init_weights(cfg)
    for k in w:
        if k.endswith("weight"):
            w[k] = (w[k].astype(np.float32) * 5).astype(np.float16)
    ids = np.random.RandomState(0).randint(0, 100, (2, 16))
    mask = np.ones((2, 16), np.int64)
    mask[1, 10:] = 0
    feeds = {"input_ids": ids, "attention_mask": mask}
    a = ort.InferenceSession(build_bert(cfg, w), providers=["CPUExecutionProvider"]).run(None, feeds)[0].astype(np.float32)
    sess = ort.InferenceSession(build_bert_fp8(cfg, w), providers=["CPUExecutionProvider"])
    b = sess.run(None, feeds)[0].astype(np.float32)
    valid = mask.astype(bool)
    assert np.abs(a - b)[valid].max() < 0.3 and np.abs(a - b)[valid].mean() < 0.05
    from helpers import op_counts
    assert op_counts(sess)["GemmFloat8"] == 8
