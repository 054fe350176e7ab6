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


def test_gpt2_graph_prefill_and_decode_with_past_match_the_numpy_model():
    """GPT-2 builder (LayerNormalization + com.microsoft Attention with past / present + FastGelu): a prompt pass followed by
    token-by-token passes over the returned state gives the logits of one full pass of the numpy restatement."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models import gpt2
    cfg = gpt2.Gpt2Config(vocab_size=97, hidden_size=32, num_layers=2, num_heads=4, max_position=32)
    w = gpt2.init_weights(cfg, seed=3)
    sess = ort.InferenceSession(gpt2.build_gpt2(cfg, w), providers=["CPUExecutionProvider"])
    assert [o.name for o in sess.get_outputs()] == ["logits", "present_0", "present_1"]
    rng = np.random.RandomState(0)
    ids = rng.randint(0, cfg.vocab_size, (2, 9))
    ref = gpt2.reference_forward(cfg, w, ids)
    outs = sess.run(None, gpt2.step_feeds(cfg, ids[:, :6], gpt2.empty_past(cfg, 2)))
    np.testing.assert_allclose(outs[0], ref[:, :6], rtol=2e-4, atol=2e-5)
    past = {f"past_{i}": outs[1 + i] for i in range(cfg.num_layers)}
    assert past["past_0"].shape == (2, 2, 4, 6, 8)
    for t in range(6, 9):
        outs = sess.run(None, gpt2.step_feeds(cfg, ids[:, t:t + 1], past))
        np.testing.assert_allclose(outs[0][:, 0], ref[:, t], rtol=2e-4, atol=2e-5)
        past = {f"past_{i}": outs[1 + i] for i in range(cfg.num_layers)}
    assert past["past_1"].shape[3] == 9


def test_gpt2_under_the_greedy_search_operator(tmp_path):
    """The GPT-2 graph has the interface of the generation operators: wrapped into GreedySearch it decodes what a plain
    arg-max loop over the numpy model decodes."""
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.models import gpt2
    from onnxruntime_b200.transformers import convert_generation as cg
    cfg = gpt2.Gpt2Config(vocab_size=61, hidden_size=32, num_layers=2, num_heads=4, max_position=32)
    w = gpt2.init_weights(cfg, seed=5)
    for k in w:                      # larger weights: well separated logits
        if k.endswith("weight") or k in ("wte", "wpe"):
            w[k] = w[k] * 8
    model = cg.convert(ol.load_model(gpt2.build_gpt2(cfg, w)), op="greedy", eos_token_id=cfg.vocab_size + 5)
    sess = ort.InferenceSession(model.serialize(), providers=["CPUExecutionProvider"])
    prompt = np.array([[7, 3, 11], [2, 40, 9]], np.int32)
    (seqs,) = sess.run(None, {"input_ids": prompt, "max_length": np.array([10], np.int32), "min_length": np.array([0], np.int32),
                              "repetition_penalty": np.array([1.0], np.float32), "attention_mask": np.ones((2, 3), np.int32)})
    want = prompt.astype(np.int64)
    for _ in range(7):
        nxt = gpt2.reference_forward(cfg, w, want)[:, -1].argmax(-1)
        want = np.concatenate([want, nxt[:, None]], 1)
    np.testing.assert_array_equal(seqs, want.astype(np.int32))


def test_encoder_decoder_builder_under_greedy_and_beam_search():
    """T5-shaped encoder / decoder graph pair: the decoder step over the encoder pass's states reproduces the numpy
    model's logits, and the GreedySearch / BeamSearch (one beam) wrappers decode what an arg-max loop over it decodes."""
    import numpy as np
    from onnxruntime_b200.models import encoder_decoder as ed
    from onnxruntime_b200.transformers import convert_generation as cg
    cfg = ed.EncoderDecoderConfig(vocab_size=53)
    w = ed.init_weights(cfg, seed=1, scale=0.3)
    encoder, decoder = ed.build_encoder_decoder(cfg, w)
    rng = np.random.RandomState(2)
    enc_ids = rng.randint(1, cfg.vocab_size, (2, 7)).astype(np.int32)
    enc_mask = np.ones((2, 7), np.int32)
    enc_mask[1, 5:] = 0
    start = 1
    # graphs by hand: encoder pass, then two decoder steps
    es = ort.InferenceSession(encoder.serialize(), providers=["CPUExecutionProvider"])
    ds = ort.InferenceSession(decoder.serialize(), providers=["CPUExecutionProvider"])
    dec = np.full((2, 1), start, np.int32)
    eo = es.run(None, {"encoder_input_ids": enc_ids, "encoder_attention_mask": enc_mask, "decoder_input_ids": dec})
    names = [o.name for o in es.get_outputs()]
    ref = ed.reference_logits(cfg, w, enc_ids, enc_mask, dec)
    np.testing.assert_allclose(eo[0], ref, rtol=2e-4, atol=2e-5)
    state = dict(zip(names, eo))
    toks = dec
    for _ in range(2):
        nxt = ed.reference_logits(cfg, w, enc_ids, enc_mask, toks)[:, -1].argmax(-1).astype(np.int32)[:, None]
        feeds = {"input_ids": nxt, "encoder_attention_mask": enc_mask}
        for i in range(cfg.decoder_layers):
            feeds[f"past_key_self_{i}"], feeds[f"past_value_self_{i}"] = state[f"present_key_self_{i}"], state[f"present_value_self_{i}"]
            feeds[f"past_key_cross_{i}"], feeds[f"past_value_cross_{i}"] = state[f"present_key_cross_{i}"], state[f"present_value_cross_{i}"]
        do = ds.run(None, feeds)
        toks = np.concatenate([toks, nxt], 1)
        np.testing.assert_allclose(do[0][:, 0], ed.reference_logits(cfg, w, enc_ids, enc_mask, toks)[:, -1], rtol=2e-4, atol=2e-5)
        for n, v in zip([o.name for o in ds.get_outputs()][1:], do[1:]):
            state[n] = v
    # the generation operators
    want = np.full((2, 1), start, np.int64)
    for _ in range(6):
        want = np.concatenate([want, ed.reference_logits(cfg, w, enc_ids, enc_mask, want)[:, -1].argmax(-1)[:, None]], 1)
    common = {"input_ids": enc_ids, "max_length": np.array([7], np.int32), "min_length": np.array([0], np.int32),
              "repetition_penalty": np.array([1.0], np.float32), "attention_mask": enc_mask}
    greedy = cg.convert(decoder, op="greedy", encoder=encoder, model_type=1, eos_token_id=cfg.vocab_size + 3, decoder_start_token_id=start)
    (seqs,) = ort.InferenceSession(greedy.serialize(), providers=["CPUExecutionProvider"]).run(None, common)
    np.testing.assert_array_equal(seqs, want.astype(np.int32))
    beam = cg.convert(decoder, op="beam", encoder=encoder, model_type=1, eos_token_id=cfg.vocab_size + 3, decoder_start_token_id=start)
    seqs, _ = ort.InferenceSession(beam.serialize(), providers=["CPUExecutionProvider"]).run(
        None, dict(common, num_beams=np.array([1], np.int32), num_return_sequences=np.array([1], np.int32), length_penalty=np.array([1.0], np.float32)))
    np.testing.assert_array_equal(seqs[:, 0], want.astype(np.int32))


def test_whisper_shaped_builder_under_whisper_beam_search():
    """Audio front end (two Conv1d + GELU, stride 2) in front of the same encoder-decoder: the WhisperBeamSearch wrapper
    with one beam decodes what the arg-max loop over the numpy model decodes."""
    import numpy as np
    from onnxruntime_b200.models import encoder_decoder as ed
    from onnxruntime_b200.transformers import convert_generation as cg
    cfg = ed.EncoderDecoderConfig(vocab_size=41, audio_features=6, encoder_layers=1, decoder_layers=2)
    w = ed.init_weights(cfg, seed=4, scale=0.3)
    encoder, decoder = ed.build_encoder_decoder(cfg, w)
    rng = np.random.RandomState(5)
    feats = rng.randn(2, 6, 20).astype(np.float32)
    start = 2
    es = ort.InferenceSession(encoder.serialize(), providers=["CPUExecutionProvider"])
    dec = np.full((2, 1), start, np.int32)
    eo = es.run(None, {"encoder_input_features": feats, "decoder_input_ids": dec})
    assert eo[1].shape == (2, 10, cfg.hidden_size)
    np.testing.assert_allclose(eo[0], ed.reference_logits(cfg, w, feats, None, dec), rtol=5e-4, atol=5e-5)
    want = np.full((2, 1), start, np.int64)
    for _ in range(5):
        want = np.concatenate([want, ed.reference_logits(cfg, w, feats, None, want)[:, -1].argmax(-1)[:, None]], 1)
    model = cg.convert(decoder, op="whisper", encoder=encoder, eos_token_id=cfg.vocab_size + 3, decoder_start_token_id=start)
    seqs, _ = ort.InferenceSession(model.serialize(), providers=["CPUExecutionProvider"]).run(
        None, {"input_features": feats, "max_length": np.array([6], np.int32), "min_length": np.array([0], np.int32), "num_beams": np.array([1], np.int32),
               "num_return_sequences": np.array([1], np.int32), "length_penalty": np.array([1.0], np.float32), "repetition_penalty": np.array([1.0], np.float32)})
    np.testing.assert_array_equal(seqs[:, 0], want.astype(np.int32))


def test_diffusion_unet_stage_matches_torch():
    """ResNet block + spatial transformer in the fused diffusion operators (GroupNorm + SiLU, NhwcConv, MultiHeadAttention,
    BiasSplitGelu, BiasAdd) against a plain torch restatement."""
    import numpy as np
    from onnxruntime_b200.models import diffusion
    cfg = diffusion.UNetStageConfig()
    w = diffusion.init_weights(cfg, seed=2)
    sess = ort.InferenceSession(diffusion.build_unet_stage(cfg, w), providers=["CPUExecutionProvider"])
    rng = np.random.RandomState(1)
    sample = rng.randn(2, cfg.channels, 6, 5).astype(np.float32)
    temb = rng.randn(2, cfg.time_dim).astype(np.float32)
    text = rng.randn(2, 7, cfg.text_dim).astype(np.float32)
    (y,) = sess.run(None, {"sample": sample, "time_embedding": temb, "encoder_hidden_states": text})
    ref = diffusion.reference_forward(cfg, w, sample, temb, text)
    assert y.shape == sample.shape
    np.testing.assert_allclose(y, ref, rtol=2e-4, atol=2e-4)


def test_phi_style_decoder_with_partial_rotary_matches_the_numpy_model():
    """Parallel attention / MLP block, rotary embedding on part of every head inside GroupQueryAttention: prompt pass plus
    token-by-token passes over the returned caches against one full pass of the numpy restatement."""
    import numpy as np
    from onnxruntime_b200.models import phi
    cfg = phi.PhiConfig()
    w = phi.init_weights(cfg, seed=7)
    sess = ort.InferenceSession(phi.build_phi(cfg, w), providers=["CPUExecutionProvider"])
    rng = np.random.RandomState(3)
    ids = rng.randint(0, cfg.vocab_size, (2, 8))
    ref = phi.reference_forward(cfg, w, ids)
    names = [o.name for o in sess.get_outputs()]
    outs = sess.run(None, phi.step_feeds(cfg, ids[:, :5], phi.empty_past(cfg, 2)))
    np.testing.assert_allclose(outs[0], ref[:, :5], rtol=3e-4, atol=3e-5)
    for t in range(5, 8):
        past = {n.replace("present", "past_key_values"): v for n, v in zip(names[1:], outs[1:])}
        outs = sess.run(None, phi.step_feeds(cfg, ids[:, t:t + 1], past))
        np.testing.assert_allclose(outs[0][:, 0], ref[:, t], rtol=3e-4, atol=3e-5)


def test_longformer_style_encoder_matches_the_numpy_model():
    import numpy as np
    from onnxruntime_b200.models import longformer as lf
    cfg = lf.LongformerConfig()
    w = lf.init_weights(cfg, seed=9)
    sess = ort.InferenceSession(lf.build_longformer(cfg, w), providers=["CPUExecutionProvider"])
    rng = np.random.RandomState(4)
    ids = rng.randint(0, cfg.vocab_size, (2, 12))
    mask = np.zeros((2, 12), np.float32)
    mask[1, 10:] = -10000.0
    glob = np.zeros((2, 12), np.int32)
    glob[:, 0] = 1
    glob[0, 7] = 1
    (y,) = sess.run(None, {"input_ids": ids, "attention_mask": mask, "global_attention_mask": glob})
    np.testing.assert_allclose(y, lf.reference_forward(cfg, w, ids, mask, glob), rtol=3e-4, atol=3e-5)
