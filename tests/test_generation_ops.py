"""com.microsoft GreedySearch / Sampling / BeamSearch over a decoder body graph, against a numpy restatement that
recomputes the toy model from scratch at every step (so cache handling and beam re-ordering are really checked)."""
import numpy as np
import pytest

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol

T = ol.TensorProto
V, D, N, HD, MAXPOS = 23, 16, 2, 8, 64
rng = np.random.RandomState(7)
W = {"E": rng.randn(V, D).astype(np.float32), "P": (rng.randn(MAXPOS, D) * 0.3).astype(np.float32),
     "Wv": (rng.randn(D, D) * 0.4).astype(np.float32), "Wo": (rng.randn(D, V) * 0.8).astype(np.float32)}


def decoder_body():
    i = lambda name, v: ol.make_tensor(name, np.asarray(v, np.int64))
    inits = [ol.make_tensor(k, v) for k, v in W.items()] + [i("kv_shape", [0, 0, N, HD]), i("ax0", [0]), i("one", 1), i("axm1", [-1]), i("ax1", [1]),
                                                             i("ctx_shape", [0, 0, D])]
    n = ol.make_node
    nodes = [n("Gather", ["E", "input_ids"], ["emb"]), n("Gather", ["P", "position_ids"], ["pe"]), n("Add", ["emb", "pe"], ["h"]),
             n("MatMul", ["h", "Wv"], ["v"]), n("Reshape", ["v", "kv_shape"], ["v4"]), n("Transpose", ["v4"], ["vt"], perm=[0, 2, 1, 3]),
             n("Unsqueeze", ["vt", "ax0"], ["vu"]), n("Concat", ["vu", "vu"], ["kv"], axis=0), n("Concat", ["past_0", "kv"], ["present_0"], axis=3),
             n("Gather", ["present_0", "one"], ["vals"], axis=0), n("Transpose", ["vals"], ["vals_t"], perm=[0, 2, 1, 3]),
             n("Reshape", ["vals_t", "ctx_shape"], ["vals2"]), n("Cast", ["attention_mask"], ["mf"], to=T.FLOAT), n("Unsqueeze", ["mf", "axm1"], ["m3"]),
             n("Mul", ["vals2", "m3"], ["masked"]), n("ReduceSum", ["masked", "ax1"], ["num"], keepdims=1), n("ReduceSum", ["m3", "ax1"], ["den"], keepdims=1),
             n("Div", ["num", "den"], ["ctx"]), n("Add", ["h", "ctx"], ["hc"]), n("Tanh", ["hc"], ["act"]), n("MatMul", ["act", "Wo"], ["logits"])]
    ins = [ol.make_tensor_value_info("input_ids", T.INT32, ["r", "s"]), ol.make_tensor_value_info("position_ids", T.INT32, ["r", "s"]),
           ol.make_tensor_value_info("attention_mask", T.INT32, ["r", "t"]), ol.make_tensor_value_info("past_0", T.FLOAT, [2, "r", N, "p", HD])]
    outs = [ol.make_tensor_value_info("logits", T.FLOAT, ["r", "s", V]), ol.make_tensor_value_info("present_0", T.FLOAT, [2, "r", N, "t", HD])]
    return ol.make_graph(nodes, "decoder", ins, outs, inits)


def ref_logits(seq):
    """last-position logits of the toy model for one full sequence (no cache)."""
    seq = np.asarray(seq)
    h = W["E"][seq] + W["P"][np.arange(len(seq))]
    ctx = (h @ W["Wv"]).mean(0)
    return np.tanh(h[-1] + ctx) @ W["Wo"]


def session(op, inputs, outputs, **attrs):
    node = ol.make_node(op, inputs, outputs, domain="com.microsoft", decoder=decoder_body(), model_type=0, **attrs)
    gi = [ol.make_tensor_value_info("input_ids", T.INT32, ["b", "s"]), ol.make_tensor_value_info("max_length", T.INT32, [1])]
    extra = {"min_length": (T.INT32, [1]), "num_beams": (T.INT32, [1]), "num_return_sequences": (T.INT32, [1]), "length_penalty": (T.FLOAT, [1]),
             "repetition_penalty": (T.FLOAT, [1])}
    for name in inputs[2:]:
        if name:
            gi.append(ol.make_tensor_value_info(name, *extra[name]))
    g = ol.make_graph([node], "g", gi, [ol.make_tensor_value_info(o, 0, None) for o in outputs])
    so = ort.SessionOptions()
    return ort.InferenceSession(ol.make_model(g).serialize(), so, providers=["CPUExecutionProvider"])


def test_greedy_search_matches_recomputation_with_eos_and_penalty():
    eos, pad = 5, 0
    sess = session("GreedySearch", ["input_ids", "max_length", "min_length", "repetition_penalty"], ["sequences"], eos_token_id=eos, pad_token_id=pad)
    ids = np.array([[3, 9, 1, 4], [7, 7, 2, 11]], np.int32)
    got = sess.run(None, {"input_ids": ids, "max_length": np.array([12], np.int32), "min_length": np.array([6], np.int32),
                          "repetition_penalty": np.array([1.3], np.float32)})[0]
    assert got.shape == (2, 12) and got.dtype == np.int32
    for b in range(2):
        seq, finished = list(ids[b]), False
        while len(seq) < 12:
            if finished:
                seq.append(pad)
                continue
            lg = ref_logits(seq).astype(np.float64)
            if len(seq) < 6:
                lg[eos] = -np.inf
            for t in set(seq):
                lg[t] = lg[t] * 1.3 if lg[t] < 0 else lg[t] / 1.3
            tok = int(np.argmax(lg))
            seq.append(tok)
            finished = tok == eos
        np.testing.assert_array_equal(got[b], np.array(seq, np.int32))


def test_sampling_is_seeded_and_respects_top_p():
    sess = session("Sampling", ["input_ids", "max_length"], ["sequences"], eos_token_id=-1, pad_token_id=0, top_p=0.05, temperature=0.7, seed=11)
    ids = np.array([[3, 9, 1, 4]], np.int32)
    feeds = {"input_ids": ids, "max_length": np.array([10], np.int32)}
    a, b = sess.run(None, feeds)[0], sess.run(None, feeds)[0]
    np.testing.assert_array_equal(a, b)            # same seed, same draw
    # with a nucleus this small only the most likely token survives: sampling degenerates to greedy
    seq = list(ids[0])
    while len(seq) < 10:
        seq.append(int(np.argmax(ref_logits(seq))))
    np.testing.assert_array_equal(a[0], np.array(seq, np.int32))


def _ref_beam(ids, K, max_length, eos, length_penalty, nrs, logits_fn=None):
    ref_logits = logits_fn or globals()["ref_logits"]
    beams = [(0.0, list(ids))] + [(-1e9, list(ids))] * (K - 1)
    finished, S0 = [], len(ids)
    while len(beams[0][1]) < max_length:
        cands = []
        for bi, (sc, seq) in enumerate(beams):
            lg = ref_logits(seq).astype(np.float64)
            logp = lg - (np.log(np.exp(lg - lg.max()).sum()) + lg.max())
            cands += [(sc + lp, bi, t) for t, lp in enumerate(logp)]
        cands.sort(key=lambda c: -c[0])
        gen_len = len(beams[0][1]) + 1 - S0
        nxt = []
        for rank, (sc, bi, t) in enumerate(cands[: 2 * K]):
            if t == eos:
                if rank < K:
                    finished.append((sc / gen_len ** length_penalty, beams[bi][1] + [t]))
                continue
            nxt.append((sc, beams[bi][1] + [t]))
            if len(nxt) == K:
                break
        beams = nxt
        if len(finished) >= K:
            worst = sorted(f[0] for f in finished)[-K]
            if worst >= max(b[0] for b in beams) / gen_len ** length_penalty:
                break
    gen_len = max(len(beams[0][1]) - S0, 1)
    hyps = finished + [(sc / gen_len ** length_penalty, seq) for sc, seq in beams]
    hyps.sort(key=lambda h: -h[0])
    return hyps[:nrs]


def test_beam_search_matches_a_plain_python_beam_search():
    eos = 5
    sess = session("BeamSearch", ["input_ids", "max_length", "min_length", "num_beams", "num_return_sequences", "length_penalty"],
                   ["sequences", "sequences_scores"], eos_token_id=eos, pad_token_id=0)
    ids = np.array([[3, 9, 1], [12, 2, 8]], np.int32)
    out = sess.run(None, {"input_ids": ids, "max_length": np.array([9], np.int32), "min_length": np.array([0], np.int32),
                          "num_beams": np.array([3], np.int32), "num_return_sequences": np.array([2], np.int32),
                          "length_penalty": np.array([1.0], np.float32)})
    seqs, scores = out
    assert seqs.shape == (2, 2, 9)
    for b in range(2):
        want = _ref_beam(ids[b], 3, 9, eos, 1.0, 2)
        for j, (sc, seq) in enumerate(want):
            padded = np.array(seq + [0] * (9 - len(seq)), np.int32)
            np.testing.assert_array_equal(seqs[b, j], padded)
            assert abs(scores[b, j] - sc) < 1e-3 * max(1.0, abs(sc))


# ---------------------------------------------------------------------------------------------- encoder-decoder form
W2 = {"Ee": rng.randn(V, D).astype(np.float32), "Wenc": (rng.randn(D, D) * 0.4).astype(np.float32), "Ed": rng.randn(V, D).astype(np.float32),
      "Wv2": (rng.randn(D, D) * 0.4).astype(np.float32), "Wo2": (rng.randn(D, V) * 0.8).astype(np.float32)}


def _encdec_common(prefix_nodes, hidden, cross_v, mask, d_emb, self_v):
    """nodes computing logits = tanh(d_emb + mean(self_v over time) + masked mean(cross_v) + 0.1 mean(hidden)) @ Wo2"""
    n = ol.make_node
    return prefix_nodes + [
        n("ReduceMean", [self_v], ["self_ctx4"], axes=[2], keepdims=0), n("Cast", [mask], ["mf"], to=T.FLOAT), n("Unsqueeze", ["mf", "axm1"], ["m3"]),
        n("Squeeze", [cross_v, "ax1"], ["cv3"]), n("Mul", ["cv3", "m3"], ["cvm"]), n("ReduceSum", ["cvm", "ax1"], ["cnum"], keepdims=1),
        n("ReduceSum", ["m3", "ax1"], ["cden"], keepdims=1), n("Div", ["cnum", "cden"], ["cross_ctx"]),
        n("ReduceMean", [hidden], ["hmean"], axes=[1], keepdims=1), n("Mul", ["hmean", "tenth"], ["hterm"]),
        n("Add", [d_emb, "self_ctx4"], ["a1"]), n("Add", ["a1", "cross_ctx"], ["a2"]), n("Add", ["a2", "hterm"], ["a3"]), n("Tanh", ["a3"], ["act"]),
        n("MatMul", ["act", "Wo2"], ["logits"])]


def _encdec_inits():
    i = lambda name, v: ol.make_tensor(name, np.asarray(v, np.int64))
    return [ol.make_tensor(k, v) for k, v in W2.items()] + [i("ax1", [1]), i("axm1", [-1]), ol.make_tensor("tenth", np.array(0.1, np.float32))]


def encoder_body():
    n = ol.make_node
    nodes = [n("Gather", ["Ee", "encoder_input_ids"], ["ee"]), n("MatMul", ["ee", "Wenc"], ["encoder_hidden_states"]),
             n("Unsqueeze", ["encoder_hidden_states", "ax1"], ["present_key_cross_0"]), n("Identity", ["present_key_cross_0"], ["present_value_cross_0"]),
             n("Gather", ["Ed", "decoder_input_ids"], ["d_emb"]), n("MatMul", ["d_emb", "Wv2"], ["dv"]),
             n("Unsqueeze", ["dv", "ax1"], ["present_key_self_0"]), n("Identity", ["present_key_self_0"], ["present_value_self_0"])]
    nodes = _encdec_common(nodes, "encoder_hidden_states", "present_value_cross_0", "encoder_attention_mask", "d_emb", "present_value_self_0")
    ins = [ol.make_tensor_value_info("encoder_input_ids", T.INT32, ["b", "se"]), ol.make_tensor_value_info("encoder_attention_mask", T.INT32, ["b", "se"]),
           ol.make_tensor_value_info("decoder_input_ids", T.INT32, ["b", "p"])]
    outs = [ol.make_tensor_value_info(o, T.FLOAT, None) for o in ("logits", "encoder_hidden_states", "present_key_self_0", "present_value_self_0",
                                                                  "present_key_cross_0", "present_value_cross_0")]
    return ol.make_graph(nodes, "encoder", ins, outs, _encdec_inits())


def encdec_decoder_body():
    n = ol.make_node
    nodes = [n("Gather", ["Ed", "input_ids"], ["d_emb"]), n("MatMul", ["d_emb", "Wv2"], ["dv"]), n("Unsqueeze", ["dv", "ax1"], ["dv4"]),
             n("Concat", ["past_key_self_0", "dv4"], ["present_key_self_0"], axis=2), n("Concat", ["past_value_self_0", "dv4"], ["present_value_self_0"], axis=2)]
    nodes = _encdec_common(nodes, "encoder_hidden_states", "past_value_cross_0", "encoder_attention_mask", "d_emb", "present_value_self_0")
    ins = [ol.make_tensor_value_info("input_ids", T.INT32, ["r", 1]), ol.make_tensor_value_info("encoder_attention_mask", T.INT32, ["r", "se"]),
           ol.make_tensor_value_info("encoder_hidden_states", T.FLOAT, ["r", "se", D])]
    ins += [ol.make_tensor_value_info(k, T.FLOAT, ["r", 1, "t", D]) for k in ("past_key_self_0", "past_value_self_0", "past_key_cross_0", "past_value_cross_0")]
    outs = [ol.make_tensor_value_info(o, T.FLOAT, None) for o in ("logits", "present_key_self_0", "present_value_self_0")]
    return ol.make_graph(nodes, "decoder", ins, outs, _encdec_inits())


def _encdec_logits_fn(enc_ids, enc_mask):
    hidden = W2["Ee"][np.asarray(enc_ids)] @ W2["Wenc"]
    m = np.asarray(enc_mask, np.float32)[:, None]
    cross = (hidden * m).sum(0) / m.sum()

    def fn(seq):
        seq = np.asarray(seq)
        return np.tanh(W2["Ed"][seq[-1]] + (W2["Ed"][seq] @ W2["Wv2"]).mean(0) + cross + 0.1 * hidden.mean(0)) @ W2["Wo2"]
    return fn


@pytest.mark.parametrize("op", ["BeamSearch", "GreedySearch"])
def test_encoder_decoder_generation_matches_recomputation(op):
    eos, start, K, max_len = 5, 2, 3, 9
    beam = op == "BeamSearch"
    inputs = (["input_ids", "max_length", "min_length", "num_beams", "num_return_sequences", "length_penalty", "repetition_penalty", "", "", "attention_mask"]
              if beam else ["input_ids", "max_length", "min_length", "repetition_penalty", "", "", "attention_mask"])
    outputs = ["sequences", "sequences_scores"] if beam else ["sequences"]
    node = ol.make_node(op, inputs, outputs, domain="com.microsoft", encoder=encoder_body(), decoder=encdec_decoder_body(), model_type=1,
                        eos_token_id=eos, pad_token_id=0, decoder_start_token_id=start)
    types = {"input_ids": (T.INT32, ["b", "s"]), "max_length": (T.INT32, [1]), "min_length": (T.INT32, [1]), "num_beams": (T.INT32, [1]),
             "num_return_sequences": (T.INT32, [1]), "length_penalty": (T.FLOAT, [1]), "repetition_penalty": (T.FLOAT, [1]), "attention_mask": (T.INT32, ["b", "s"])}
    g = ol.make_graph([node], "g", [ol.make_tensor_value_info(k, *types[k]) for k in inputs if k], [ol.make_tensor_value_info(o, 0, None) for o in outputs])
    sess = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    enc = np.array([[3, 9, 1, 4, 0], [7, 7, 2, 11, 13]], np.int32)
    mask = np.array([[1, 1, 1, 1, 0], [1, 1, 1, 1, 1]], np.int32)
    feeds = {"input_ids": enc, "max_length": np.array([max_len], np.int32), "min_length": np.array([2], np.int32),
             "repetition_penalty": np.array([1.0], np.float32), "attention_mask": mask}
    if beam:
        feeds.update({"num_beams": np.array([K], np.int32), "num_return_sequences": np.array([2], np.int32), "length_penalty": np.array([0.8], np.float32)})
    res = sess.run(None, feeds)
    for b in range(2):
        fn = _encdec_logits_fn(enc[b], mask[b])
        if beam:
            def fn_min(seq, fn=fn):           # min_length = 2 decoder tokens: no end of sequence as the second token
                lg = fn(seq).astype(np.float64)
                if len(seq) < 2:
                    lg[eos] = -np.inf
                return lg
            hyps = _ref_beam([start], K, max_len, eos, 0.8, 2, logits_fn=fn_min)
            for j, (score, seq) in enumerate(hyps):
                np.testing.assert_array_equal(res[0][b, j, :len(seq)], np.array(seq, np.int32))
                assert np.all(res[0][b, j, len(seq):] == 0) and abs(res[1][b, j] - score) < 1e-3
        else:
            seq, finished = [start], False
            while len(seq) < max_len:
                if finished:
                    seq.append(0)
                    continue
                lg = fn(seq).astype(np.float64)
                if len(seq) < 2:
                    lg[eos] = -np.inf
                seq.append(int(np.argmax(lg)))
                finished = seq[-1] == eos
            np.testing.assert_array_equal(res[0][b], np.array(seq, np.int32))


def test_whisper_beam_search_with_forced_decoder_prompt():
    """WhisperBeamSearch (model_type 2): float features into the encoder, no encoder attention mask anywhere, and a forced
    decoder prompt (input 10) of two tokens per batch entry."""
    eos, K, max_len = 5, 2, 8
    n = ol.make_node
    ones_mask = lambda hidden: [n("ReduceSum", [hidden, "axm1"], ["hs"], keepdims=0), n("Mul", ["hs", "zerof"], ["hz"]), n("Add", ["hz", "onef"], ["mask_f"])]
    extra = [ol.make_tensor("zerof", np.array(0.0, np.float32)), ol.make_tensor("onef", np.array(1.0, np.float32))]
    enc_nodes = [n("MatMul", ["encoder_input_ids", "Wenc"], ["encoder_hidden_states"]),
                 n("Unsqueeze", ["encoder_hidden_states", "ax1"], ["present_key_cross_0"]), n("Identity", ["present_key_cross_0"], ["present_value_cross_0"]),
                 n("Gather", ["Ed", "decoder_input_ids"], ["d_emb"]), n("MatMul", ["d_emb", "Wv2"], ["dv"]),
                 n("Unsqueeze", ["dv", "ax1"], ["present_key_self_0"]), n("Identity", ["present_key_self_0"], ["present_value_self_0"])] + ones_mask("encoder_hidden_states")
    enc_nodes = _encdec_common(enc_nodes, "encoder_hidden_states", "present_value_cross_0", "mask_f", "d_emb", "present_value_self_0")
    enc = ol.make_graph(enc_nodes, "encoder", [ol.make_tensor_value_info("encoder_input_ids", T.FLOAT, ["b", "se", D]),
                                                ol.make_tensor_value_info("decoder_input_ids", T.INT32, ["b", "p"])],
                        [ol.make_tensor_value_info(o, T.FLOAT, None) for o in ("logits", "encoder_hidden_states", "present_key_self_0", "present_value_self_0",
                                                                               "present_key_cross_0", "present_value_cross_0")], _encdec_inits() + extra)
    dec_nodes = [n("Gather", ["Ed", "input_ids"], ["d_emb"]), n("MatMul", ["d_emb", "Wv2"], ["dv"]), n("Unsqueeze", ["dv", "ax1"], ["dv4"]),
                 n("Concat", ["past_key_self_0", "dv4"], ["present_key_self_0"], axis=2), n("Concat", ["past_value_self_0", "dv4"], ["present_value_self_0"], axis=2),
                 n("Squeeze", ["past_key_cross_0", "ax1"], ["hidden_from_cross"])] + ones_mask("hidden_from_cross")
    dec_nodes = _encdec_common(dec_nodes, "hidden_from_cross", "past_value_cross_0", "mask_f", "d_emb", "present_value_self_0")
    dec_ins = [ol.make_tensor_value_info("input_ids", T.INT32, ["r", 1])]
    dec_ins += [ol.make_tensor_value_info(k, T.FLOAT, ["r", 1, "t", D]) for k in ("past_key_self_0", "past_value_self_0", "past_key_cross_0", "past_value_cross_0")]
    dec = ol.make_graph(dec_nodes, "decoder", dec_ins, [ol.make_tensor_value_info(o, T.FLOAT, None) for o in ("logits", "present_key_self_0", "present_value_self_0")],
                        _encdec_inits() + extra)
    inputs = ["input_features", "max_length", "min_length", "num_beams", "num_return_sequences", "length_penalty", "repetition_penalty", "", "", "", "decoder_input_ids"]
    node = ol.make_node("WhisperBeamSearch", inputs, ["sequences"], domain="com.microsoft", encoder=enc, decoder=dec, eos_token_id=eos, pad_token_id=0,
                        decoder_start_token_id=2)
    types = {"input_features": (T.FLOAT, ["b", "se", D]), "max_length": (T.INT32, [1]), "min_length": (T.INT32, [1]), "num_beams": (T.INT32, [1]),
             "num_return_sequences": (T.INT32, [1]), "length_penalty": (T.FLOAT, [1]), "repetition_penalty": (T.FLOAT, [1]), "decoder_input_ids": (T.INT32, ["b", "p"])}
    g = ol.make_graph([node], "g", [ol.make_tensor_value_info(k, *types[k]) for k in inputs if k], [ol.make_tensor_value_info("sequences", 0, None)])
    sess = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    feats = rng.randn(2, 6, D).astype(np.float32)
    prompt = np.array([[2, 7], [2, 9]], np.int32)
    got = sess.run(None, {"input_features": feats, "max_length": np.array([max_len], np.int32), "min_length": np.array([0], np.int32),
                          "num_beams": np.array([K], np.int32), "num_return_sequences": np.array([1], np.int32), "length_penalty": np.array([1.0], np.float32),
                          "repetition_penalty": np.array([1.0], np.float32), "decoder_input_ids": prompt})[0]
    for b in range(2):
        hidden = feats[b] @ W2["Wenc"]

        def fn(seq, hidden=hidden):
            seq = np.asarray(seq)
            return np.tanh(W2["Ed"][seq[-1]] + (W2["Ed"][seq] @ W2["Wv2"]).mean(0) + hidden.mean(0) + 0.1 * hidden.mean(0)) @ W2["Wo2"]
        (score, seq), = _ref_beam(list(prompt[b]), K, max_len, eos, 1.0, 1, logits_fn=fn)
        np.testing.assert_array_equal(got[b, 0, :len(seq)], np.array(seq, np.int32))


def test_convert_generation_tool_wraps_a_decoder_file(tmp_path):
    """transformers.convert_generation: decoder.onnx -> a model with one BeamSearch node, same result as the hand-built one."""
    from onnxruntime_b200.transformers import convert_generation as cg
    dec_path, out_path = tmp_path / "decoder.onnx", tmp_path / "beam.onnx"
    dec_path.write_bytes(ol.make_model(decoder_body()).serialize())
    assert cg.main(["--decoder_onnx", str(dec_path), "--output", str(out_path), "--num_beams_op", "beam", "--eos_token_id", "5"]) == 0
    sess = ort.InferenceSession(str(out_path), providers=["CPUExecutionProvider"])
    assert [i.name for i in sess.get_inputs()] == ["input_ids", "max_length", "min_length", "num_beams", "num_return_sequences", "length_penalty",
                                                   "repetition_penalty", "attention_mask"]
    ids = np.array([[3, 9, 1, 4]], np.int32)
    seqs, scores = sess.run(None, {"input_ids": ids, "max_length": np.array([10], np.int32), "min_length": np.array([0], np.int32),
                                   "num_beams": np.array([3], np.int32), "num_return_sequences": np.array([1], np.int32),
                                   "length_penalty": np.array([1.0], np.float32), "repetition_penalty": np.array([1.0], np.float32),
                                   "attention_mask": np.ones((1, 4), np.int32)})
    (score, seq), = _ref_beam(list(ids[0]), 3, 10, 5, 1.0, 1)
    np.testing.assert_array_equal(seqs[0, 0, :len(seq)], np.array(seq, np.int32))
    assert abs(scores[0, 0] - score) < 1e-3
