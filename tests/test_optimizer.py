"""Graph optimizer: each fusion is checked by op counts before/after AND by numerical equivalence of the
optimized and unoptimized sessions (the approach of the reference's TransformerTester,
onnxruntime/test/optimizer/graph_transform_test.cc)."""
import math

import numpy as np
import pytest

import onnxruntime_b200 as ort
from onnxruntime_b200 import _core as C
from onnxruntime_b200 import onnx_lite as ol
from helpers import graph_model, op_counts

T = ol.TensorProto
rng = np.random.RandomState(0)


def both(model, feeds, disabled=()):
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    ref = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    opt = ort.InferenceSession(model, providers=["CPUExecutionProvider"], disabled_optimizers=list(disabled))
    a, b = ref.run(None, feeds), opt.run(None, feeds)
    for x, y in zip(a, b):
        np.testing.assert_allclose(x, y, rtol=2e-5, atol=2e-6)
    return op_counts(ref), op_counts(opt)


def c(name, value, dtype=np.float32):
    return ol.make_tensor(name, np.asarray(value, dtype=dtype))


X = [ol.make_tensor_value_info("x", T.FLOAT, ["b", 8, 16])]
Y = [ol.make_tensor_value_info("y", T.FLOAT, None)]
xs = {"x": rng.randn(2, 8, 16).astype(np.float32)}


def test_identity_dropout_noop_elimination():
    nodes = [ol.make_node("Identity", ["x"], ["a"]), ol.make_node("Dropout", ["a"], ["b"]),
             ol.make_node("Add", ["b", "zero"], ["c"]), ol.make_node("Mul", ["c", "one"], ["d"]), ol.make_node("Relu", ["d"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, [c("zero", 0.0), c("one", 1.0)]), xs)
    assert after == {"Relu": 1}


def test_constant_folding_and_cse():
    nodes = [ol.make_node("Add", ["k1", "k2"], ["k3"]), ol.make_node("Mul", ["x", "k3"], ["a"]),
             ol.make_node("Mul", ["x", "k3"], ["b"]), ol.make_node("Add", ["a", "b"], ["y"]),
             ol.make_node("Constant", [], ["unused"], value=np.ones(2, np.float32))]
    before, after = both(graph_model(nodes, X, Y, [c("k1", [1.0] * 16), c("k2", [2.0] * 16)]), xs)
    assert before["Mul"] == 2 and after == {"Mul": 1, "Add": 1}
    # disabling a pass by name keeps its pattern
    _, kept = both(graph_model(nodes, X, Y, [c("k1", [1.0] * 16), c("k2", [2.0] * 16)]), xs,
                   disabled=["CommonSubexpressionElimination"])
    assert kept["Mul"] == 2


def test_shape_chain_folds_with_static_initializer():
    nodes = [ol.make_node("Shape", ["w"], ["s"]), ol.make_node("Gather", ["s", "i0"], ["d"], axis=0),
             ol.make_node("Unsqueeze", ["d", "ax"], ["d1"]), ol.make_node("Concat", ["m1", "d1"], ["shape"], axis=0),
             ol.make_node("Reshape", ["x", "shape"], ["y"])]
    inits = [c("w", np.zeros((16, 4))), c("i0", 0, np.int64), c("ax", [0], np.int64), c("m1", [-1], np.int64)]
    before, after = both(graph_model(nodes, X, Y, inits), xs)
    assert after == {"Reshape": 1}


@pytest.mark.parametrize("form", [0, 1, 2])
def test_gelu_fusion(form):
    e = [ol.make_node("Div", ["x", "sqrt2"], ["d"]), ol.make_node("Erf", ["d"], ["e"]), ol.make_node("Add", ["e", "one"], ["p"])]
    if form == 0:
        tail = [ol.make_node("Mul", ["x", "p"], ["m"]), ol.make_node("Mul", ["m", "half"], ["y"])]
    elif form == 1:
        tail = [ol.make_node("Mul", ["x", "half"], ["m"]), ol.make_node("Mul", ["m", "p"], ["y"])]
    else:
        tail = [ol.make_node("Mul", ["half", "p"], ["m"]), ol.make_node("Mul", ["x", "m"], ["y"])]
    before, after = both(graph_model(e + tail, X, Y, [c("sqrt2", math.sqrt(2)), c("one", 1.0), c("half", 0.5)]), xs)
    assert after == {"Gelu": 1}


@pytest.mark.parametrize("form", [0, 1])
def test_fast_gelu_fusion(form):
    k0 = math.sqrt(2 / math.pi)
    if form == 0:
        inner = [ol.make_node("Pow", ["x", "three"], ["x3"]), ol.make_node("Mul", ["k1", "x3"], ["a"]),
                 ol.make_node("Add", ["x", "a"], ["b"]), ol.make_node("Mul", ["k0", "b"], ["inner"])]
    else:
        inner = [ol.make_node("Mul", ["x", "x"], ["x2"]), ol.make_node("Mul", ["k1", "x2"], ["a"]),
                 ol.make_node("Add", ["one", "a"], ["b"]), ol.make_node("Mul", ["x", "k0"], ["xk"]),
                 ol.make_node("Mul", ["xk", "b"], ["inner"])]
    tail = [ol.make_node("Tanh", ["inner"], ["t"]), ol.make_node("Add", ["one", "t"], ["p"]),
            ol.make_node("Mul", ["x", "half"], ["h"]), ol.make_node("Mul", ["h", "p"], ["y"])]
    inits = [c("three", 3.0), c("k1", 0.044715), c("k0", k0), c("one", 1.0), c("half", 0.5)]
    before, after = both(graph_model(inner + tail, X, Y, inits), xs)
    assert after == {"FastGelu": 1}


def _layernorm_nodes(src, out, dup_sub=False):
    n = [ol.make_node("ReduceMean", [src], ["mu"], axes=[-1]), ol.make_node("Sub", [src, "mu"], ["d"])]
    d2 = "d"
    if dup_sub:
        n.append(ol.make_node("Sub", [src, "mu"], ["d_b"]))
        d2 = "d_b"
    n += [ol.make_node("Pow", [d2, "two"], ["sq"]), ol.make_node("ReduceMean", ["sq"], ["var"], axes=[-1]),
          ol.make_node("Add", ["var", "eps"], ["ve"]), ol.make_node("Sqrt", ["ve"], ["sd"]), ol.make_node("Div", ["d", "sd"], ["nrm"]),
          ol.make_node("Mul", ["nrm", "gamma"], ["sc"]), ol.make_node("Add", ["sc", "beta"], [out])]
    return n


LN_INITS = [c("two", 2.0), c("eps", 1e-5), c("gamma", rng.randn(16)), c("beta", rng.randn(16))]


@pytest.mark.parametrize("dup_sub", [False, True])
def test_layernorm_fusion(dup_sub):
    before, after = both(graph_model(_layernorm_nodes("x", "y", dup_sub), X, Y, LN_INITS), xs)
    assert after == {"LayerNormalization": 1}


def test_layernorm_not_fused_when_interior_value_escapes():
    nodes = _layernorm_nodes("x", "y0") + [ol.make_node("Add", ["y0", "var"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, LN_INITS), xs)
    assert "LayerNormalization" not in after


@pytest.mark.parametrize("form", ["div", "recip_mul", "cast"])
def test_simplified_layernorm_fusion(form):
    n = [ol.make_node("Pow", ["x", "two"], ["sq"]), ol.make_node("ReduceMean", ["sq"], ["ms"], axes=[-1]),
         ol.make_node("Add", ["ms", "eps"], ["ve"]), ol.make_node("Sqrt", ["ve"], ["rms"])]
    if form == "div":
        n += [ol.make_node("Div", ["x", "rms"], ["nrm"]), ol.make_node("Mul", ["nrm", "gamma"], ["y"])]
    elif form == "recip_mul":
        n += [ol.make_node("Div", ["one", "rms"], ["inv"]), ol.make_node("Mul", ["x", "inv"], ["nrm"]),
              ol.make_node("Mul", ["gamma", "nrm"], ["y"])]
    else:
        n += [ol.make_node("Div", ["x", "rms"], ["nrm"]), ol.make_node("Cast", ["nrm"], ["nc"], to=T.FLOAT),
              ol.make_node("Mul", ["nc", "gamma"], ["y"])]
    before, after = both(graph_model(n, X, Y, LN_INITS + [c("one", 1.0)]), xs)
    assert after == {"SimplifiedLayerNormalization": 1}


def test_skip_layernorm_and_bias_gelu_fusion():
    # (x @ W + b) -> gelu ; residual add -> layernorm, with the sum consumed twice
    W, b = rng.randn(16, 16).astype(np.float32), rng.randn(16).astype(np.float32)
    nodes = [ol.make_node("MatMul", ["x", "W"], ["mm"]), ol.make_node("Add", ["mm", "b"], ["mb"]),
             ol.make_node("Gelu", ["mb"], ["g"], domain="com.microsoft"),
             ol.make_node("Add", ["g", "x"], ["sum"]),
             ol.make_node("LayerNormalization", ["sum", "gamma", "beta"], ["ln"], axis=-1, epsilon=1e-5),
             ol.make_node("Add", ["ln", "sum"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, LN_INITS + [c("W", W), c("b", b)]), xs)
    assert after.get("SkipLayerNormalization") == 1 and after.get("BiasGelu") == 1 and "LayerNormalization" not in after
    # bias feeding the residual add is absorbed as the SkipLayerNorm bias input
    nodes = [ol.make_node("MatMul", ["x", "W"], ["mm"]), ol.make_node("Add", ["mm", "b"], ["mb"]), ol.make_node("Add", ["mb", "x"], ["sum"]),
             ol.make_node("SimplifiedLayerNormalization", ["sum", "gamma"], ["y"], axis=-1, epsilon=1e-5)]
    before, after = both(graph_model(nodes, X, Y, LN_INITS + [c("W", W), c("b", b)]), xs)
    assert after == {"MatMul": 1, "SkipSimplifiedLayerNormalization": 1}


def test_bert_fusions_end_to_end():
    from onnxruntime_b200.models.bert import BertConfig, build_bert, init_weights, reference_forward
    cfg = BertConfig(type_vocab_size=2)
    w = init_weights(cfg, 0)
    model = build_bert(cfg, w)
    ids = rng.randint(0, cfg.vocab_size, (2, 32)).astype(np.int64)
    mask = np.ones((2, 32), np.int64)
    mask[1, 25:] = 0
    tt = rng.randint(0, 2, (2, 32)).astype(np.int64)
    feeds = {"input_ids": ids, "attention_mask": mask, "token_type_ids": tt}
    before, after = both(model, feeds)
    assert after["Attention"] == cfg.num_layers and after["SkipLayerNormalization"] == 2 * cfg.num_layers
    assert after["BiasGelu"] == cfg.num_layers and after["EmbedLayerNormalization"] == 1
    assert "Softmax" not in after and "Erf" not in after and sum(after.values()) < sum(before.values()) // 4
    s = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    out = s.run(None, feeds)[0]
    ref = reference_forward(cfg, w, ids, mask, tt)
    valid = mask.astype(bool)
    np.testing.assert_allclose(out[valid], ref[valid], rtol=1e-4, atol=2e-5)


def test_conv_batchnorm_fusion():
    x = rng.randn(1, 3, 8, 8).astype(np.float32)
    inits = [c("w", rng.randn(4, 3, 3, 3)), c("s", rng.rand(4) + 0.5), c("b", rng.randn(4)), c("m", rng.randn(4)), c("v", rng.rand(4) + 0.5)]
    nodes = [ol.make_node("Conv", ["x", "w"], ["cv"], kernel_shape=[3, 3]), ol.make_node("BatchNormalization", ["cv", "s", "b", "m", "v"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, [1, 3, 8, 8])], Y, inits)
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    a = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    opt = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(opt.run(None, {"x": x})[0], a, rtol=1e-4, atol=1e-4)
    assert op_counts(opt) == {"Conv": 1}


def test_gpu_lowering_passes_on_graph_level():
    """The GPU-only passes are pure graph rewrites, so their structure can be checked without a GPU."""
    import torch
    W1, W2, W3 = (torch.randn(64, 128) * 0.05).half(), (torch.randn(64, 128) * 0.05).half(), (torch.randn(128, 64) * 0.05).half()
    bias = torch.randn(64).half()
    nodes = [ol.make_node("MatMul", ["x", "Wg"], ["g"]), ol.make_node("MatMul", ["x", "Wu"], ["u"]),
             ol.make_node("Sigmoid", ["g"], ["sg"]), ol.make_node("Mul", ["g", "sg"], ["act"]), ol.make_node("Mul", ["act", "u"], ["h"]),
             ol.make_node("MatMul", ["h", "Wd"], ["d"]), ol.make_node("Add", ["d", "bias"], ["db"]),
             ol.make_node("FastGelu", ["db"], ["fg"], domain="com.microsoft"), ol.make_node("Add", ["fg", "x"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", 64])], [ol.make_tensor_value_info("y", T.FLOAT16, ["b", 64])],
                        [ol.make_tensor("Wg", W1), ol.make_tensor("Wu", W2), ol.make_tensor("Wd", W3), ol.make_tensor("bias", bias)])
    out, stats = C.optimize_model(model, 99, [], True)
    ops = [(n["op_type"], n["domain"]) for n in C.model_nodes(out)]
    assert ops == [("GemmSwiGLU", "com.ortb200"), ("FusedGemm", "com.ortb200")]
    fused = C.model_nodes(out)[1]
    assert fused["attrs"]["activation"] == b"fastgelu" and len(fused["inputs"]) == 4
    # the fused ops also run on the CPU provider (ATen reference kernels), so the rewrite can be verified numerically
    x = (torch.randn(3, 64) * 0.5).half().numpy()
    a = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    b = ort.InferenceSession(out, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    np.testing.assert_allclose(a.astype(np.float32), b.astype(np.float32), rtol=2e-2, atol=2e-2)


def test_rms_norm_folds_into_the_surrounding_gemms():
    """x -> GEMM -> (+residual, RMS norm) -> GEMM / SwiGLU pair: the add moves into the first GEMM's epilogue and the
    norm into the second GEMM (gamma into its weights, 1/rms as an epilogue factor)."""
    import torch
    torch.manual_seed(0)
    H, F = 64, 128
    W1, Wq = (torch.randn(H, H) * 0.1).half(), (torch.randn(H, 96) * 0.1).half()
    Wg, Wu, Wd = (torch.randn(H, F) * 0.1).half(), (torch.randn(H, F) * 0.1).half(), (torch.randn(F, H) * 0.1).half()
    g0, g1, g2 = (torch.rand(H) + 0.5).half(), (torch.rand(H) + 0.5).half(), (torch.rand(H) + 0.5).half()
    nodes = [ol.make_node("SimplifiedLayerNormalization", ["x", "g0"], ["n0"], axis=-1, epsilon=1e-5),
             ol.make_node("MatMul", ["n0", "W1"], ["o"]),
             ol.make_node("SkipSimplifiedLayerNormalization", ["o", "x", "g1"], ["n1", "", "", "res1"], domain="com.microsoft", epsilon=1e-5),
             ol.make_node("MatMul", ["n1", "Wg"], ["g"]), ol.make_node("MatMul", ["n1", "Wu"], ["u"]),
             ol.make_node("Sigmoid", ["g"], ["sg"]), ol.make_node("Mul", ["g", "sg"], ["act"]), ol.make_node("Mul", ["act", "u"], ["h"]),
             ol.make_node("MatMul", ["h", "Wd"], ["d"]),
             ol.make_node("SkipSimplifiedLayerNormalization", ["d", "res1", "g2"], ["n2", "", "", "res2"], domain="com.microsoft", epsilon=1e-5),
             ol.make_node("MatMul", ["n2", "Wq"], ["q"]), ol.make_node("Identity", ["res2"], ["stream"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", H])],
                        [ol.make_tensor_value_info("q", T.FLOAT16, None), ol.make_tensor_value_info("stream", T.FLOAT16, None)],
                        [ol.make_tensor(n, v) for n, v in (("W1", W1), ("Wq", Wq), ("Wg", Wg), ("Wu", Wu), ("Wd", Wd), ("g0", g0), ("g1", g1), ("g2", g2))])
    out, stats = C.optimize_model(model, 99, [], True)
    assert stats["RmsNormGemmFusion"] == 3
    nodes_out = C.model_nodes(out)
    ops = [n["op_type"] for n in nodes_out]
    assert "SkipSimplifiedLayerNormalization" not in ops and "SimplifiedLayerNormalization" not in ops
    assert ops.count("FusedGemm") == 3 and ops.count("GemmSwiGLU") == 1
    assert sum(1 for n in nodes_out if "rms_eps" in n["attrs"]) == 3
    x = (torch.randn(5, H) * 0.7).half().numpy()
    a = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    b = ort.InferenceSession(out, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    for u, v in zip(a, b):
        np.testing.assert_allclose(u.astype(np.float32), v.astype(np.float32), rtol=2e-2, atol=2e-2)
    # without the GPU passes the norms stay
    plain, _ = C.optimize_model(model, 99, [], False)
    assert "SkipSimplifiedLayerNormalization" in [n["op_type"] for n in C.model_nodes(plain)]


def _attention_block(scale_node: bool, mask_kind: str):
    """One self-attention block on x [b, 8, 16] with 2 heads, built node by node.  mask_kind: "none", "keep" (the
    (1 - mask) * -10000 expansion of a 2-D keep-mask) or "additive" (a float [b, 1, 1, 8] term added to the scores)."""
    Hd, heads, hs = 16, 2, 8
    inits = [c("shape4", [0, 0, heads, hs], np.int64), c("shape3", [0, 0, Hd], np.int64)]
    nodes = []
    for nm in "qkv":
        inits += [c("W" + nm, rng.randn(Hd, Hd) * 0.3), c("B" + nm, rng.randn(Hd) * 0.1)]
        nodes += [ol.make_node("MatMul", ["x", "W" + nm], [nm + "_mm"]), ol.make_node("Add", [nm + "_mm", "B" + nm], [nm + "_b"]),
                  ol.make_node("Reshape", [nm + "_b", "shape4"], [nm + "_r"]),
                  ol.make_node("Transpose", [nm + "_r"], [nm + "_t"], perm=[0, 2, 3, 1] if nm == "k" else [0, 2, 1, 3])]
    nodes.append(ol.make_node("MatMul", ["q_t", "k_t"], ["qk"]))
    scores = "qk"
    if scale_node:
        inits.append(c("sqrt_hs", math.sqrt(hs)))
        nodes.append(ol.make_node("Div", ["qk", "sqrt_hs"], ["qk_s"]))
        scores = "qk_s"
    ins = list(X)
    if mask_kind == "keep":
        ins.append(ol.make_tensor_value_info("mask", T.INT64, ["b", 8]))
        inits += [c("ax1", [1], np.int64), c("ax2", [2], np.int64), c("one", 1.0), c("neg", -10000.0)]
        nodes += [ol.make_node("Unsqueeze", ["mask", "ax1"], ["m1"]), ol.make_node("Unsqueeze", ["m1", "ax2"], ["m2"]),
                  ol.make_node("Cast", ["m2"], ["mf"], to=T.FLOAT), ol.make_node("Sub", ["one", "mf"], ["inv"]),
                  ol.make_node("Mul", ["inv", "neg"], ["addm"]), ol.make_node("Add", [scores, "addm"], ["masked"])]
        scores = "masked"
    elif mask_kind == "additive":
        ins.append(ol.make_tensor_value_info("bias4", T.FLOAT, ["b", 1, 1, 8]))
        nodes.append(ol.make_node("Add", [scores, "bias4"], ["masked"]))
        scores = "masked"
    nodes += [ol.make_node("Softmax", [scores], ["p"], axis=-1), ol.make_node("MatMul", ["p", "v_t"], ["ctx"]),
              ol.make_node("Transpose", ["ctx"], ["ctx_t"], perm=[0, 2, 1, 3]), ol.make_node("Reshape", ["ctx_t", "shape3"], ["y"])]
    return graph_model(nodes, ins, Y, inits)


@pytest.mark.parametrize("scale_node", [True, False])
def test_attention_fusion_keeps_the_blocks_own_scaling(scale_node):
    """A block without a Div / Mul on the scores (scale folded into the weights, or none) must not pick up the fused
    operator's default 1 / sqrt(head size)."""
    before, after = both(_attention_block(scale_node, "none"), xs)
    assert after.get("Attention") == 1 and "Softmax" not in after


def test_attention_fusion_understands_only_the_keep_mask_expansion():
    keep = np.ones((2, 8), np.int64)
    keep[1, 5:] = 0
    before, after = both(_attention_block(True, "keep"), dict(xs, mask=keep))
    assert after.get("Attention") == 1
    # an additive float term is not a keep-mask: the block stays as it is and the numbers stay right
    bias4 = np.zeros((2, 1, 1, 8), np.float32)
    bias4[0, ..., 6:] = -10000.0
    before, after = both(_attention_block(True, "additive"), dict(xs, bias4=bias4))
    assert "Attention" not in after and after.get("Softmax", 0) + after.get("BiasSoftmax", 0) == 1


# ---------------------------------------------------------------------------------------------------------------
# smaller rewrite rules (matmul_add_fusion, reshape_fusion, constant_sharing, bias_softmax_fusion, cast_elimination, ...)
X2 = [ol.make_tensor_value_info("x", T.FLOAT, ["b", 16])]
x2 = {"x": rng.randn(3, 16).astype(np.float32)}


def test_matmul_add_becomes_gemm_for_2d_inputs_only():
    inits = [c("W", rng.randn(16, 8)), c("bias", rng.randn(8))]
    nodes = [ol.make_node("MatMul", ["x", "W"], ["m"]), ol.make_node("Add", ["m", "bias"], ["y"])]
    before, after = both(graph_model(nodes, X2, Y, inits), x2)
    assert after == {"Gemm": 1}
    before, after = both(graph_model(nodes, X, Y, inits), xs)   # 3-D input: left alone
    assert "Gemm" not in after


def test_reshape_fusion_replaces_the_shape_gather_concat_target():
    inits = [c("i0", 0, np.int64), c("i1", 1, np.int64), c("ax", [0], np.int64), c("hh", [4, 4], np.int64)]
    nodes = [ol.make_node("Shape", ["x"], ["s"]), ol.make_node("Gather", ["s", "i0"], ["b"], axis=0), ol.make_node("Gather", ["s", "i1"], ["q"], axis=0),
             ol.make_node("Unsqueeze", ["b", "ax"], ["b1"]), ol.make_node("Unsqueeze", ["q", "ax"], ["q1"]),
             ol.make_node("Concat", ["b1", "q1", "hh"], ["target"], axis=0), ol.make_node("Reshape", ["x", "target"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, inits), xs)
    assert after == {"Reshape": 1}


def test_constant_sharing_cast_and_trivial_node_elimination():
    inits = [c("e1", 1e-5), c("e2", 1e-5), c("st", [0], np.int64), c("en", [2 ** 31 - 1], np.int64), c("ax", [1], np.int64)]
    nodes = [ol.make_node("Cast", ["x"], ["xc"], to=T.FLOAT), ol.make_node("Add", ["xc", "e1"], ["a"]), ol.make_node("Add", ["a", "e2"], ["b"]),
             ol.make_node("Slice", ["b", "st", "en", "ax"], ["sl"]), ol.make_node("Relu", ["sl"], ["y"])]
    model = graph_model(nodes, X, Y, inits)
    before, after = both(model, xs)
    assert after == {"Add": 2, "Relu": 1}
    out, stats = C.optimize_model(model, 1, [], False)
    assert stats.get("ConstantSharing") == 1 and stats.get("CastElimination") == 1 and stats.get("TrivialNodeElimination") == 1


def test_bias_softmax_div_mul_not_where_relu_clip():
    inits = [c("bias", rng.randn(8, 16)), c("one", 1.0), c("lo", -1.0), c("hi", 2.0)]
    nodes = [ol.make_node("Add", ["x", "bias"], ["xb"]), ol.make_node("Softmax", ["xb"], ["p"], axis=-1),
             ol.make_node("Div", ["one", "p"], ["inv"]), ol.make_node("Mul", ["inv", "x"], ["q"]),
             ol.make_node("Greater", ["q", "one"], ["g"]), ol.make_node("Not", ["g"], ["ng"]), ol.make_node("Where", ["ng", "x", "q"], ["w"]),
             ol.make_node("Relu", ["w"], ["r"]), ol.make_node("Clip", ["r", "lo", "hi"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, inits), xs)
    assert after.get("BiasSoftmax") == 1 and "Softmax" not in after
    assert after.get("Div") == 1 and "Mul" not in after
    assert "Not" not in after and "Relu" not in after and after.get("Clip") == 1


def test_transpose_pairs_and_gemm_transposes():
    inits = [c("W", rng.randn(8, 16))]
    nodes = [ol.make_node("Transpose", ["x"], ["t1"], perm=[0, 2, 1]), ol.make_node("Transpose", ["t1"], ["t2"], perm=[0, 2, 1]),
             ol.make_node("Transpose", ["t2"], ["t3"], perm=[1, 0, 2]), ol.make_node("Transpose", ["t3"], ["t4"], perm=[0, 2, 1]),
             ol.make_node("Relu", ["t4"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, []), xs)
    assert after == {"Transpose": 1, "Relu": 1}
    nodes = [ol.make_node("Transpose", ["W"], ["wt"], perm=[1, 0]), ol.make_node("Transpose", ["x"], ["xt"], perm=[1, 0]),
             ol.make_node("Transpose", ["xt"], ["xtt"], perm=[1, 0]), ol.make_node("Gemm", ["xtt", "wt"], ["y"])]
    # W is a graph input here so that constant folding does not remove the Transpose first
    ins = X2 + [ol.make_tensor_value_info("W", T.FLOAT, [8, 16])]
    before, after = both(graph_model(nodes, ins, Y, []), dict(x2, W=rng.randn(8, 16).astype(np.float32)))
    assert after == {"Gemm": 1}


def test_double_qdq_pair_removed():
    inits = [c("s", 0.02), ol.make_tensor("z", np.array(128, np.uint8))]
    nodes = [ol.make_node("QuantizeLinear", ["x", "s", "z"], ["q1"]), ol.make_node("DequantizeLinear", ["q1", "s", "z"], ["d1"]),
             ol.make_node("QuantizeLinear", ["d1", "s", "z"], ["q2"]), ol.make_node("DequantizeLinear", ["q2", "s", "z"], ["y"])]
    before, after = both(graph_model(nodes, X, Y, inits), xs)
    assert after == {"QuantizeLinear": 1, "DequantizeLinear": 1}


def test_nbits_gate_up_merge_and_swiglu_on_graph_level():
    """4-bit gate / up projections sharing an input become one MatMulNBits over the stacked rows plus a streaming SwiGLU."""
    import torch
    torch.manual_seed(0)
    K, I = 64, 96
    def q4(seed):
        g = torch.Generator().manual_seed(seed)
        return (torch.randint(0, 256, (I, K // 32, 16), generator=g, dtype=torch.uint8), (torch.rand(I, K // 32, generator=g) * 0.02 + 0.01).half())
    (bg, sg), (bu, su) = q4(1), q4(2)
    nodes = [ol.make_node("MatMulNBits", ["x", "Bg", "Sg"], ["g"], domain="com.microsoft", K=K, N=I, bits=4, block_size=32),
             ol.make_node("MatMulNBits", ["x", "Bu", "Su"], ["u"], domain="com.microsoft", K=K, N=I, bits=4, block_size=32),
             ol.make_node("Sigmoid", ["g"], ["sg"]), ol.make_node("Mul", ["g", "sg"], ["act"]), ol.make_node("Mul", ["act", "u"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", K])], [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                        [ol.make_tensor("Bg", bg), ol.make_tensor("Sg", sg), ol.make_tensor("Bu", bu), ol.make_tensor("Su", su)])
    out, stats = C.optimize_model(model, 99, [], True)
    ops = [(n["op_type"], n["domain"]) for n in C.model_nodes(out)]
    assert stats.get("NBitsSwiGLUFusion") == 1 and ops == [("MatMulNBits", "com.microsoft"), ("SwiGLU", "com.ortb200")]
    x = (torch.randn(5, K) * 0.5).half().numpy()
    a = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    b = ort.InferenceSession(out, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    np.testing.assert_allclose(a.astype(np.float32), b.astype(np.float32), rtol=2e-2, atol=2e-3)


def test_qdq_fusion_turns_node_groups_into_quantised_operators():
    """DequantizeLinear -> op -> QuantizeLinear groups become QLinear* operators; results stay the same because the
    quantised kernels compute dequantise / float operator / requantise."""
    T = ol.TensorProto
    rng = np.random.default_rng(21)

    def qparams(name, scale, zp, dtype=np.uint8):
        return [ol.make_tensor(name + "_s", np.array(scale, np.float32)), ol.make_tensor(name + "_z", np.array(zp, dtype))]
    inits = []
    inits += qparams("x", 0.02, 128) + qparams("w", 0.01, 0, np.int8) + qparams("c", 0.05, 120) + qparams("p", 0.05, 120)
    inits += qparams("m", 0.1, 100) + qparams("a", 0.08, 110) + qparams("sm", 1 / 256, 0)
    wq = rng.integers(-100, 100, (4, 3, 3, 3)).astype(np.int8)
    bq = rng.integers(-500, 500, (4,)).astype(np.int32)
    w2q = rng.integers(-100, 100, (16, 8)).astype(np.int8)
    inits += [ol.make_tensor("wq", wq), ol.make_tensor("bq", bq), ol.make_tensor("b_s", np.array(0.02 * 0.01, np.float32)),
              ol.make_tensor("w2q", w2q), ol.make_tensor("shape", np.array([2, 16], np.int64))]
    nodes = [
        ol.make_node("QuantizeLinear", ["x", "x_s", "x_z"], ["xq"]),
        ol.make_node("DequantizeLinear", ["xq", "x_s", "x_z"], ["xd"]),
        ol.make_node("DequantizeLinear", ["wq", "w_s", "w_z"], ["wd"]),
        ol.make_node("DequantizeLinear", ["bq", "b_s"], ["bd"]),
        ol.make_node("Conv", ["xd", "wd", "bd"], ["conv"], pads=[1, 1, 1, 1], name="conv0"),
        ol.make_node("QuantizeLinear", ["conv", "c_s", "c_z"], ["convq"]),
        ol.make_node("DequantizeLinear", ["convq", "c_s", "c_z"], ["convd"]),
        ol.make_node("MaxPool", ["convd"], ["pool"], kernel_shape=[2, 2], strides=[2, 2], name="pool0"),
        ol.make_node("QuantizeLinear", ["pool", "p_s", "p_z"], ["poolq"]),
        ol.make_node("Reshape", ["poolq", "shape"], ["flatq"]),
        ol.make_node("DequantizeLinear", ["flatq", "p_s", "p_z"], ["flatd"]),
        ol.make_node("DequantizeLinear", ["w2q", "w_s", "w_z"], ["w2d"]),
        ol.make_node("MatMul", ["flatd", "w2d"], ["mm"], name="mm0"),
        ol.make_node("QuantizeLinear", ["mm", "m_s", "m_z"], ["mmq"]),
        ol.make_node("DequantizeLinear", ["mmq", "m_s", "m_z"], ["mmd1"]),
        ol.make_node("DequantizeLinear", ["mmq", "m_s", "m_z"], ["mmd2"]),
        ol.make_node("Add", ["mmd1", "mmd2"], ["sum"], name="add0"),
        ol.make_node("QuantizeLinear", ["sum", "a_s", "a_z"], ["sumq"]),
        ol.make_node("DequantizeLinear", ["sumq", "a_s", "a_z"], ["sumd"]),
        ol.make_node("Softmax", ["sumd"], ["soft"], axis=-1, name="soft0"),
        ol.make_node("QuantizeLinear", ["soft", "sm_s", "sm_z"], ["softq"]),
        ol.make_node("DequantizeLinear", ["softq", "sm_s", "sm_z"], ["y"]),
    ]
    g = ol.make_graph(nodes, "qdq", [ol.make_tensor_value_info("x", T.FLOAT, [2, 3, 4, 4])], [ol.make_tensor_value_info("y", T.FLOAT, [2, 8])], inits)
    model = ol.make_model(g, opset=17).serialize()
    x = rng.uniform(-2, 2, (2, 3, 4, 4)).astype(np.float32)
    so0 = ort.SessionOptions()
    so0.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    plain = ort.InferenceSession(model, so0, providers=["CPUExecutionProvider"])
    fused = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    counts = op_counts(fused)
    assert counts.get("QLinearConv") == 1 and counts.get("QLinearMatMul") == 1 and counts.get("QLinearAdd") == 1
    assert counts.get("QLinearSoftmax") == 1 and counts.get("MaxPool") == 1
    assert counts.get("Conv", 0) == 0 and counts.get("MatMul", 0) == 0 and counts.get("Softmax", 0) == 0
    assert counts.get("DequantizeLinear", 0) == 1 and counts.get("QuantizeLinear", 0) == 1   # only the model's two ends remain
    want = plain.run(None, {"x": x})[0]
    got = fused.run(None, {"x": x})[0]
    assert np.abs(got - want).max() <= 1 / 256 + 1e-6     # at most one quantisation step of the last stage
    so = ort.SessionOptions()
    so.add_session_config_entry("session.disable_quant_qdq", "1")
    off = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    assert "QLinearConv" not in op_counts(off)


def test_group_query_attention_fusion_takes_rotary_and_packs_qkv():
    B, S, N, Nk, H, maxpos = 2, 4, 2, 1, 8, 16
    hidden = N * H
    r = np.random.RandomState(5)
    ang = np.arange(maxpos)[:, None] * (1.0 / 10000 ** (np.arange(H // 2) / (H // 2)))[None, :]
    inits = [c("wq", r.randn(hidden, N * H) * 0.3), c("wk", r.randn(hidden, Nk * H) * 0.3), c("wv", r.randn(hidden, Nk * H) * 0.3),
             c("cos", np.cos(ang)), c("sin", np.sin(ang)),
             c("seqlens", np.full((B,), S - 1), np.int32), c("total", np.array(S), np.int32)]
    nodes = [
        ol.make_node("MatMul", ["x", "wq"], ["q"], name="q_proj"),
        ol.make_node("MatMul", ["x", "wk"], ["k"], name="k_proj"),
        ol.make_node("MatMul", ["x", "wv"], ["v"], name="v_proj"),
        ol.make_node("RotaryEmbedding", ["q", "pos", "cos", "sin"], ["qr"], domain="com.microsoft", num_heads=N),
        ol.make_node("RotaryEmbedding", ["k", "pos", "cos", "sin"], ["kr"], domain="com.microsoft", num_heads=Nk),
        ol.make_node("GroupQueryAttention", ["qr", "kr", "v", "pk", "pv", "seqlens", "total"], ["y", "nk", "nv"], domain="com.microsoft",
                     num_heads=N, kv_num_heads=Nk, name="gqa"),
    ]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, [B, S, hidden]), ol.make_tensor_value_info("pos", T.INT64, [B, S]),
                                   ol.make_tensor_value_info("pk", T.FLOAT, [B, Nk, 0, H]), ol.make_tensor_value_info("pv", T.FLOAT, [B, Nk, 0, H])],
                      [ol.make_tensor_value_info("y", T.FLOAT, None), ol.make_tensor_value_info("nk", T.FLOAT, None)], inits)
    model = ol.make_model(g, opset=17).serialize()
    feeds = {"x": r.randn(B, S, hidden).astype(np.float32), "pos": np.tile(np.arange(S, dtype=np.int64), (B, 1)),
             "pk": np.zeros((B, Nk, 0, H), np.float32), "pv": np.zeros((B, Nk, 0, H), np.float32)}
    before, after = both(model, feeds)
    assert before["RotaryEmbedding"] == 2 and before["MatMul"] == 3
    assert after.get("RotaryEmbedding", 0) == 0 and after["MatMul"] == 1 and after["GroupQueryAttention"] == 1


def test_slice_expand_conv_gemm_rewrites():
    r = np.random.RandomState(11)
    x4 = [ol.make_tensor_value_info("x", T.FLOAT, [2, 3, 6, 6])]
    inits = [c("w", r.randn(4, 3, 3, 3) * 0.3), c("b", r.randn(4)), c("addk", r.randn(1, 4, 1, 1)), c("mulk", r.randn(4, 1, 1)),
             c("starts", [0, 0], np.int64), c("ends", [2**31 - 1, 6], np.int64), c("axes", [1, 3], np.int64), c("shape", [1, 1, 4, 4], np.int64)]
    nodes = [ol.make_node("Slice", ["x", "starts", "ends", "axes"], ["xs"]),
             ol.make_node("Conv", ["xs", "w", "b"], ["cv"], name="conv0"),
             ol.make_node("Mul", ["cv", "mulk"], ["cm"]), ol.make_node("Add", ["addk", "cm"], ["ca"]),
             ol.make_node("Expand", ["ca", "shape"], ["ce"]), ol.make_node("Relu", ["ce"], ["y"])]
    model = graph_model(nodes, x4, Y, inits)
    before, after = both(model, {"x": r.randn(2, 3, 6, 6).astype(np.float32)})
    assert before["Slice"] == 1 and before["Expand"] == 1
    assert after == {"FusedConv": 1}                                  # slice and expand gone, Mul / Add folded, Relu fused
    # Gemm + Sum
    g_in = [ol.make_tensor_value_info("a", T.FLOAT, [5, 8]), ol.make_tensor_value_info("cc", T.FLOAT, [1, 7])]
    model = graph_model([ol.make_node("Gemm", ["a", "w2"], ["gm"]), ol.make_node("Sum", ["cc", "gm"], ["y"])], g_in, Y, [c("w2", r.randn(8, 7))])
    before, after = both(model, {"a": r.randn(5, 8).astype(np.float32), "cc": r.randn(1, 7).astype(np.float32)})
    assert after == {"Gemm": 1}


def test_matmul_scale_and_transpose_become_fused_matmul():
    r = np.random.RandomState(12)
    ins = [ol.make_tensor_value_info("a", T.FLOAT, [2, 4, 5]), ol.make_tensor_value_info("b", T.FLOAT, [2, 6, 5])]
    nodes = [ol.make_node("Mul", ["a", "two"], ["a2"]), ol.make_node("Transpose", ["b"], ["bt"], perm=[0, 2, 1]),
             ol.make_node("MatMul", ["a2", "bt"], ["mm"]), ol.make_node("Div", ["mm", "four"], ["y"])]
    model = graph_model(nodes, ins, Y, [c("two", 2.0), c("four", 4.0)])
    before, after = both(model, {"a": r.randn(2, 4, 5).astype(np.float32), "b": r.randn(2, 6, 5).astype(np.float32)})
    assert after == {"FusedMatMul": 1}


def test_integer_matmul_chain_becomes_dynamic_quantize_matmul():
    r = np.random.RandomState(13)
    wq = r.randint(-100, 100, (8, 6)).astype(np.int8)
    nodes = [ol.make_node("DynamicQuantizeLinear", ["x"], ["xq", "xs", "xz"]),
             ol.make_node("MatMulInteger", ["xq", "wq", "xz", "wz"], ["acc"]), ol.make_node("Cast", ["acc"], ["accf"], to=T.FLOAT),
             ol.make_node("Mul", ["xs", "ws"], ["s"]), ol.make_node("Mul", ["accf", "s"], ["scaled"]), ol.make_node("Add", ["scaled", "bias"], ["y"])]
    inits = [ol.make_tensor("wq", wq), c("wz", 0, np.int8), c("ws", [0.02]), c("bias", r.randn(6))]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, [3, 8])], Y, inits)
    before, after = both(model, {"x": r.randn(3, 8).astype(np.float32)})
    assert before["MatMulInteger"] == 1 and after == {"DynamicQuantizeMatMul": 1}


def test_bias_skip_layer_norm_and_gelu_approximation():
    r = np.random.RandomState(14)
    nodes = [ol.make_node("Add", ["x", "bias"], ["xb"]),
             ol.make_node("SkipLayerNormalization", ["xb", "skip", "gamma", "beta"], ["n"], domain="com.microsoft", epsilon=1e-5),
             ol.make_node("Gelu", ["n"], ["y"], domain="com.microsoft")]
    inits = [c("bias", r.randn(16)), c("gamma", r.randn(16)), c("beta", r.randn(16))]
    model = graph_model(nodes, X + [ol.make_tensor_value_info("skip", T.FLOAT, ["b", 8, 16])], Y, inits)
    feeds = {"x": xs["x"], "skip": r.randn(2, 8, 16).astype(np.float32)}
    before, after = both(model, feeds)
    assert after == {"SkipLayerNormalization": 1, "Gelu": 1}
    so = ort.SessionOptions()
    so.add_session_config_entry("optimization.enable_gelu_approximation", "1")
    approx = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    assert op_counts(approx) == {"SkipLayerNormalization": 1, "FastGelu": 1}
    so0 = ort.SessionOptions()
    so0.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    exact = ort.InferenceSession(model, so0, providers=["CPUExecutionProvider"]).run(None, feeds)[0]
    np.testing.assert_allclose(approx.run(None, feeds)[0], exact, rtol=0, atol=2e-3)     # tanh form: close, not equal


def test_allgather_matmul_fusion_on_graph_level():
    """AllGather (axis 0) feeding a MatMul with a constant 16-bit weight becomes one node when the job has several ranks."""
    w = (np.arange(32 * 16).reshape(32, 16) % 7 - 3).astype(np.float16)
    nodes = [ol.make_node("AllGather", ["x"], ["g"], domain="com.microsoft", axis=0, group_size=2), ol.make_node("MatMul", ["g", "w"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", 32])], [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                        [ol.make_tensor("w", w)])
    out, stats = C.optimize_model(model, 99, [], True, 2)
    assert stats.get("AllGatherMatMulFusion") == 1
    assert [(n["op_type"], n["domain"]) for n in C.model_nodes(out)] == [("AllGatherMatMul", "com.ortb200")]
    out1, stats1 = C.optimize_model(model, 99, [], True, 1)        # a single rank keeps the pair
    assert not stats1.get("AllGatherMatMulFusion")
    nodes[0] = ol.make_node("AllGather", ["x"], ["g"], domain="com.microsoft", axis=1, group_size=2)   # another axis: no fusion
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", 16])], [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                        [ol.make_tensor("w", w)])
    assert not C.optimize_model(model, 99, [], True, 2)[1].get("AllGatherMatMulFusion")


def test_cast_chain_and_pre_shape_elimination():
    nodes = [ol.make_node("Cast", ["h"], ["f"], to=T.FLOAT), ol.make_node("Cast", ["f"], ["d"], to=T.DOUBLE),
             ol.make_node("Cast", ["f2"], ["s_in"], to=T.FLOAT16), ol.make_node("Shape", ["s_in"], ["s"]),
             ol.make_node("Cast", ["h"], ["f2"], to=T.FLOAT), ol.make_node("Reshape", ["d", "s"], ["y"])]
    h = rng.randn(3, 4).astype(np.float16)
    model = graph_model([nodes[0], nodes[1], nodes[4], nodes[2], nodes[3], nodes[5]], [ol.make_tensor_value_info("h", T.FLOAT16, [3, 4])], Y)
    before, after = both(model, {"h": h})
    assert before["Cast"] == 4 and after == {"Cast": 1, "Shape": 1, "Reshape": 1}
    # a narrowing first cast is kept: fp32 -> fp16 -> fp32 rounds
    nodes = [ol.make_node("Cast", ["x"], ["a"], to=T.FLOAT16), ol.make_node("Cast", ["a"], ["y"], to=T.FLOAT)]
    _, after = both(graph_model(nodes, X, Y), xs)
    assert after == {"Cast": 2}


def test_pad_fusion_into_conv_and_average_pool():
    x = rng.randn(1, 3, 8, 8).astype(np.float32)
    w = rng.randn(4, 3, 3, 3).astype(np.float32)
    inputs = [ol.make_tensor_value_info("x", T.FLOAT, [1, 3, 8, 8])]
    pads = ol.make_tensor("pads", np.array([0, 0, 1, 2, 0, 0, 2, 1], np.int64))
    nodes = [ol.make_node("Pad", ["x", "pads"], ["p"], mode="constant"), ol.make_node("Conv", ["p", "w"], ["y"], pads=[1, 0, 0, 1])]
    before, after = both(graph_model(nodes, inputs, Y, [pads, ol.make_tensor("w", w)]), {"x": x})
    assert before == {"Pad": 1, "Conv": 1} and after == {"Conv": 1}
    nodes = [ol.make_node("Pad", ["x", "pads"], ["p"], mode="constant"), ol.make_node("AveragePool", ["p"], ["y"], kernel_shape=[3, 3], count_include_pad=1)]
    _, after = both(graph_model(nodes, inputs, Y, [pads]), {"x": x})
    assert after == {"AveragePool": 1}
    # pads that do not average in (count_include_pad = 0), a non-zero fill and padded batch / channel dims stay
    for node, extra in ((ol.make_node("AveragePool", ["p"], ["y"], kernel_shape=[3, 3]), [pads]),
                        (ol.make_node("Conv", ["p", "w"], ["y"]), [pads, ol.make_tensor("w", w), ol.make_tensor("v", np.array(1.5, np.float32))])):
        pad_inputs = ["x", "pads"] + (["v"] if len(extra) == 3 else [])
        _, after = both(graph_model([ol.make_node("Pad", pad_inputs, ["p"], mode="constant"), node], inputs, Y, extra), {"x": x})
        assert after.get("Pad") == 1


def test_matmul_batchnorm_fusion():
    x2 = rng.randn(5, 16).astype(np.float32)
    w = rng.randn(16, 6).astype(np.float32)
    inits = [ol.make_tensor("w", w), c("scale", rng.rand(6) + 0.5), c("beta", rng.randn(6)), c("mean", rng.randn(6)), c("var", rng.rand(6) + 0.1)]
    nodes = [ol.make_node("MatMul", ["x", "w"], ["m"]), ol.make_node("BatchNormalization", ["m", "scale", "beta", "mean", "var"], ["y"], epsilon=1e-3)]
    before, after = both(graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, ["n", 16])], Y, inits), {"x": x2})
    assert before == {"MatMul": 1, "BatchNormalization": 1} and after == {"Gemm": 1}


def test_label_encoder_fusion():
    nodes = [ol.make_node("LabelEncoder", ["x"], ["a"], domain="ai.onnx.ml", keys_int64s=[1, 2, 3], values_strings=["one", "two", "three"], default_string="none"),
             ol.make_node("LabelEncoder", ["a"], ["y"], domain="ai.onnx.ml", keys_strings=["one", "three", "none"], values_floats=[1.5, 3.5, -1.0], default_float=9.0)]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.INT64, ["n"])], Y)
    m = ol.make_model(g, opset=17)
    m.opset_imports["ai.onnx.ml"] = 4
    before, after = both(m.serialize(), {"x": np.array([1, 2, 3, 7], np.int64)})
    assert before == {"LabelEncoder": 2} and after == {"LabelEncoder": 1}
    out = ort.InferenceSession(m.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": np.array([1, 2, 3, 7], np.int64)})[0]
    np.testing.assert_array_equal(out, np.array([1.5, 9.0, 3.5, -1.0], np.float32))


def test_gemm_activation_fusion_and_shared_dequantize_is_duplicated():
    x2 = rng.randn(5, 16).astype(np.float32)
    inits = [ol.make_tensor("w", rng.randn(16, 6).astype(np.float32)), c("b", rng.randn(6))]
    for act, attrs in (("Relu", {}), ("LeakyRelu", {"alpha": 0.2}), ("Selu", {}), ("HardSigmoid", {"alpha": 0.3, "beta": 0.4}), ("Softsign", {})):
        nodes = [ol.make_node("Gemm", ["x", "w", "b"], ["g"], alpha=0.5), ol.make_node(act, ["g"], ["y"], **attrs)]
        before, after = both(graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, ["n", 16])], Y, inits), {"x": x2})
        assert after == {"FusedGemm": 1}, act
    # one DequantizeLinear of a constant feeding two MatMuls: each consumer gets its own copy
    wq = rng.randint(-100, 100, (16, 6)).astype(np.int8)
    nodes = [ol.make_node("DequantizeLinear", ["wq", "s", "z"], ["wd"]), ol.make_node("MatMul", ["x", "wd"], ["a"]),
             ol.make_node("MatMul", ["x", "wd"], ["b2"]), ol.make_node("Sub", ["a", "b2"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, ["n", 16])], Y, [ol.make_tensor("wq", wq), c("s", 0.02), ol.make_tensor("z", np.array(0, np.int8))])
    out, stats = C.optimize_model(model, 1, ["ConstantFolding", "CommonSubexpressionElimination"], False)
    assert stats.get("EnsureUniqueDQForNodeUnit") == 1
    assert [n["op_type"] for n in C.model_nodes(out)].count("DequantizeLinear") == 2


def test_qdq_final_cleanup():
    inits = [c("s", 0.05), ol.make_tensor("z", np.array(3, np.uint8))]
    q = rng.randint(0, 255, (4, 8)).astype(np.uint8)
    nodes = [ol.make_node("Transpose", ["q"], ["t"], perm=[1, 0]), ol.make_node("DequantizeLinear", ["t", "s", "z"], ["d"]),
             ol.make_node("QuantizeLinear", ["d", "s", "z"], ["q2"]), ol.make_node("Transpose", ["q2"], ["y"], perm=[1, 0])]
    model = graph_model(nodes, [ol.make_tensor_value_info("q", T.UINT8, [4, 8])], Y, inits)
    before, after = both(model, {"q": q}, disabled=["TransposePairFusion"])
    assert before["DequantizeLinear"] == 1 and "DequantizeLinear" not in after and "QuantizeLinear" not in after
    # Q -> DQ stands for a rounding step: kept unless the session asks for the clean-up
    nodes = [ol.make_node("Relu", ["x"], ["r"]), ol.make_node("QuantizeLinear", ["r", "s", "z"], ["qq"]), ol.make_node("DequantizeLinear", ["qq", "s", "z"], ["dd"]),
             ol.make_node("Relu", ["dd"], ["y"])]
    model = graph_model(nodes, X, Y, inits)
    _, after = both(model, xs, disabled=["QDQFusion"])
    assert after.get("QuantizeLinear") == 1
    so = ort.SessionOptions()
    so.add_session_config_entry("session.enable_quant_qdq_cleanup", "1")
    sess = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"], disabled_optimizers=["QDQFusion"])
    assert "QuantizeLinear" not in op_counts(sess)


def _pack4(values):
    v = (np.asarray(values).astype(np.int64).reshape(-1) & 15).astype(np.uint8)
    if v.size % 2:
        v = np.append(v, np.uint8(0))
    return (v[0::2] | (v[1::2] << 4)).tobytes()


@pytest.mark.parametrize("signed,with_zp", [(False, True), (False, False), (True, False), (True, True)])
def test_int4_dequantize_and_dq_matmul_nbits_fusion(signed, with_zp, tmp_path):
    """4-bit initializers load as one value per element; DequantizeLinear (block-wise along K) -> MatMul becomes
    MatMulNBits when the session asks for it, with the same result; the saved model keeps the 4-bit type."""
    K, N, bs = 48, 8, 16
    lo, hi = (-8, 8) if signed else (0, 16)
    w = rng.randint(lo, hi, (K, N))
    zp = rng.randint(lo, hi, (K // bs, N))
    scale = (rng.rand(K // bs, N) * 0.05 + 0.01).astype(np.float32)
    t4 = T.INT4 if signed else T.UINT4
    inits = [ol.Tensor("w", t4, (K, N), _pack4(w)), ol.make_tensor("s", scale)]
    dq_in = ["w", "s"]
    if with_zp:
        inits.append(ol.Tensor("z", t4, (K // bs, N), _pack4(zp)))
        dq_in.append("z")
    nodes = [ol.make_node("DequantizeLinear", dq_in, ["wd"], axis=0, block_size=bs), ol.make_node("MatMul", ["x", "wd"], ["y"])]
    model = ol.make_model(ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, ["n", K])], Y, inits), opset=21).serialize()
    x = rng.randn(5, K).astype(np.float32)
    ref = x @ ((w - (np.repeat(zp, bs, 0) if with_zp else 0)) * np.repeat(scale, bs, 0))
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    plain = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(plain.run(None, {"x": x})[0], ref, rtol=1e-4, atol=1e-4)
    so = ort.SessionOptions()
    so.add_session_config_entry("session.enable_dq_matmulnbits_fusion", "1")
    so.optimized_model_filepath = str(tmp_path / "fused.onnx")
    fused = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    assert op_counts(fused) == {"MatMulNBits": 1}
    np.testing.assert_allclose(fused.run(None, {"x": x})[0], ref, rtol=1e-4, atol=1e-4)
    # without the key a CPU session keeps the pair; a model saved from it still declares the 4-bit type
    so = ort.SessionOptions()
    so.optimized_model_filepath = str(tmp_path / "kept.onnx")
    kept = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"], disabled_optimizers=["ConstantFolding"])
    assert op_counts(kept).get("DequantizeLinear") == 1
    saved = ol.load_model(str(tmp_path / "kept.onnx"))
    wt = [t for t in saved.graph.initializers if t.name == "w"][0]
    assert wt.data_type == t4 and tuple(wt.dims) == (K, N) and bytes(wt.raw) == _pack4(w)
    np.testing.assert_allclose(ort.InferenceSession(str(tmp_path / "kept.onnx"), providers=["CPUExecutionProvider"]).run(None, {"x": x})[0], ref, rtol=1e-4, atol=1e-4)
