"""Static type / shape inference (per-operator functions) checked against what the engine actually produces."""
import numpy as np
import pytest

import onnxruntime_b200 as ort
from onnxruntime_b200 import _core as C
from onnxruntime_b200 import onnx_lite as ol
from helpers import graph_model

T = ol.TensorProto


def _value_info(model_bytes):
    m = ol.load_model(model_bytes)
    return {vi.name: (vi.elem_type, vi.shape) for vi in list(m.graph.value_info) + list(m.graph.outputs)}


def test_shape_chain_resolves_a_computed_reshape_target():
    """Shape -> Gather -> Unsqueeze -> Concat -> Reshape, the pattern exporters emit for [B, S, heads, head]."""
    inits = [ol.make_tensor("i0", np.array(0, np.int64)), ol.make_tensor("i1", np.array(1, np.int64)), ol.make_tensor("ax", np.array([0], np.int64)),
             ol.make_tensor("hh", np.array([4, 16], np.int64)), ol.make_tensor("W", np.zeros((64, 64), np.float32))]
    nodes = [ol.make_node("MatMul", ["x", "W"], ["p"]), ol.make_node("Shape", ["x"], ["s"]),
             ol.make_node("Gather", ["s", "i0"], ["b"], axis=0), ol.make_node("Gather", ["s", "i1"], ["q"], axis=0),
             ol.make_node("Unsqueeze", ["b", "ax"], ["b1"]), ol.make_node("Unsqueeze", ["q", "ax"], ["q1"]),
             ol.make_node("Concat", ["b1", "q1", "hh"], ["target"], axis=0), ol.make_node("Reshape", ["p", "target"], ["r"]),
             ol.make_node("Transpose", ["r"], ["t"], perm=[0, 2, 1, 3]), ol.make_node("Softmax", ["t"], ["y"], axis=-1)]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT, ["batch", "seq", 64])], [ol.make_tensor_value_info("y", T.FLOAT, None)], inits)
    out, rep = C.infer_shapes(model)
    vi = _value_info(out)
    assert rep["problems"] == [] and rep["inferred"] == rep["nodes"]
    assert vi["r"] == (T.FLOAT, ["batch", "seq", 4, 16])
    assert vi["y"] == (T.FLOAT, ["batch", 4, "seq", 16])
    # the session reports the inferred output shape although the file declared none
    sess = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    assert sess.get_outputs()[0].shape == ["batch", 4, "seq", 16]


def test_inferred_shapes_agree_with_execution_on_the_bert_graph():
    from onnxruntime_b200.models.bert import BertConfig, build_bert, init_weights
    cfg = BertConfig(type_vocab_size=2)
    model = build_bert(cfg, init_weights(cfg, 0))
    for level, strict in ((0, True), (99, True)):
        m = model if level == 0 else C.optimize_model(model, 99, [], False)[0]
        out, rep = C.infer_shapes(m, strict)
        assert rep["problems"] == []
        assert rep["inferred"] >= 0.9 * rep["nodes"], rep
        vi = _value_info(out)
        # the tracing tool runs the graph twice and observes every intermediate: both must agree where both resolve
        from onnxruntime_b200.tools.shape_inference import infer_shapes as traced_shapes
        tm = traced_shapes(m, {"batch": 2, "seq": 8})
        traced = {v.name: v.shape for v in list(tm.graph.value_info) + list(tm.graph.outputs)}
        sub = {"batch": 2, "seq": 8}
        checked = 0
        for name, shape in traced.items():
            if name not in vi or vi[name][1] is None or shape is None:
                continue
            want = [sub.get(d, d) for d in vi[name][1]]
            got = [sub.get(d, d) for d in shape]
            if all(isinstance(d, int) for d in want) and all(isinstance(d, int) for d in got):
                assert want == got, (name, vi[name], shape)
                checked += 1
        assert checked >= min(20, rep["nodes"] // 2), (checked, rep)


def test_contrib_operator_shapes_and_schema_violations():
    g = [ol.make_node("GroupQueryAttention", ["qkv", "", "", "pk", "pv", "sl", "tl"], ["o", "k2", "v2"], domain="com.microsoft", num_heads=8, kv_num_heads=2),
         ol.make_node("MatMulNBits", ["o", "B", "sc"], ["m"], domain="com.microsoft", K=512, N=96, bits=4, block_size=32),
         ol.make_node("SkipSimplifiedLayerNormalization", ["m", "skip", "gamma"], ["n", "", "", "sum"], domain="com.microsoft")]
    ins = [ol.make_tensor_value_info("qkv", T.FLOAT16, ["b", "s", 768]), ol.make_tensor_value_info("pk", T.FLOAT16, ["b", 2, "p", 64]),
           ol.make_tensor_value_info("pv", T.FLOAT16, ["b", 2, "p", 64]), ol.make_tensor_value_info("sl", T.INT32, ["b"]),
           ol.make_tensor_value_info("tl", T.INT32, []), ol.make_tensor_value_info("skip", T.FLOAT16, ["b", "s", 96])]
    inits = [ol.make_tensor("B", np.zeros((96, 16, 16), np.uint8)), ol.make_tensor("sc", np.zeros((96, 16), np.float16)),
             ol.make_tensor("gamma", np.ones(96, np.float16))]
    model = graph_model(g, ins, [ol.make_tensor_value_info("n", T.FLOAT16, None), ol.make_tensor_value_info("sum", T.FLOAT16, None)], inits)
    out, rep = C.infer_shapes(model)
    vi = _value_info(out)
    assert vi["o"][1] == ["b", "s", 512] and vi["m"][1] == ["b", "s", 96] and vi["n"][1] == ["b", "s", 96] and vi["sum"][1] == ["b", "s", 96]
    assert vi["k2"][1][:2] == ["b", 2] and vi["k2"][1][3] == 64
    # a MatMul with one input violates its schema: reported, and an error in strict mode
    bad = graph_model([ol.make_node("MatMul", ["x"], ["y"])], [ol.make_tensor_value_info("x", T.FLOAT, [2, 2])], [ol.make_tensor_value_info("y", T.FLOAT, None)])
    _, rep = C.infer_shapes(bad)
    assert len(rep["problems"]) == 1 and "MatMul" in rep["problems"][0]
    with pytest.raises(Exception):
        C.infer_shapes(bad, True)
    names = {(s["domain"], s["op_type"]) for s in C.op_schemas()}
    assert ("com.microsoft", "GroupQueryAttention") in names and ("", "Reshape") in names and len(names) > 150
