"""Offline tools: model loader, MatMulNBits quantizer, float16 converter, optimizer front end, perf_test and
onnx_test_runner command lines."""
import json
import os

import numpy as np
import pytest

import onnxruntime_b200 as ort
from onnxruntime_b200 import _core as C
from onnxruntime_b200 import onnx_lite as ol

T = ol.TensorProto


def _mlp_model(K=64, N=48, dtype=np.float32):
    rng = np.random.RandomState(0)
    w1 = rng.randn(K, N).astype(dtype) * 0.2
    w2 = rng.randn(N, K).astype(dtype) * 0.2
    b = rng.randn(N).astype(dtype) * 0.1
    nodes = [ol.make_node("MatMul", ["x", "w1"], ["h0"], name="fc1"), ol.make_node("Add", ["h0", "b"], ["h1"], name="bias"),
             ol.make_node("Relu", ["h1"], ["h2"], name="act"), ol.make_node("MatMul", ["h2", "w2"], ["y"], name="fc2")]
    et = ol.np_dtype_to_onnx(dtype)
    g = ol.make_graph(nodes, "mlp", [ol.make_tensor_value_info("x", et, ["batch", K])], [ol.make_tensor_value_info("y", et, ["batch", K])],
                      [ol.make_tensor("w1", w1), ol.make_tensor("w2", w2), ol.make_tensor("b", b)])
    return ol.make_model(g).serialize(), (w1, w2, b)


def test_load_model_round_trip_keeps_every_field():
    mb, _ = _mlp_model()
    m = ol.load_model(mb)
    assert [n.op_type for n in m.graph.nodes] == ["MatMul", "Add", "Relu", "MatMul"]
    assert m.graph.inputs[0].shape == ["batch", 64] and m.opset_imports[""] == 17
    assert C.model_nodes(m.serialize()) == C.model_nodes(mb)
    # typed (non-raw) tensor fields are read too: float_data / int64_data as another writer would emit them
    raw = ol._packed_varints(1, [3]) + ol._f_varint(2, T.INT64) + ol._f_str(8, "v") + ol._packed_varints(7, [5, -2, 9])
    t = ol.load_tensor(raw)
    np.testing.assert_array_equal(ol.to_array(t), np.array([5, -2, 9], dtype=np.int64))


@pytest.mark.parametrize("symmetric", [True, False])
@pytest.mark.parametrize("bits", [4, 8])
def test_matmul_nbits_quantizer(symmetric, bits):
    from onnxruntime_b200.quantization import MatMulNBitsQuantizer, dequantize_blockwise, quantize_blockwise
    mb, (w1, w2, b) = _mlp_model()
    q = MatMulNBitsQuantizer(mb, block_size=16, is_symmetric=symmetric, bits=bits, nodes_to_exclude=["fc2"])
    qm = q.process().serialize()
    ops = [n["op_type"] for n in C.model_nodes(qm)]
    assert ops == ["MatMulNBits", "Add", "Relu", "MatMul"] and q.quantized_nodes == ["fc1"]
    packed, scales, zp = quantize_blockwise(w1, 16, bits, symmetric)
    wq = dequantize_blockwise(packed, scales, zp, 64, bits, 16).T
    step = np.abs(w1).max() / (7 if bits == 4 else 127)
    assert np.abs(wq - w1).max() <= step * 0.75
    x = np.random.RandomState(1).randn(5, 64).astype(np.float32)
    y = ort.InferenceSession(qm, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    ref = np.maximum(x @ wq + b, 0) @ w2
    np.testing.assert_allclose(y, ref, rtol=1e-4, atol=1e-4)


def test_float16_conversion_keep_io_types_and_block_list():
    from onnxruntime_b200.transformers import convert_float_to_float16
    mb, (w1, w2, b) = _mlp_model()
    x = np.random.RandomState(1).randn(3, 64).astype(np.float32)
    ref = ort.InferenceSession(mb, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    m16 = convert_float_to_float16(mb, keep_io_types=True).serialize()
    s = ort.InferenceSession(m16, providers=["CPUExecutionProvider"])
    assert s.get_inputs()[0].type == "tensor(float)" and s.get_outputs()[0].type == "tensor(float)"
    assert all(t.data_type == T.FLOAT16 for t in ol.load_model(m16).graph.initializers)
    np.testing.assert_allclose(s.run(None, {"x": x})[0], ref, rtol=2e-2, atol=2e-2)
    m16b = convert_float_to_float16(mb, keep_io_types=False).serialize()
    s2 = ort.InferenceSession(m16b, providers=["CPUExecutionProvider"])
    assert s2.get_inputs()[0].type == "tensor(float16)"
    np.testing.assert_allclose(s2.run(None, {"x": x.astype(np.float16)})[0].astype(np.float32), ref, rtol=3e-2, atol=3e-2)
    # a blocked op keeps float32 and is wrapped in casts
    m16c = convert_float_to_float16(mb, keep_io_types=True, op_block_list=["Relu"]).serialize()
    ops = [n["op_type"] for n in C.model_nodes(m16c)]
    assert ops.count("Cast") >= 2
    np.testing.assert_allclose(ort.InferenceSession(m16c, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0], ref, rtol=2e-2, atol=2e-2)


def test_optimizer_front_end_fuses_bert(tmp_path):
    from onnxruntime_b200.models.bert import BertConfig, build_bert
    from onnxruntime_b200.transformers import optimize_model
    from onnxruntime_b200.transformers import optimizer as opt_cli
    mb = build_bert(BertConfig.tiny())
    m = optimize_model(mb, model_type="bert")
    stats = m.get_fused_operator_statistics()
    assert stats.get("Attention", 0) > 0 and stats.get("SkipLayerNormalization", 0) > 0 and m.is_fully_optimized()
    src, dst = tmp_path / "bert.onnx", tmp_path / "bert_opt.onnx"
    src.write_bytes(mb)
    assert opt_cli.main(["--input", str(src), "--output", str(dst)]) == 0
    assert "Attention" in {n["op_type"] for n in C.model_nodes(dst.read_bytes())}
    none = optimize_model(mb, opt_level=0)
    assert none.get_fused_operator_statistics().get("Attention", 0) == 0


def test_perf_test_cli(tmp_path, capsys):
    from onnxruntime_b200.tools import perf_test
    mb, _ = _mlp_model()
    path = tmp_path / "m.onnx"
    path.write_bytes(mb)
    out = tmp_path / "res.json"
    assert perf_test.main(["-e", "cpu", "-m", "times", "-r", "20", "-c", "2", "-f", "batch:4", "-I", str(path), str(out)]) == 0
    res = json.loads(out.read_text())
    assert res["runs"] == 20 and res["p50_ms"] <= res["p99_ms"] <= res["max_ms"] and res["inferences_per_s"] > 0
    text = capsys.readouterr().out
    assert "P50 Latency" in text and "P999 Latency" in text
    assert perf_test.main(["-m", "duration", "-t", "0.2", "-I", str(path)]) == 0


def test_onnx_test_runner(tmp_path):
    from onnxruntime_b200.tools import onnx_test_runner
    mb, (w1, w2, b) = _mlp_model()
    case = tmp_path / "test_mlp"
    ds = case / "test_data_set_0"
    os.makedirs(ds)
    (case / "model.onnx").write_bytes(mb)
    x = np.random.RandomState(2).randn(2, 64).astype(np.float32)
    y = np.maximum(x @ w1 + b, 0) @ w2
    (ds / "input_0.pb").write_bytes(ol.make_tensor("x", x).serialize())
    (ds / "output_0.pb").write_bytes(ol.make_tensor("y", y).serialize())
    assert onnx_test_runner.main([str(tmp_path)]) == 0
    (ds / "output_0.pb").write_bytes(ol.make_tensor("y", y + 1).serialize())
    assert onnx_test_runner.main([str(tmp_path)]) == 1


def _two_layer_mlp():
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    rng = np.random.default_rng(0)
    w1, w2 = rng.standard_normal((16, 32)).astype(np.float32) * 0.3, rng.standard_normal((32, 8)).astype(np.float32) * 0.3
    g = ol.make_graph([ol.make_node("MatMul", ["x", "w1"], ["h"], name="fc1"), ol.make_node("Relu", ["h"], ["r"]),
                       ol.make_node("MatMul", ["r", "w2"], ["y"], name="fc2")], "mlp",
                      [ol.make_tensor_value_info("x", T.FLOAT, ["n", 16])], [ol.make_tensor_value_info("y", T.FLOAT, ["n", 8])],
                      [ol.make_tensor("w1", w1), ol.make_tensor("w2", w2)])
    return ol.make_model(g, opset=17).serialize(), rng


def test_quantize_dynamic_and_static_keep_the_model_close_to_float():
    """quantize_dynamic -> DynamicQuantizeMatMul; quantize_static -> QDQ pairs from calibrated ranges
    (reference: onnxruntime/python/tools/quantization/quantize.py)."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.quantization import quantize_dynamic, quantize_static
    model, rng = _two_layer_mlp()
    x = rng.standard_normal((12, 16)).astype(np.float32)
    (ref,) = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    for per_channel in (False, True):
        qd = quantize_dynamic(model, per_channel=per_channel, nodes_to_exclude=["fc2"])
        ops = [n.op_type for n in qd.graph.nodes]
        assert ops == ["DynamicQuantizeMatMul", "Relu", "MatMul"]
        qd = quantize_dynamic(model, per_channel=per_channel)
        assert [n.op_type for n in qd.graph.nodes] == ["DynamicQuantizeMatMul", "Relu", "DynamicQuantizeMatMul"]
        assert all(ol.to_array(t).dtype == np.int8 for t in qd.graph.initializers if t.name.endswith("_quantized"))
        (y,) = ort.InferenceSession(qd.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x})
        assert np.abs(y - ref).max() < 0.05 * np.abs(ref).max()
        calib = [{"x": rng.standard_normal((12, 16)).astype(np.float32)} for _ in range(4)] + [{"x": x}]
        qs = quantize_static(model, calib, per_channel=per_channel)
        ops = [n.op_type for n in qs.graph.nodes]
        assert ops.count("QuantizeLinear") == 2 and ops.count("DequantizeLinear") == 4 and ops.count("MatMul") == 2
        (y,) = ort.InferenceSession(qs.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x})
        assert np.abs(y - ref).max() < 0.05 * np.abs(ref).max()


def test_shape_inference_by_tracing_names_symbolic_dimensions():
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.tools.shape_inference import infer_shapes
    T = ol.TensorProto
    w = np.zeros((16, 4), np.float32)
    nodes = [ol.make_node("MatMul", ["x", "w"], ["h"]),                      # [batch, seq, 4]
             ol.make_node("Shape", ["h"], ["shp"]),                           # [3]
             ol.make_node("Transpose", ["h"], ["t"], perm=[0, 2, 1]),         # [batch, 4, seq]
             ol.make_node("ReduceSum", ["t"], ["r"], keepdims=0),             # scalar (all axes)
             ol.make_node("Concat", ["h", "h"], ["c"], axis=1)]               # [batch, 2 * seq, 4]: a new symbol
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, ["batch", "seq", 16])],
                      [ol.make_tensor_value_info("c", T.FLOAT, None), ol.make_tensor_value_info("r", T.FLOAT, None)],
                      [ol.make_tensor("w", w)])
    m = infer_shapes(ol.make_model(g, opset=17).serialize())
    info = {v.name: (v.elem_type, list(v.shape)) for v in m.graph.value_info}
    assert info["h"] == (T.FLOAT, ["batch", "seq", 4])
    assert info["shp"] == (T.INT64, [3])
    assert info["t"] == (T.FLOAT, ["batch", 4, "seq"])
    out = {v.name: v for v in m.graph.outputs}
    assert list(out["r"].shape) == [] and out["c"].shape[0] == "batch" and out["c"].shape[2] == 4
    assert isinstance(out["c"].shape[1], str) and out["c"].shape[1].startswith("unk__")
    # the annotated model still loads and runs
    import onnxruntime_b200 as ort
    sess = ort.InferenceSession(m.serialize(), providers=["CPUExecutionProvider"])
    assert sess.run(None, {"x": np.ones((2, 3, 16), np.float32)})[0].shape == (2, 6, 4)


def test_ort_format_round_trip_and_conversion_tool(tmp_path):
    """ONNX -> ORT format (FlatBuffers, identifier ORTM) -> session: same results, also for control flow bodies;
    session.save_model_format / load_model_format and the conversion tool go through the same writer / reader."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol, ort_format
    from onnxruntime_b200.tools import convert_onnx_models_to_ort as tool
    T = ol.TensorProto
    rs = np.random.RandomState(9)
    then_g = ol.make_graph([ol.make_node("Mul", ["h", "two"], ["t_out"])], "then", [], [ol.make_tensor_value_info("t_out", T.FLOAT, None)],
                           [ol.make_tensor("two", np.array(2.0, np.float32))])
    else_g = ol.make_graph([ol.make_node("Neg", ["h"], ["e_out"])], "else", [], [ol.make_tensor_value_info("e_out", T.FLOAT, None)])
    nodes = [ol.make_node("Gemm", ["x", "w", "b"], ["h"], alpha=0.5, transB=1, name="gemm0"),
             ol.make_node("If", ["flag"], ["branch"], then_branch=then_g, else_branch=else_g),
             ol.make_node("Concat", ["h", "branch"], ["c"], axis=1),
             ol.make_node("Transpose", ["c"], ["y"], perm=[1, 0])]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 4]), ol.make_tensor_value_info("flag", T.BOOL, [])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [6, "n"])],
                      [ol.make_tensor("w", rs.randn(3, 4).astype(np.float32)), ol.make_tensor("b", rs.randn(3).astype(np.float32))])
    model = ol.make_model(g, opset=17, metadata={"origin": "unit test"})
    onnx_path = tmp_path / "m.onnx"
    onnx_path.write_bytes(model.serialize())
    buf = ort_format.onnx_to_ort(model)
    assert buf[4:8] == b"ORTM" and ort_format.is_ort_format(buf)
    back = ort_format.ort_to_onnx(buf)
    assert [n.op_type for n in back.graph.nodes] == ["Gemm", "If", "Concat", "Transpose"]
    assert back.opset_imports[""] == 17 and back.metadata == {"origin": "unit test"}
    assert [(v.name, v.elem_type, list(v.shape)) for v in back.graph.inputs] == [("x", T.FLOAT, ["n", 4]), ("flag", T.BOOL, [])]
    x = rs.randn(5, 4).astype(np.float32)
    ref = ort.InferenceSession(str(onnx_path), providers=["CPUExecutionProvider"])
    ort_path = tmp_path / "m.ort"
    ort_path.write_bytes(buf)
    for source in (str(ort_path), buf):
        sess = ort.InferenceSession(source, providers=["CPUExecutionProvider"])
        for flag in (True, False):
            feeds = {"x": x, "flag": np.array(flag)}
            np.testing.assert_allclose(sess.run(None, feeds)[0], ref.run(None, feeds)[0], rtol=1e-6, atol=1e-6)
        assert sess.get_modelmeta().custom_metadata_map == {"origin": "unit test"}
    out_dir = tmp_path / "converted"
    assert tool.main([str(onnx_path), "--output_dir", str(out_dir), "--optimization_level", "basic"]) == 0
    conv = ort.InferenceSession(str(out_dir / "m.ort"), providers=["CPUExecutionProvider"])
    feeds = {"x": x, "flag": np.array(True)}
    np.testing.assert_allclose(conv.run(None, feeds)[0], ref.run(None, feeds)[0], rtol=1e-6, atol=1e-6)
    with pytest.raises(Exception):
        ort.InferenceSession(buf[:60], providers=["CPUExecutionProvider"])


def test_entropy_and_percentile_calibration_and_bnb4_quantizer():
    """Histogram calibrators cut outliers that min-max keeps; NF4 / FP4 weights run through MatMulBnb4
    (reference: onnxruntime/python/tools/quantization/calibrate.py, matmul_bnb4_quantizer.py)."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.quantization import (CalibrationDataReader, CalibrationMethod, MatMulBnb4Quantizer, dequantize_bnb4, quantize_bnb4,
                                               quantize_static)
    model, rng = _two_layer_mlp()
    x = rng.standard_normal((64, 16)).astype(np.float32)
    (ref,) = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    spiky = x.copy()
    spiky[0, 0] = 400.0          # one outlier: min-max stretches the input range over it

    class Reader(CalibrationDataReader):
        def __init__(self):
            self.items = iter([{"x": spiky}, {"x": x}])

        def get_next(self):
            return next(self.items, None)

    errs = {}
    for method in (CalibrationMethod.MinMax, CalibrationMethod.Entropy, CalibrationMethod.Percentile):
        q = quantize_static(model, Reader(), calibrate_method=method, percentile=99.9)
        (y,) = ort.InferenceSession(q.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x})
        errs[method] = float(np.abs(y - ref).max() / np.abs(ref).max())
    assert errs[CalibrationMethod.Entropy] < errs[CalibrationMethod.MinMax] and errs[CalibrationMethod.Percentile] < errs[CalibrationMethod.MinMax]
    assert errs[CalibrationMethod.Entropy] < 0.1
    # NF4 round trip and the rewritten graph
    w = rng.standard_normal((16, 24)).astype(np.float32)
    for qt in (0, 1):
        packed, absmax = quantize_bnb4(w, qt, 32)
        back = dequantize_bnb4(packed, absmax, 16, 24, qt, 32)
        assert np.abs(back - w).max() < (0.2 if qt == 1 else 0.35) * np.abs(w).max()
    qm = MatMulBnb4Quantizer(model, quant_type=1, block_size=32, nodes_to_exclude=["fc2"]).process()
    assert [n.op_type for n in qm.graph.nodes] == ["MatMulBnb4", "Relu", "MatMul"]
    (y,) = ort.InferenceSession(qm.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x})
    assert np.abs(y - ref).max() < 0.25 * np.abs(ref).max()


def test_offline_tuning_profile_explorer_and_io_binding_helper(tmp_path, capsys):
    import json
    import numpy as np
    import torch
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.tools import offline_tuning, profile_explorer
    from onnxruntime_b200.transformers.io_binding_helper import CudaSession, IOBindingHelper, TypeHelper
    model, rng = _two_layer_mlp()
    path = tmp_path / "m.onnx"
    path.write_bytes(model)
    results = [{"ep": "CUDAExecutionProvider", "results": {"Gemm": {"8x16x16": 3}}, "validators": {"arch": "sm_100a"}}]
    (tmp_path / "t.json").write_text(json.dumps(results))
    assert offline_tuning.main(["embed", str(tmp_path / "tuned.onnx"), str(path), str(tmp_path / "t.json")]) == 0
    assert offline_tuning.extract(ol.load_model(str(tmp_path / "tuned.onnx"))) == results
    assert offline_tuning.main(["extract", str(tmp_path / "tuned.onnx"), str(tmp_path / "out.json")]) == 0
    assert json.loads((tmp_path / "out.json").read_text()) == results
    assert offline_tuning.main(["extract", str(path), str(tmp_path / "none.json")]) == 1
    # a profile of two runs -> per-operator table
    so = ort.SessionOptions()
    so.enable_profiling = True
    so.profile_file_prefix = str(tmp_path / "prof")
    sess = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    x = rng.standard_normal((4, 16)).astype(np.float32)
    sess.run(None, {"x": x})
    sess.run(None, {"x": x})
    prof = sess.end_profiling()
    rows = profile_explorer.summarise(profile_explorer.load_events(prof))
    by_op = {r[0]: r for r in rows}
    assert by_op["MatMul"][2] % 2 == 0 and by_op["MatMul"][2] >= 2 and abs(sum(r[5] for r in rows) - 100.0) < 1e-6
    assert profile_explorer.main([prof, "--csv", str(tmp_path / "p.csv"), "--top", "3"]) == 0
    assert "MatMul" in capsys.readouterr().out and (tmp_path / "p.csv").read_text().startswith("name,provider")
    # io binding helpers on the CPU device
    assert TypeHelper.get_input_type(sess, "x") == "tensor(float)" and TypeHelper.ort_type_to_torch_type("tensor(float16)") == torch.float16
    assert TypeHelper.numpy_type_to_torch_type(np.int64) == torch.int64 and TypeHelper.torch_type_to_numpy_type(torch.float32) == np.float32
    plain = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    out_name = plain.get_outputs()[0].name
    (ref,) = plain.run(None, {"x": x})
    bufs = IOBindingHelper.get_output_buffers(plain, {out_name: ref.shape}, "cpu")
    binding = IOBindingHelper.prepare_io_binding(plain, {"x": torch.from_numpy(x)}, bufs)
    plain.run_with_iobinding(binding)
    np.testing.assert_allclose(bufs[out_name].numpy(), ref, rtol=1e-6)
    cs = CudaSession(plain, torch.device("cpu"))
    cs.allocate_buffers({out_name: ref.shape})
    np.testing.assert_allclose(cs.infer({"x": torch.from_numpy(x)})[out_name].numpy(), ref, rtol=1e-6)


def test_symbolic_shape_inference_front_end(tmp_path):
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    from onnxruntime_b200.tools.symbolic_shape_infer import SymbolicShapeInference, main
    model, _ = _two_layer_mlp()
    out = SymbolicShapeInference.infer_shapes(model)
    shapes = {v.name: list(v.shape) for v in out.graph.value_info if v.shape is not None}
    assert any(len(s) == 2 for s in shapes.values()) and len(shapes) >= 2
    src, dst = tmp_path / "m.onnx", tmp_path / "s.onnx"
    src.write_bytes(model)
    assert main(["--input", str(src), "--output", str(dst)]) == 0
    assert len(ol.load_model(str(dst)).graph.value_info) >= len(shapes)


def test_quantize_static_qoperator_format():
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200.quantization import QuantFormat, quantize_static
    model, rng = _two_layer_mlp()
    x = rng.standard_normal((32, 16)).astype(np.float32)
    (ref,) = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    for per_channel in (False, True):
        q = quantize_static(model, [{"x": x}], quant_format=QuantFormat.QOperator, per_channel=per_channel)
        ops = [n.op_type for n in q.graph.nodes]
        assert ops.count("QLinearMatMul") == 2 and "MatMul" not in ops
        so = ort.SessionOptions()
        so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
        (y,) = ort.InferenceSession(q.serialize(), so, providers=["CPUExecutionProvider"]).run(None, {"x": x})
        assert np.abs(y - ref).max() < 0.06 * np.abs(ref).max()


def test_hqq_weight_quantization_beats_round_to_nearest_on_outliers():
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200.quantization import MatMulNBitsQuantizer, dequantize_blockwise, quantize_blockwise, quantize_blockwise_hqq
    rng = np.random.default_rng(0)
    w = rng.standard_normal((128, 24)).astype(np.float32)
    w[rng.integers(0, 128, 40), rng.integers(0, 24, 40)] *= 6.0        # outliers stretch the min-max range
    p0, s0, z0 = quantize_blockwise(w, 32, 4, symmetric=False)
    p1, s1, z1 = quantize_blockwise_hqq(w, 32, 4)
    e_rtn = np.abs(dequantize_blockwise(p0, s0, z0, 128, 4, 32).T - w).mean()
    e_hqq = np.abs(dequantize_blockwise(p1, s1, z1, 128, 4, 32).T - w).mean()
    assert z1.dtype == np.float32 and e_hqq <= e_rtn * 1.001
    model, mrng = _two_layer_mlp()
    x = mrng.standard_normal((6, 16)).astype(np.float32)
    (ref,) = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, {"x": x})
    q = MatMulNBitsQuantizer(model, block_size=16, algorithm="hqq").process()
    node = [n for n in q.graph.nodes if n.op_type == "MatMulNBits"][0]
    assert len(node.inputs) == 4                                        # float zero points ride along
    (y,) = ort.InferenceSession(q.serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x})
    assert np.abs(y - ref).max() < 0.15 * np.abs(ref).max()


def test_gptq_weight_quantization_keeps_the_layer_output_closer_than_round_to_nearest():
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200.quantization import MatMulNBitsQuantizer, dequantize_blockwise, quantize_blockwise, quantize_blockwise_gptq
    rng = np.random.default_rng(0)
    K, N = 128, 24
    w = rng.standard_normal((K, N)).astype(np.float32)
    mix = rng.standard_normal((K, K)) * (rng.random(K) ** 3)[None, :]            # correlated activations of uneven scale
    x = (rng.standard_normal((512, K)) @ mix).astype(np.float32)
    p0, s0, z0 = quantize_blockwise(w, 32, 4, symmetric=False)
    p1, s1, z1 = quantize_blockwise_gptq(w, x.T.astype(np.float64) @ x, 32, 4)
    assert p1.shape == p0.shape and s1.shape == s0.shape and z1.shape == z0.shape and z1.dtype == np.uint8
    e_rtn = np.linalg.norm(x @ dequantize_blockwise(p0, s0, z0, K, 4, 32).T - x @ w)
    e_gptq = np.linalg.norm(x @ dequantize_blockwise(p1, s1, z1, K, 4, 32).T - x @ w)
    assert e_gptq < 0.9 * e_rtn, (e_gptq, e_rtn)

    class Reader:
        def __init__(self, batches):
            self.it = iter(batches)

        def get_next(self):
            return next(self.it, None)
    model, mrng = _two_layer_mlp()
    batches = [{"x": mrng.standard_normal((32, 16)).astype(np.float32)} for _ in range(4)]
    (ref,) = ort.InferenceSession(model, providers=["CPUExecutionProvider"]).run(None, batches[0])
    q = MatMulNBitsQuantizer(model, block_size=16, algorithm="gptq", calibration_data_reader=Reader(batches)).process()
    assert sum(n.op_type == "MatMulNBits" for n in q.graph.nodes) == 2
    (y,) = ort.InferenceSession(q.serialize(), providers=["CPUExecutionProvider"]).run(None, batches[0])
    assert np.abs(y - ref).max() < 0.15 * np.abs(ref).max()
