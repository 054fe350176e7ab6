"""Python API contract: InferenceSession / SessionOptions / RunOptions / IOBinding / OrtValue."""
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol
from helpers import graph_model

T = ol.TensorProto


def _model(dynamic=True):
    w = np.arange(12, dtype=np.float32).reshape(4, 3)
    return graph_model([ol.make_node("MatMul", ["x", "w"], ["y0"]), ol.make_node("Relu", ["y0"], ["y"]),
                        ol.make_node("ReduceSum", ["y0"], ["s"], keepdims=0)],
                       [ol.make_tensor_value_info("x", T.FLOAT, ["batch" if dynamic else 2, 4])],
                       [ol.make_tensor_value_info("y", T.FLOAT, ["batch" if dynamic else 2, 3]), ol.make_tensor_value_info("s", T.FLOAT, [])],
                       [ol.make_tensor("w", w)], opset=12), w


def test_run_and_metadata():
    m, w = _model()
    s = ort.InferenceSession(m, providers=["CPUExecutionProvider"])
    assert [i.name for i in s.get_inputs()] == ["x"]
    assert [o.name for o in s.get_outputs()] == ["y", "s"]
    assert s.get_inputs()[0].type == "tensor(float)" and s.get_inputs()[0].shape == ["batch", 4]
    assert s.get_providers() == ["CPUExecutionProvider"]
    assert "CPUExecutionProvider" in s.get_provider_options()
    x = np.random.RandomState(0).randn(5, 4).astype(np.float32)
    y, total = s.run(None, {"x": x})
    np.testing.assert_allclose(y, np.maximum(x @ w, 0), rtol=1e-5, atol=1e-5)
    only = s.run(["s"], {"x": x})
    assert len(only) == 1 and only[0] == pytest.approx((x @ w).sum(), rel=1e-4)
    vals = s.run_with_ort_values(["y"], {"x": ort.OrtValue.ortvalue_from_numpy(x)})
    assert isinstance(vals[0], ort.OrtValue) and vals[0].shape() == [5, 3] and vals[0].data_type() == "tensor(float)"
    assert vals[0].device_name() == "cpu"


def test_input_validation_errors():
    m, _ = _model(dynamic=False)
    s = ort.InferenceSession(m, providers=["CPUExecutionProvider"])
    with pytest.raises(ValueError):
        s.run(None, {})
    with pytest.raises(ort.InvalidArgument, match="Unexpected input data type"):
        s.run(None, {"x": np.zeros((2, 4), np.float64)})
    with pytest.raises(ort.InvalidArgument, match="Invalid rank"):
        s.run(None, {"x": np.zeros((2, 4, 1), np.float32)})
    with pytest.raises(ort.InvalidArgument, match="invalid dimensions"):
        s.run(None, {"x": np.zeros((3, 4), np.float32)})
    with pytest.raises(ort.InvalidArgument, match="Invalid output name"):
        s.run(["nope"], {"x": np.zeros((2, 4), np.float32)})
    with pytest.raises(ort.InvalidArgument):
        s.run(None, {"x": np.zeros((2, 4), np.float32), "zzz": np.zeros(1, np.float32)})


def test_load_errors_and_providers(tmp_path):
    with pytest.raises(ort.NoSuchFile):
        ort.InferenceSession(str(tmp_path / "missing.onnx"), providers=["CPUExecutionProvider"])
    m, _ = _model()
    with pytest.raises(ValueError):
        ort.InferenceSession(m, providers=["NoSuchExecutionProvider"])
    with pytest.raises(ValueError):
        ort.InferenceSession(m, providers="CPUExecutionProvider")
    assert ort.get_all_providers()[-1] == "CPUExecutionProvider"
    assert "CPUExecutionProvider" in ort.get_available_providers()
    assert ort.get_device() in ("CPU", "GPU")
    # requesting the GPU provider on a machine without one falls back to the CPU provider
    if not torch.cuda.is_available():
        s = ort.InferenceSession(m, providers=["CUDAExecutionProvider", "CPUExecutionProvider"])
        assert s.get_providers() == ["CPUExecutionProvider"]
    bad = graph_model([ol.make_node("NoSuchOp", ["x"], ["y"])], [ol.make_tensor_value_info("x", T.FLOAT, [1])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [1])])
    with pytest.raises(ort.NotImplemented, match="NoSuchOp"):
        ort.InferenceSession(bad, providers=["CPUExecutionProvider"])
    cyc = graph_model([ol.make_node("Relu", ["b"], ["a"]), ol.make_node("Relu", ["a"], ["b"])], [], [ol.make_tensor_value_info("b", T.FLOAT, [1])])
    with pytest.raises(ort.InvalidGraph):
        ort.InferenceSession(cyc, providers=["CPUExecutionProvider"])


def test_session_options_and_config_entries(tmp_path):
    so = ort.SessionOptions()
    assert so.graph_optimization_level == ort.GraphOptimizationLevel.ORT_ENABLE_ALL
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_ENABLE_BASIC
    assert so.graph_optimization_level == ort.GraphOptimizationLevel.ORT_ENABLE_BASIC
    so.execution_mode = ort.ExecutionMode.ORT_PARALLEL
    assert so.execution_mode == ort.ExecutionMode.ORT_PARALLEL
    so.intra_op_num_threads = 2
    so.log_severity_level = 3
    assert so.intra_op_num_threads == 2 and so.log_severity_level == 3
    so.add_session_config_entry("session.disable_prepacking", "1")
    assert so.get_session_config_entry("session.disable_prepacking") == "1"
    with pytest.raises(ort.RuntimeException):
        so.get_session_config_entry("missing.key")
    with pytest.raises(AttributeError):
        so.no_such_option = 1
    so.optimized_model_filepath = str(tmp_path / "opt.onnx")
    m, w = _model()
    s = ort.InferenceSession(m, so, providers=["CPUExecutionProvider"])
    assert os.path.exists(so.optimized_model_filepath)
    s2 = ort.InferenceSession(so.optimized_model_filepath, providers=["CPUExecutionProvider"])
    x = np.ones((1, 4), np.float32)
    np.testing.assert_allclose(s.run(["y"], {"x": x})[0], s2.run(["y"], {"x": x})[0])
    ro = ort.RunOptions()
    ro.add_run_config_entry("gpu_graph_id", "3")
    assert ro.get_run_config_entry("gpu_graph_id") == "3"
    ro.terminate = True
    with pytest.raises(ort.Fail, match="terminate"):
        s.run(None, {"x": x}, ro)


def test_free_dimension_override_and_add_initializer():
    m, w = _model()
    so = ort.SessionOptions()
    so.add_free_dimension_override_by_name("batch", 2)
    s = ort.InferenceSession(m, so, providers=["CPUExecutionProvider"])
    assert s.get_inputs()[0].shape == [2, 4]
    with pytest.raises(ort.InvalidArgument):
        s.run(None, {"x": np.zeros((3, 4), np.float32)})
    so2 = ort.SessionOptions()
    so2.add_initializer("w", ort.OrtValue.ortvalue_from_numpy(np.ones((4, 3), np.float32)))
    s2 = ort.InferenceSession(m, so2, providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(s2.run(["y"], {"x": np.ones((1, 4), np.float32)})[0], np.full((1, 3), 4.0))


def test_overridable_initializer():
    g = graph_model([ol.make_node("Add", ["x", "b"], ["y"])],
                    [ol.make_tensor_value_info("x", T.FLOAT, [2]), ol.make_tensor_value_info("b", T.FLOAT, [2])],
                    [ol.make_tensor_value_info("y", T.FLOAT, [2])], [ol.make_tensor("b", np.array([1, 2], np.float32))])
    s = ort.InferenceSession(g, providers=["CPUExecutionProvider"])
    assert [i.name for i in s.get_inputs()] == ["x"]
    assert [i.name for i in s.get_overridable_initializers()] == ["b"]
    x = np.zeros(2, np.float32)
    np.testing.assert_array_equal(s.run(None, {"x": x})[0], [1, 2])
    np.testing.assert_array_equal(s.run(None, {"x": x, "b": np.array([5, 5], np.float32)})[0], [5, 5])


def test_iobinding_cpu():
    m, w = _model()
    s = ort.InferenceSession(m, providers=["CPUExecutionProvider"])
    x = np.random.RandomState(1).randn(3, 4).astype(np.float32)
    b = s.io_binding()
    b.bind_cpu_input("x", x)
    b.bind_output("y")
    out_s = ort.OrtValue.ortvalue_from_shape_and_type([], np.float32)
    b.bind_ortvalue_output("s", out_s)
    b.synchronize_inputs()
    s.run_with_iobinding(b)
    b.synchronize_outputs()
    outs = b.copy_outputs_to_cpu()
    np.testing.assert_allclose(outs[0], np.maximum(x @ w, 0), rtol=1e-5, atol=1e-5)
    assert out_s.numpy() == pytest.approx((x @ w).sum(), rel=1e-4)
    # bind by raw pointer
    buf = np.zeros((3, 3), np.float32)
    b2 = s.io_binding()
    b2.bind_input("x", "cpu", 0, np.float32, x.shape, x.ctypes.data)
    b2.bind_output("y", "cpu", 0, np.float32, buf.shape, buf.ctypes.data)
    s.run_with_iobinding(b2)
    np.testing.assert_allclose(buf, np.maximum(x @ w, 0), rtol=1e-5, atol=1e-5)
    with pytest.raises(ort.InvalidArgument):
        b2.bind_cpu_input("nope", x)
    b2.clear_binding_inputs()
    b2.clear_binding_outputs()


def test_ortvalue():
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    v = ort.OrtValue.ortvalue_from_numpy(a)
    assert v.shape() == [2, 3] and v.is_tensor() and v.has_value() and v.element_type() == 1
    np.testing.assert_array_equal(v.numpy(), a)
    doubled = a * 2
    v.update_inplace(doubled)  # the OrtValue shares memory with `a`
    np.testing.assert_array_equal(v.numpy(), doubled)
    back = ort.OrtValue.from_dlpack(v.to_dlpack())
    np.testing.assert_array_equal(back.numpy(), doubled)
    z = ort.OrtValue.ortvalue_from_shape_and_type([4], np.int64)
    assert z.data_type() == "tensor(int64)" and z.data_ptr() != 0


def test_profiling(tmp_path):
    m, _ = _model()
    so = ort.SessionOptions()
    so.enable_profiling = True
    so.profile_file_prefix = str(tmp_path / "prof")
    s = ort.InferenceSession(m, so, providers=["CPUExecutionProvider"])
    s.run(None, {"x": np.ones((1, 4), np.float32)})
    path = s.end_profiling()
    assert path.startswith(str(tmp_path / "prof")) and path.endswith(".json")
    events = json.load(open(path))
    names = [e["name"] for e in events]
    assert "model_run" in names and "session_initialization" in names
    assert all({"cat", "pid", "tid", "dur", "ts", "ph", "name", "args"} <= set(e) for e in events)
    node_events = [e for e in events if e["cat"] == "Node"]
    assert any(e["name"].endswith("_kernel_time") and e["args"].get("op_name") == "MatMul" for e in node_events)


def test_run_async_and_disabled_optimizers():
    import threading
    m, w = _model()
    s = ort.InferenceSession(m, providers=["CPUExecutionProvider"], disabled_optimizers=["ConstantFolding"])
    done = threading.Event()
    box = {}

    def cb(res, user, err):
        box["res"], box["user"], box["err"] = res, user, err
        done.set()
    s.run_async(None, {"x": np.ones((1, 4), np.float32)}, cb, "tag")
    assert done.wait(10) and box["user"] == "tag" and box["err"] == ""
    np.testing.assert_allclose(box["res"][0], np.maximum(np.ones((1, 4), np.float32) @ w, 0))


def test_logging_severity_sink_and_session_ids(capfd):
    """Per-session logger id and threshold, process default, replaceable sink (the reference's LoggingManager:
    onnxruntime/core/common/logging/logging.h; python: set_default_logger_severity, SessionOptions.logid)."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    g = ol.make_graph([ol.make_node("Relu", ["x"], ["y"])], "g", [ol.make_tensor_value_info("x", T.FLOAT, [2])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [2])])
    model = ol.make_model(g, opset=17).serialize()
    lines = []
    ort.set_log_sink(lambda sev, logid, line: lines.append((sev, logid, line)))
    try:
        so = ort.SessionOptions()
        so.logid = "quiet"
        ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
        assert lines == []                      # default threshold is WARNING
        so = ort.SessionOptions()
        so.logid = "chatty"
        so.log_severity_level = 1
        sess = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
        assert any(sev == 1 and logid == "chatty" and "session initialized" in line for sev, logid, line in lines)
        assert all(logid == "chatty" for _, logid, _ in lines)
        n = len(lines)
        ro = ort.RunOptions()
        ro.logid = "run7"
        ro.log_severity_level = 0
        ro.log_verbosity_level = 1
        sess.run(None, {"x": np.zeros(2, np.float32)}, ro)
        assert any(sev == 0 and logid == "run7" for sev, logid, _ in lines[n:])
    finally:
        ort.set_log_sink(None)
    # without a sink lines go to stderr in the "[I:ortb200:<id>, file:line function] message" form
    so = ort.SessionOptions()
    so.logid = "stderr-session"
    so.log_severity_level = 1
    ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    err = capfd.readouterr().err
    assert "[I:ortb200:stderr-session, session.cc:" in err


def _wide_model(branches=6, depth=4, n=64):
    """`branches` independent chains of MatMul + Tanh over one input, summed at the end: work an inter-op pool can spread."""
    import numpy as np
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    rng = np.random.RandomState(3)
    nodes, inits, tails = [], [], []
    for b in range(branches):
        cur = "x"
        for d in range(depth):
            w = f"w{b}_{d}"
            inits.append(ol.make_tensor(w, (rng.randn(n, n) * 0.2).astype(np.float32)))
            nodes += [ol.make_node("MatMul", [cur, w], [f"m{b}_{d}"]), ol.make_node("Tanh", [f"m{b}_{d}"], [f"t{b}_{d}"])]
            cur = f"t{b}_{d}"
        tails.append(cur)
    nodes.append(ol.make_node("Sum", tails, ["y"]))
    g = ol.make_graph(nodes, "wide", [ol.make_tensor_value_info("x", T.FLOAT, ["b", n])], [ol.make_tensor_value_info("y", T.FLOAT, None)], inits)
    return ol.make_model(g, opset=17).serialize()


def test_parallel_execution_mode_matches_sequential():
    """ExecutionMode.ORT_PARALLEL runs independent nodes on the inter-op pool; results equal the sequential run, errors
    surface as the usual exception, control-flow nodes keep their place."""
    import numpy as np
    import onnxruntime_b200 as ort
    model = _wide_model()
    x = np.random.RandomState(0).randn(5, 64).astype(np.float32)
    so0 = ort.SessionOptions()
    so0.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    ref = ort.InferenceSession(model, so0, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    so.execution_mode = ort.ExecutionMode.ORT_PARALLEL
    so.inter_op_num_threads = 4
    so.intra_op_num_threads = 1
    sess = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    for _ in range(5):
        np.testing.assert_array_equal(sess.run(None, {"x": x})[0], ref)
    # a failing node surfaces as the same kind of exception as in the sequential executor
    with pytest.raises(ort.capi.OrtException):
        sess.run(None, {"x": np.zeros((5, 63), np.float32)})
    np.testing.assert_array_equal(sess.run(None, {"x": x})[0], ref)   # and the session stays usable


def test_ignored_options_are_reported_and_mapped_ones_applied():
    import numpy as np
    import torch
    import onnxruntime_b200 as ort
    model = _wide_model(2, 1, 8)
    lines = []
    ort.set_log_sink(lambda sev, logid, line: lines.append((sev, line)))
    before = torch.get_num_threads()
    try:
        so = ort.SessionOptions()
        so.enable_mem_reuse = False
        so.inter_op_num_threads = 3
        so.intra_op_num_threads = 2
        so.add_session_config_entry("session.no_such_key", "1")
        so.add_session_config_entry("session.disable_prepacking", "1")
        ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
        text = "\\n".join(l for _, l in lines)
        assert "enable_mem_reuse" in text and "inter_op_num_threads is only used" in text
        assert "session.no_such_key" in text and "session.disable_prepacking" not in text
        assert torch.get_num_threads() == 2
    finally:
        ort.set_log_sink(None)
        torch.set_num_threads(before)


def test_memory_plan_reuses_buffers_of_dead_values():
    """A chain of elementwise nodes needs two live buffers at a time, not one per node: the plan traced on the first
    run packs the values accordingly and never lets two live values overlap."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    nodes, prev = [], "x"
    for i in range(8):
        nodes.append(ol.make_node("Relu" if i % 2 else "Neg", [prev], [f"v{i}"]))
        prev = f"v{i}"
    nodes.append(ol.make_node("Reshape", [prev, "shape"], ["flat"]))       # a view: allocates nothing
    nodes.append(ol.make_node("Add", ["flat", "flat"], ["y"]))
    g = ol.make_graph(nodes, "chain", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 256])], [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_tensor("shape", np.array([-1], np.int64))])
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), so, providers=["CPUExecutionProvider"])
    assert sess.get_memory_plans() == []
    sess.run(None, {"x": np.ones((4, 256), np.float32)})
    sess.run(None, {"x": np.ones((4, 256), np.float32)})          # same pattern: no second plan
    sess.run(None, {"x": np.ones((8, 256), np.float32)})
    plans = sess.get_memory_plans()
    assert len(plans) == 2 and all(p["valid"] for p in plans)
    p = next(p for p in plans if "[4, 256]" in p["pattern"])
    one = 4 * 256 * 4
    assert p["host_total_bytes"] == 9 * one                        # 8 chain values + y; the reshape is a view
    assert p["host_live_peak_bytes"] == 2 * one
    assert p["host_peak_bytes"] <= 3 * one and p["host_values_reusing_memory"] >= 6
    by_name = {b[0]: b for b in p["buffers"]}
    assert by_name["flat"][1] == 0 and by_name["flat"][5] == -1
    assert sess.get_memory_stats() == {}


def test_compiled_model_round_trip_through_an_ep_context_node(tmp_path):
    """ModelCompiler / ep.context_enable store the prepared graph in one EPContext node; loading that model gives the
    same results and runs no optimizer pass again."""
    import numpy as np
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from helpers import op_counts
    T = ol.TensorProto
    rs = np.random.RandomState(3)
    nodes = [ol.make_node("MatMul", ["x", "w"], ["m"]), ol.make_node("Add", ["m", "b"], ["a"]),
             ol.make_node("Mul", ["a", "half"], ["h"]), ol.make_node("Div", ["a", "sqrt2"], ["d"]), ol.make_node("Erf", ["d"], ["e"]),
             ol.make_node("Add", ["e", "one"], ["p"]), ol.make_node("Mul", ["h", "p"], ["y"])]
    inits = [ol.make_tensor("w", rs.randn(8, 8).astype(np.float32)), ol.make_tensor("b", rs.randn(8).astype(np.float32)),
             ol.make_tensor("half", np.array(0.5, np.float32)), ol.make_tensor("sqrt2", np.array(np.sqrt(2.0), np.float32)),
             ol.make_tensor("one", np.array(1.0, np.float32))]
    g = ol.make_graph(nodes, "gelu_mlp", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 8])], [ol.make_tensor_value_info("y", T.FLOAT, ["n", 8])], inits)
    src = tmp_path / "model.onnx"
    src.write_bytes(ol.make_model(g, opset=17, metadata={"k": "v"}).serialize())
    x = rs.randn(3, 8).astype(np.float32)
    want = ort.InferenceSession(str(src), providers=["CPUExecutionProvider"]).run(None, {"x": x})[0]

    embedded = tmp_path / "embedded_ctx.onnx"
    ort.ModelCompiler(None, str(src), embed_compiled_data_into_model=True, providers=["CPUExecutionProvider"]).compile_to_file(str(embedded))
    side = tmp_path / "side_ctx.onnx"
    ort.ModelCompiler(None, str(src), embed_compiled_data_into_model=False, providers=["CPUExecutionProvider"]).compile_to_file(str(side))
    assert (tmp_path / "side_ctx_ortb200.bin").exists() and side.stat().st_size < embedded.stat().st_size
    for path in (embedded, side):
        outer = ol.load(str(path)) if hasattr(ol, "load") else None
        so = ort.SessionOptions()
        so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL    # the payload is already optimized
        sess = ort.InferenceSession(str(path), so, providers=["CPUExecutionProvider"])
        counts = op_counts(sess)
        assert "EPContext" not in counts and "Erf" not in counts and counts.get("Gelu", 0) + counts.get("BiasGelu", 0) == 1
        np.testing.assert_allclose(sess.run(None, {"x": x})[0], want, rtol=1e-6, atol=1e-6)
        assert sess.get_modelmeta().custom_metadata_map == {"k": "v"}
        assert [i.name for i in sess.get_inputs()] == ["x"] and sess.get_inputs()[0].shape == ["n", 8]
    blob = ort.ModelCompiler(None, src.read_bytes(), providers=["CPUExecutionProvider"]).compile_to_bytes()
    np.testing.assert_allclose(ort.InferenceSession(blob, providers=["CPUExecutionProvider"]).run(None, {"x": x})[0], want, rtol=1e-6, atol=1e-6)


def test_tuning_results_are_empty_on_cpu_and_imports_are_validated():
    import onnxruntime_b200 as ort
    sess = ort.InferenceSession(_wide_model(2, 1, 8), providers=["CPUExecutionProvider"])
    assert sess.get_tuning_results() == []
    good = [{"ep": "CUDAExecutionProvider", "validators": {"ORTB200_VERSION": "0.1.0", "DEVICE_ARCH": "sm_100a"},
             "results": {"Gemm": {"Gemm_BFloat16_in0_8_64_64_act0": "splits=2,bn=16,tile_rows=0"}}}]
    sess.set_tuning_results(good)
    assert sess.get_tuning_results()[0]["results"]["Gemm"] == good[0]["results"]["Gemm"]
    sess.set_tuning_results([{"ep": "ROCMExecutionProvider", "validators": {}, "results": {}}])      # skipped silently
    import pytest
    with pytest.raises(ort.capi.InvalidArgument):
        sess.set_tuning_results([{"ep": "ROCMExecutionProvider", "validators": {}, "results": {}}], error_on_invalid=True)


def test_debug_node_io_environment_variables(tmp_path):
    """ORT_DEBUG_NODE_IO_*: shapes, placement, statistics and output snippets of the selected nodes, to stdout or files."""
    import subprocess
    import sys
    script = r'''
import numpy as np, onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol
T = ol.TensorProto
g = ol.make_graph([ol.make_node("Relu", ["x"], ["r"], name="relu0"), ol.make_node("Log", ["r"], ["y"], name="log0")], "g",
                  [ol.make_tensor_value_info("x", T.FLOAT, [2, 3])], [ol.make_tensor_value_info("y", T.FLOAT, [2, 3])])
so = ort.SessionOptions(); so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
s = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), so, providers=["CPUExecutionProvider"])
s.run(None, {"x": np.array([[-1, 2, 3], [4, -5, 6]], np.float32)})
'''
    env = dict(os.environ, ORT_DEBUG_NODE_IO_DUMP_SHAPE_DATA="1", ORT_DEBUG_NODE_IO_DUMP_NODE_PLACEMENT="1",
               ORT_DEBUG_NODE_IO_DUMP_STATISTICS_DATA="1", ORT_DEBUG_NODE_IO_DUMP_OUTPUT_DATA="1", ORT_DEBUG_NODE_IO_OP_TYPE_FILTER="Log",
               ORT_DEBUG_NODE_IO_SNIPPET_EDGE_ITEMS="2")
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__))), env.get("PYTHONPATH", "")])
    out = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    text = out.stdout
    assert "node 'log0' (Log) on CPUExecutionProvider" in text and "relu0" not in text
    assert "input 'r' Float [2, 3]" in text and "output 'y' Float [2, 3]" in text
    assert "inf 2" in text and "count 6" in text                 # log(0) twice
    assert "data: [-inf 0.693147 ... -inf 1.79176]" in text
    env.update(ORT_DEBUG_NODE_IO_DUMP_DATA_DESTINATION="files", ORT_DEBUG_NODE_IO_OUTPUT_DIR=str(tmp_path), ORT_DEBUG_NODE_IO_OP_TYPE_FILTER="Relu")
    out = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0 and "node '" not in out.stdout
    assert "output 'r' Float [2, 3]" in (tmp_path / "relu0.txt").read_text()


def test_python_api_vectors_sparse_tensors_and_module_functions(tmp_path):
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    from helpers import graph_model
    T = ol.TensorProto
    model = graph_model([ol.make_node("MatMul", ["a", "b"], ["y"])], [ol.make_tensor_value_info("a", T.FLOAT, [3, 4]), ol.make_tensor_value_info("b", T.FLOAT, [4, 2])],
                        [ol.make_tensor_value_info("y", T.FLOAT, None)])
    sess = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    a = np.zeros((3, 4), np.float32)
    a[0, 1], a[2, 3] = 2.0, -1.0
    b = np.arange(8, dtype=np.float32).reshape(4, 2)
    # OrtValueVector + run_with_ortvaluevector
    feeds = ort.OrtValueVector()
    feeds.push_back(ort.OrtValue.ortvalue_from_numpy(a))
    feeds.push_back(b)
    fetches = ort.OrtValueVector()
    sess.run_with_ortvaluevector(None, ["a", "b"], feeds, ["y"], fetches, [ort.OrtDevice("cpu", 0)])
    assert len(fetches) == 1
    np.testing.assert_allclose(fetches[0].numpy(), a @ b)
    # sparse tensors are expanded on their way in
    sp = ort.SparseTensor.sparse_coo_from_numpy([3, 4], np.array([2.0, -1.0], np.float32), np.array([1, 11], np.int64))
    assert sp.format() == "COO" and sp.dense_shape() == [3, 4] and sp.data_type() == "sparse_tensor(float)"
    np.testing.assert_array_equal(sp.as_coo_view().indices(), [[0, 1], [2, 3]])
    np.testing.assert_array_equal(sp.to_dense(), a)
    ov = ort.OrtValue.ort_value_from_sparse_tensor(sp)
    assert ov.is_sparse_tensor() and ov.as_sparse_tensor().values().tolist() == [2.0, -1.0]
    np.testing.assert_allclose(sess.run(None, {"a": sp, "b": b})[0], a @ b)
    csr = ort.SparseTensor.sparse_csr_from_numpy([3, 4], np.array([2.0, -1.0], np.float32), np.array([1, 3]), np.array([0, 1, 1, 2]))
    assert csr.format() == "CSR" and csr.as_csrc_view().outer().tolist() == [0, 1, 1, 2]
    np.testing.assert_array_equal(csr.to_dense(), a)
    # module-level functions
    assert ort.get_version_string() and "sm_100a" in ort.get_build_info() and ort.has_collective_ops()
    devices = ort.get_ep_devices()
    assert devices[0].ep_name == "CPUExecutionProvider"
    ort.set_seed(7)
    ort.disable_telemetry_events()
    # provider selection through the options object
    so = ort.SessionOptions()
    so.add_provider_for_devices([devices[0]])
    assert ort.InferenceSession(model, so).get_providers() == ["CPUExecutionProvider"]
    so = ort.SessionOptions()
    so.set_provider_selection_policy(ort.OrtExecutionProviderDevicePolicy.PREFER_CPU)
    assert ort.InferenceSession(model, so).get_providers() == ["CPUExecutionProvider"]
    so = ort.SessionOptions()
    so.set_load_cancellation_flag(True)
    with pytest.raises(ort.ModelLoadCanceled):
        ort.InferenceSession(model, so)
    # external data handed over as memory
    w = np.arange(8, dtype=np.float32).reshape(4, 2)
    ext = graph_model([ol.make_node("MatMul", ["a", "w"], ["y"])], [ol.make_tensor_value_info("a", T.FLOAT, [3, 4])], [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_external_tensor("w", T.FLOAT, [4, 2], location="weights.bin", offset=16, length=32)])
    so = ort.SessionOptions()
    blob = bytes(16) + w.tobytes()
    so.add_external_initializers_from_files_in_memory(["weights.bin"], [blob], [len(blob)])
    np.testing.assert_allclose(ort.InferenceSession(ext, so).run(None, {"a": a})[0], a @ w)
