"""ONNX protobuf reader/writer: the Python writer and the C++ parser/serializer check each other."""
import numpy as np
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200 import _core as C
from onnxruntime_b200 import onnx_lite as ol

T = ol.TensorProto


def _model():
    w = np.arange(12, dtype=np.float32).reshape(4, 3)
    nodes = [ol.make_node("MatMul", ["x", "w"], ["y0"], name="mm"),
             ol.make_node("LeakyRelu", ["y0"], ["y1"], alpha=0.25),
             ol.make_node("Transpose", ["y1"], ["y"], perm=[1, 0]),
             ol.make_node("FastGelu", ["y"], ["z"], domain="com.microsoft")]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, ["batch", 4])],
                      [ol.make_tensor_value_info("z", T.FLOAT, [3, "batch"])], [ol.make_tensor("w", w)])
    return ol.make_model(g, metadata={"k": "v"}).serialize()


def test_roundtrip_preserves_graph():
    m = _model()
    again = C.model_roundtrip(m)
    n1, n2 = C.model_nodes(m), C.model_nodes(again)
    assert [(n["op_type"], n["domain"], n["inputs"], n["outputs"]) for n in n1] == \
           [(n["op_type"], n["domain"], n["inputs"], n["outputs"]) for n in n2]
    assert n2[1]["attrs"]["alpha"] == pytest.approx(0.25)
    assert n2[2]["attrs"]["perm"] == [1, 0]
    # a second round trip is byte-stable
    assert C.model_roundtrip(again) == again
    s = ort.InferenceSession(again, providers=["CPUExecutionProvider"])
    assert s.get_modelmeta().custom_metadata_map == {"k": "v"}
    assert s.get_inputs()[0].shape == ["batch", 4]
    assert s.get_outputs()[0].type == "tensor(float)"


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.float64, np.int64, np.int32, np.int8, np.uint8, np.bool_, np.int16])
def test_tensor_roundtrip_numpy_types(dtype):
    a = (np.random.RandomState(0).randn(3, 5) * 10).astype(dtype)
    t = C.tensor_from_proto(ol.make_tensor("t", a).serialize())
    assert t.shape == (3, 5)
    np.testing.assert_array_equal(t.numpy(), a)
    back = C.tensor_from_proto(C.tensor_to_proto(t, "t"))
    np.testing.assert_array_equal(back.numpy(), a)


def test_tensor_bf16_and_fp8():
    a = torch.randn(4, 4).bfloat16()
    t = C.tensor_from_proto(ol.make_tensor("t", a).serialize())
    assert t.dtype == torch.bfloat16 and torch.equal(t, a)
    f8 = torch.randn(8).to(torch.float8_e4m3fn)
    t8 = C.tensor_from_proto(ol.make_tensor("t", f8).serialize())
    assert t8.dtype == torch.float8_e4m3fn and torch.equal(t8.view(torch.uint8), f8.view(torch.uint8))


def test_typed_fields_are_decoded():
    # float_data (field 4, packed) instead of raw_data
    import struct
    vals = [1.5, -2.0, 3.25]
    body = ol._packed_varints(1, [3]) + ol._f_varint(2, T.FLOAT) + ol._f_bytes(4, struct.pack("<3f", *vals)) + ol._f_str(8, "t")
    t = C.tensor_from_proto(body)
    np.testing.assert_allclose(t.numpy(), vals)
    # int64_data as unpacked varints (field 7, wire type 0)
    body = ol._packed_varints(1, [2]) + ol._f_varint(2, T.INT64) + ol._f_varint(7, 7) + ol._f_varint(7, -3)
    np.testing.assert_array_equal(C.tensor_from_proto(body).numpy(), [7, -3])
    # fp16 bit patterns in int32_data
    h = np.array([1.0, -0.5], np.float16)
    body = ol._packed_varints(1, [2]) + ol._f_varint(2, T.FLOAT16) + ol._packed_varints(5, h.view(np.uint16).tolist())
    np.testing.assert_array_equal(C.tensor_from_proto(body).numpy(), h)


def test_malformed_input_is_rejected():
    m = _model()
    with pytest.raises(ort.InvalidProtobuf):
        ort.InferenceSession(b"\x08", providers=["CPUExecutionProvider"])  # truncated varint after a key
    with pytest.raises((ort.InvalidProtobuf, ort.InvalidArgument, ort.InvalidGraph, ort.Fail, ort.NotImplemented)):
        ort.InferenceSession(m[: len(m) // 2], providers=["CPUExecutionProvider"])
    with pytest.raises(ort.InvalidProtobuf):
        ort.InferenceSession(b"not an onnx file at all \xff\xff\xff", providers=["CPUExecutionProvider"])


def test_truncation_never_crashes():
    m = _model()
    rng = np.random.RandomState(0)
    for _ in range(200):
        cut = rng.randint(1, len(m))
        data = bytearray(m[:cut])
        if rng.rand() < 0.5 and len(data) > 4:
            data[rng.randint(0, len(data))] ^= 1 << rng.randint(0, 8)
        try:
            C.model_nodes(bytes(data))
        except ort.OrtException:
            pass


def test_unknown_fields_are_skipped():
    m = _model()
    extra = ol._f_str(99, "future field") + ol._f_varint(98, 5)
    s = ort.InferenceSession(m + extra, providers=["CPUExecutionProvider"])
    assert len(s.graph_nodes()) >= 1


def test_external_data_file(tmp_path):
    w = np.random.RandomState(0).randn(4, 3).astype(np.float32)
    (tmp_path / "weights.bin").write_bytes(b"\0" * 16 + w.tobytes())
    g = ol.make_graph([ol.make_node("MatMul", ["x", "w"], ["y"])], "g", [ol.make_tensor_value_info("x", T.FLOAT, [2, 4])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [2, 3])],
                      [ol.make_external_tensor("w", T.FLOAT, [4, 3], location="weights.bin", offset=16, length=w.nbytes)])
    path = tmp_path / "m.onnx"
    path.write_bytes(ol.make_model(g).serialize())
    s = ort.InferenceSession(str(path), providers=["CPUExecutionProvider"])
    x = np.ones((2, 4), np.float32)
    np.testing.assert_allclose(s.run(None, {"x": x})[0], x @ w, rtol=1e-6)
    # a location that escapes the model directory is refused
    g.initializers[0] = ol.make_external_tensor("w", T.FLOAT, [4, 3], location="../weights.bin")
    path.write_bytes(ol.make_model(g).serialize())
    with pytest.raises(ort.InvalidArgument):
        ort.InferenceSession(str(path), providers=["CPUExecutionProvider"])


def test_session_supplied_external_initializers():
    g = ol.make_graph([ol.make_node("Add", ["x", "w"], ["y"])], "g", [ol.make_tensor_value_info("x", T.FLOAT, [3])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [3])], [ol.make_external_tensor("w", T.FLOAT, [3])])
    m = ol.make_model(g).serialize()
    with pytest.raises(ort.InvalidArgument):
        ort.InferenceSession(m, providers=["CPUExecutionProvider"])
    so = ort.SessionOptions()
    so.add_external_initializers(["w"], [ort.OrtValue.ortvalue_from_numpy(np.array([1, 2, 3], np.float32))])
    s = ort.InferenceSession(m, so, providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(s.run(None, {"x": np.zeros(3, np.float32)})[0], [1, 2, 3])


def test_function_inlining():
    # a model-local function Twice(x) = x + x, called once
    fn_node = ol.make_node("Add", ["a", "a"], ["b"])
    fn = ol._f_str(1, "Twice") + ol._f_str(4, "a") + ol._f_str(5, "b") + ol._f_bytes(7, fn_node.serialize()) + \
        ol._f_bytes(9, ol._f_varint(2, 17)) + ol._f_str(10, "local")
    g = ol.make_graph([ol.make_node("Twice", ["x"], ["y"], domain="local")], "g", [ol.make_tensor_value_info("x", T.FLOAT, [2])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [2])])
    m = ol.make_model(g, extra_opsets={"local": 1}).serialize() + ol._f_bytes(25, fn)
    s = ort.InferenceSession(m, providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(s.run(None, {"x": np.array([1.5, -2], np.float32)})[0], [3, -4])
