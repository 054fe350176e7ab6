"""Custom operators (Python callables and a C-ABI shared library) and LoRA adapters."""
import os
import subprocess

import numpy as np
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol

T = ol.TensorProto
HERE = os.path.dirname(os.path.abspath(__file__))


def test_python_custom_op_with_attributes_and_two_outputs():
    def scale_and_sum(x, y=None, *, factor=1.0, tag=b""):
        assert tag == b"demo"
        s = x * factor if y is None else (x + y) * factor
        return s, s.sum(dim=-1)

    ort.register_custom_op("test.domain", "ScaleAndSum", scale_and_sum)
    g = ol.make_graph([ol.make_node("ScaleAndSum", ["a", ""], ["s", "t"], domain="test.domain", factor=2.5, tag="demo"),
                       ol.make_node("Neg", ["t"], ["u"])], "g",
                      [ol.make_tensor_value_info("a", T.FLOAT, [2, 3])],
                      [ol.make_tensor_value_info("s", T.FLOAT, None), ol.make_tensor_value_info("u", T.FLOAT, None)])
    m = ol.make_model(g, extra_opsets={"test.domain": 1}).serialize()
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    s, u = ort.InferenceSession(m, providers=["CPUExecutionProvider"]).run(None, {"a": a})
    np.testing.assert_allclose(s, a * 2.5)
    np.testing.assert_allclose(u, -(a * 2.5).sum(-1))


def test_python_custom_op_error_is_reported():
    def boom(x):
        raise ValueError("bad input")
    ort.register_custom_op("test.domain", "Boom", boom)
    g = ol.make_graph([ol.make_node("Boom", ["a"], ["b"], domain="test.domain")], "g", [ol.make_tensor_value_info("a", T.FLOAT, [1])],
                      [ol.make_tensor_value_info("b", T.FLOAT, None)])
    sess = ort.InferenceSession(ol.make_model(g, extra_opsets={"test.domain": 1}).serialize(), providers=["CPUExecutionProvider"])
    with pytest.raises(ort.OrtException, match="bad input"):
        sess.run(None, {"a": np.zeros(1, np.float32)})


C_SOURCE = r"""
#include <string.h>
#include "custom_op_api.h"
/* y = alpha * x + 1 for float tensors; fails on any other type */
static int axpb(const ortb200_custom_op_api* api, ortb200_kernel_context* ctx, const ortb200_tensor* in, int n_in, int n_out, void* user) {
  (void)user; (void)n_out;
  if (n_in < 1 || !in[0].present || in[0].elem_type != 1) { api->set_error(ctx, "expects one float tensor"); return 3; }
  float alpha = 1.0f;
  api->attr_float(ctx, "alpha", &alpha);
  ortb200_tensor out;
  if (api->allocate_output(ctx, 0, in[0].dims, in[0].ndim, 1, &out) != 0) return 4;
  long long n = 1;
  for (int i = 0; i < in[0].ndim; ++i) n *= in[0].dims[i];
  const float* x = (const float*)in[0].data; float* y = (float*)out.data;
  for (long long i = 0; i < n; ++i) y[i] = alpha * x[i] + 1.0f;
  return 0;
}
int ortb200_register_custom_ops(const ortb200_custom_op_api* api) {
  if (api->version != ORTB200_CUSTOM_OP_API_VERSION) return 1;
  return api->register_op("test.native", "Axpb", axpb, 0);
}
"""


def test_shared_library_custom_op(tmp_path):
    src = tmp_path / "ops.c"
    src.write_text(C_SOURCE)
    lib = tmp_path / "libops.so"
    inc = os.path.join(os.path.dirname(HERE), "onnxruntime_b200", "csrc", "core")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", f"-I{inc}", str(src), "-o", str(lib)], check=True)
    so = ort.SessionOptions()
    so.register_custom_ops_library(str(lib))
    g = ol.make_graph([ol.make_node("Axpb", ["a"], ["b"], domain="test.native", alpha=3.0)], "g",
                      [ol.make_tensor_value_info("a", T.FLOAT, [4])], [ol.make_tensor_value_info("b", T.FLOAT, None)])
    m = ol.make_model(g, extra_opsets={"test.native": 1}).serialize()
    sess = ort.InferenceSession(m, so, providers=["CPUExecutionProvider"])
    a = np.array([1, 2, 3, 4], dtype=np.float32)
    np.testing.assert_allclose(sess.run(None, {"a": a})[0], 3 * a + 1)
    g2 = ol.make_graph([ol.make_node("Axpb", ["a"], ["b"], domain="test.native")], "g",
                       [ol.make_tensor_value_info("a", T.INT64, [2])], [ol.make_tensor_value_info("b", T.FLOAT, None)])
    s2 = ort.InferenceSession(ol.make_model(g2, extra_opsets={"test.native": 1}).serialize(), providers=["CPUExecutionProvider"])
    with pytest.raises(ort.OrtException, match="expects one float tensor"):
        s2.run(None, {"a": np.array([1, 2], dtype=np.int64)})
    with pytest.raises(ort.NoSuchFile):
        so.register_custom_ops_library(str(tmp_path / "missing.so"))


def test_lora_adapter_round_trip_and_activation(tmp_path):
    # y = x @ (W + A @ B); A and B are optional inputs whose defaults (zeros) are overridable initializers
    rng = np.random.RandomState(0)
    W = rng.randn(8, 8).astype(np.float32)
    g = ol.make_graph([ol.make_node("MatMul", ["lora_a", "lora_b"], ["delta"]), ol.make_node("Add", ["w", "delta"], ["w_eff"]),
                       ol.make_node("MatMul", ["x", "w_eff"], ["y"])], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [2, 8]), ol.make_tensor_value_info("lora_a", T.FLOAT, [8, 2]),
                       ol.make_tensor_value_info("lora_b", T.FLOAT, [2, 8])],
                      [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_tensor("w", W), ol.make_tensor("lora_a", np.zeros((8, 2), np.float32)),
                       ol.make_tensor("lora_b", np.zeros((2, 8), np.float32))])
    sess = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    x = rng.randn(2, 8).astype(np.float32)
    np.testing.assert_allclose(sess.run(None, {"x": x})[0], x @ W, rtol=1e-5)

    A, B = rng.randn(8, 2).astype(np.float32), rng.randn(2, 8).astype(np.float32)
    fmt = ort.AdapterFormat()
    fmt.set_adapter_version(3)
    fmt.set_model_version(7)
    fmt.set_parameters({"lora_a": A, "lora_b": torch.from_numpy(B), "unused": np.ones(1, np.float32)})
    path = str(tmp_path / "adapter.bin")
    fmt.export_adapter(path)
    back = ort.AdapterFormat.read_adapter(path)
    assert back.get_adapter_version() == 3 and back.get_model_version() == 7
    np.testing.assert_array_equal(back.get_parameters()["lora_a"].numpy(), A)

    adapter = ort.LoraAdapter()
    adapter.Load(path)
    ro = ort.RunOptions()
    ro.add_active_adapter(adapter)
    np.testing.assert_allclose(sess.run(None, {"x": x}, ro)[0], x @ (W + A @ B), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(sess.run(None, {"x": x})[0], x @ W, rtol=1e-5)  # without the options the base model runs


def test_adapter_files_use_the_flatbuffer_layout_of_the_reference(tmp_path):
    """export_adapter writes a FlatBuffer with identifier TORT (Adapter{format_version, adapter_version, model_version,
    parameters[name, dims, data_type, raw_data aligned to 8]}); a hand-assembled buffer in that layout reads back."""
    import struct
    import torch
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import flatbuf_lite as fb
    a = ort.AdapterFormat()
    a.set_adapter_version(7)
    a.set_model_version(3)
    a.set_parameters({"lora_a": np.arange(8, dtype=np.float32).reshape(4, 2), "lora_b": torch.arange(6).reshape(2, 3).to(torch.bfloat16),
                      "steps": np.array([5], np.int64)})
    path = tmp_path / "a.onnx_adapter"
    a.export_adapter(str(path))
    buf = path.read_bytes()
    assert buf[4:8] == b"TORT"
    fmt, av, mv, params = fb.read_adapter(buf)
    assert (fmt, av, mv) == (1, 7, 3) and [p[0] for p in params] == ["lora_a", "lora_b", "steps"]
    assert params[0][1:3] == ([4, 2], 1) and params[1][1:3] == ([2, 3], 16) and params[2][1:3] == ([1], 7)
    for name, dims, et, raw in params:
        assert buf.find(raw) % 8 == 0                       # raw_data: force_align 8
    b = ort.AdapterFormat.read_adapter(str(path))
    assert b.get_adapter_version() == 7 and b.get_model_version() == 3
    got = b.get_parameters()
    np.testing.assert_array_equal(got["lora_a"].numpy(), np.arange(8, dtype=np.float32).reshape(4, 2))
    assert got["lora_b"]._tensor.dtype == torch.bfloat16 and got["lora_b"]._tensor.float().tolist() == [[0, 1, 2], [3, 4, 5]]
    # a buffer laid out by hand, fields in another order and one field absent (default 0), as another writer might do
    raw = struct.pack("<2f", 1.5, -2.0)
    out = bytearray(b"\0\0\0\0TORT")
    vt = len(out); out += struct.pack("<HHHHHH", 12, 12, 0, 4, 0, 8)          # format_version, model_version absent
    tab = len(out); out += struct.pack("<iiI", tab - vt, 9, 0)
    struct.pack_into("<I", out, 0, tab)
    vec = len(out); struct.pack_into("<I", out, tab + 8, vec - (tab + 8)); out += struct.pack("<II", 1, 0)
    pvt = len(out); out += struct.pack("<HHHHHH", 12, 20, 16, 12, 4, 8)       # name at 16, dims at 12, type at 4, data at 8
    while len(out) % 4:
        out.append(0)
    pt = len(out); out += struct.pack("<iiIII", pt - pvt, 1, 0, 0, 0)
    struct.pack_into("<I", out, vec + 4, pt - (vec + 4))
    while (len(out) + 4) % 8:
        out.append(0)
    struct.pack_into("<I", out, pt + 8, len(out) - (pt + 8)); out += struct.pack("<I", len(raw)) + raw
    struct.pack_into("<I", out, pt + 12, len(out) - (pt + 12)); out += struct.pack("<Iq", 1, 2)
    struct.pack_into("<I", out, pt + 16, len(out) - (pt + 16)); out += struct.pack("<I", 1) + b"w\0"
    fmt, av, mv, params = fb.read_adapter(bytes(out))
    assert (fmt, av, mv) == (0, 9, 0) and params == [("w", [2], 1, raw)]
    bad = tmp_path / "bad.onnx_adapter"
    bad.write_bytes(bytes(out[:40]))
    with pytest.raises(Exception):
        ort.AdapterFormat.read_adapter(str(bad))
