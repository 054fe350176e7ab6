"""ONNX-domain operators on the CPU provider versus numpy / torch references (one-node models)."""
import numpy as np
import pytest
import torch

from helpers import run_node

rng = np.random.RandomState(0)


def f32(*shape):
    return rng.randn(*shape).astype(np.float32)


@pytest.mark.parametrize("op,fn", [
    ("Abs", np.abs), ("Neg", np.negative), ("Floor", np.floor), ("Ceil", np.ceil), ("Exp", np.exp), ("Tanh", np.tanh),
    ("Sigmoid", lambda x: 1 / (1 + np.exp(-x))), ("Relu", lambda x: np.maximum(x, 0)), ("Sin", np.sin), ("Cos", np.cos),
    ("Sign", np.sign), ("Round", np.round), ("Softsign", lambda x: x / (1 + np.abs(x))),
    ("Softplus", lambda x: np.log1p(np.exp(x))), ("Erf", lambda x: torch.erf(torch.from_numpy(x)).numpy()),
])
def test_unary(op, fn):
    x = f32(3, 5)
    np.testing.assert_allclose(run_node(op, {"x": x})[0], fn(x), rtol=1e-5, atol=1e-6)


def test_sqrt_log_reciprocal():
    x = np.abs(f32(4, 4)) + 0.1
    np.testing.assert_allclose(run_node("Sqrt", {"x": x})[0], np.sqrt(x), rtol=1e-6)
    np.testing.assert_allclose(run_node("Log", {"x": x})[0], np.log(x), rtol=1e-6)
    np.testing.assert_allclose(run_node("Reciprocal", {"x": x})[0], 1 / x, rtol=1e-6)


@pytest.mark.parametrize("op,fn", [("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply), ("Div", np.divide),
                                   ("Max", np.maximum), ("Min", np.minimum)])
def test_binary_broadcast(op, fn):
    a, b = f32(2, 3, 4), f32(3, 1) + 2.0
    np.testing.assert_allclose(run_node(op, {"a": a, "b": b})[0], fn(a, b), rtol=1e-6)


def test_integer_div_truncates_and_mod():
    a = np.array([7, -7, 9, -9], np.int32)
    b = np.array([2, 2, -4, -4], np.int32)
    np.testing.assert_array_equal(run_node("Div", {"a": a, "b": b})[0], np.trunc(a / b).astype(np.int32))
    np.testing.assert_array_equal(run_node("Mod", {"a": a, "b": b})[0], np.mod(a, b))
    np.testing.assert_array_equal(run_node("Mod", {"a": a, "b": b}, fmod=1)[0], np.fmod(a, b))


def test_compare_logical_where():
    a, b = f32(4, 4), f32(4, 4)
    np.testing.assert_array_equal(run_node("Less", {"a": a, "b": b})[0], a < b)
    np.testing.assert_array_equal(run_node("GreaterOrEqual", {"a": a, "b": b})[0], a >= b)
    np.testing.assert_array_equal(run_node("Equal", {"a": a, "b": a.copy()})[0], np.ones((4, 4), bool))
    c = a > 0
    np.testing.assert_array_equal(run_node("Where", {"c": c, "a": a, "b": b})[0], np.where(c, a, b))
    np.testing.assert_array_equal(run_node("And", {"a": c, "b": b > 0})[0], c & (b > 0))
    np.testing.assert_array_equal(run_node("Not", {"a": c})[0], ~c)


def test_cast_and_clip():
    x = np.array([-1.7, 0.2, 2.9], np.float32)
    np.testing.assert_array_equal(run_node("Cast", {"x": x}, to=7)[0], np.array([-1, 0, 2], np.int64))
    np.testing.assert_array_equal(run_node("Cast", {"x": x}, to=9)[0], np.array([True, True, True]))
    out = run_node("Cast", {"x": x}, to=10)[0]
    assert out.dtype == np.float16
    lo, hi = np.array(-1.0, np.float32), np.array(1.0, np.float32)
    np.testing.assert_allclose(run_node("Clip", {"x": x, "lo": lo, "hi": hi})[0], np.clip(x, -1, 1))
    np.testing.assert_allclose(run_node("Clip", {"x": x}, opset=6, min=-0.5, max=0.5)[0], np.clip(x, -0.5, 0.5))


def test_activations_with_attrs():
    x = f32(4, 6)
    np.testing.assert_allclose(run_node("LeakyRelu", {"x": x}, alpha=0.1)[0], np.where(x > 0, x, 0.1 * x), rtol=1e-6)
    np.testing.assert_allclose(run_node("Elu", {"x": x}, alpha=1.5)[0], np.where(x > 0, x, 1.5 * (np.exp(x) - 1)), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run_node("HardSigmoid", {"x": x}, alpha=0.3, beta=0.4)[0], np.clip(0.3 * x + 0.4, 0, 1), rtol=1e-6)
    np.testing.assert_allclose(run_node("Gelu", {"x": x}, opset=20)[0], torch.nn.functional.gelu(torch.from_numpy(x)).numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run_node("Gelu", {"x": x}, opset=20, approximate="tanh")[0],
                               torch.nn.functional.gelu(torch.from_numpy(x), approximate="tanh").numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run_node("PRelu", {"x": x, "s": np.array([0.2], np.float32)})[0], np.where(x < 0, 0.2 * x, x), rtol=1e-6)


def test_matmul_gemm_einsum():
    a, b, c = f32(2, 3, 4), f32(4, 5), f32(5)
    np.testing.assert_allclose(run_node("MatMul", {"a": a, "b": b})[0], a @ b, rtol=1e-5, atol=1e-5)
    a2 = f32(3, 4)
    np.testing.assert_allclose(run_node("Gemm", {"a": a2, "b": b, "c": c}, alpha=0.5, beta=2.0)[0], 0.5 * a2 @ b + 2 * c, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(run_node("Gemm", {"a": a2.T.copy(), "b": b.T.copy()}, transA=1, transB=1)[0], a2 @ b, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(run_node("Einsum", {"a": a, "b": b}, equation="bij,jk->bik")[0], a @ b, rtol=1e-5, atol=1e-5)


def test_softmax_variants():
    x = f32(2, 3, 4)
    ref = torch.softmax(torch.from_numpy(x), -1).numpy()
    np.testing.assert_allclose(run_node("Softmax", {"x": x})[0], ref, rtol=1e-6)
    # opset 11: flatten to 2-D at axis=1
    ref11 = torch.softmax(torch.from_numpy(x).reshape(2, 12), 1).reshape(2, 3, 4).numpy()
    np.testing.assert_allclose(run_node("Softmax", {"x": x}, opset=11)[0], ref11, rtol=1e-6)
    np.testing.assert_allclose(run_node("LogSoftmax", {"x": x}, axis=1)[0], torch.log_softmax(torch.from_numpy(x), 1).numpy(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("op,fn", [("ReduceSum", np.sum), ("ReduceMean", np.mean), ("ReduceMax", np.max), ("ReduceMin", np.min), ("ReduceProd", np.prod)])
def test_reduce(op, fn):
    x = f32(2, 3, 4)
    axes_in = np.array([1], np.int64)
    if op == "ReduceSum":
        np.testing.assert_allclose(run_node(op, {"x": x, "axes": axes_in}, keepdims=0)[0], fn(x, axis=1), rtol=1e-5)
    else:
        np.testing.assert_allclose(run_node(op, {"x": x}, axes=[1], keepdims=0)[0], fn(x, axis=1), rtol=1e-5)
        np.testing.assert_allclose(run_node(op, {"x": x, "axes": axes_in}, opset=18, keepdims=1)[0], fn(x, axis=1, keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(run_node(op, {"x": x}, opset=12, keepdims=0)[0], fn(x), rtol=1e-4)


def test_reduce_other_and_arg():
    x = f32(3, 5)
    np.testing.assert_allclose(run_node("ReduceL2", {"x": x}, axes=[1], keepdims=0)[0], np.sqrt((x * x).sum(1)), rtol=1e-5)
    np.testing.assert_allclose(run_node("ReduceLogSumExp", {"x": x}, axes=[1], keepdims=0)[0], np.log(np.exp(x).sum(1)), rtol=1e-5)
    np.testing.assert_array_equal(run_node("ArgMax", {"x": x}, axis=1, keepdims=0)[0], x.argmax(1))
    np.testing.assert_array_equal(run_node("ArgMin", {"x": x}, axis=0, keepdims=1)[0], x.argmin(0)[None])


def test_shape_ops():
    x = f32(2, 3, 4)
    np.testing.assert_array_equal(run_node("Shape", {"x": x})[0], [2, 3, 4])
    np.testing.assert_array_equal(run_node("Shape", {"x": x}, start=1, end=-1)[0], [3])
    np.testing.assert_array_equal(run_node("Size", {"x": x})[0], 24)
    np.testing.assert_array_equal(run_node("Reshape", {"x": x, "s": np.array([0, -1], np.int64)})[0], x.reshape(2, 12))
    np.testing.assert_array_equal(run_node("Flatten", {"x": x}, axis=2)[0], x.reshape(6, 4))
    np.testing.assert_array_equal(run_node("Transpose", {"x": x}, perm=[2, 0, 1])[0], x.transpose(2, 0, 1))
    np.testing.assert_array_equal(run_node("Transpose", {"x": x})[0], x.transpose())
    np.testing.assert_array_equal(run_node("Unsqueeze", {"x": x, "a": np.array([0, 4], np.int64)})[0], x[None, ..., None])
    np.testing.assert_array_equal(run_node("Squeeze", {"x": x[:, :1], "a": np.array([1], np.int64)})[0], x[:, 0])
    np.testing.assert_array_equal(run_node("Squeeze", {"x": x[:, :1]}, opset=11, axes=[1])[0], x[:, 0])
    np.testing.assert_array_equal(run_node("Expand", {"x": x[:, :1], "s": np.array([2, 3, 4], np.int64)})[0], np.broadcast_to(x[:, :1], (2, 3, 4)))
    np.testing.assert_array_equal(run_node("Tile", {"x": x, "r": np.array([1, 2, 1], np.int64)})[0], np.tile(x, (1, 2, 1)))


def test_concat_split_slice():
    a, b = f32(2, 3), f32(2, 2)
    np.testing.assert_array_equal(run_node("Concat", {"a": a, "b": b}, axis=1)[0], np.concatenate([a, b], 1))
    x = f32(6, 4)
    outs = run_node("Split", {"x": x, "s": np.array([1, 2, 3], np.int64)}, n_outputs=3, axis=0)
    for o, r in zip(outs, np.split(x, [1, 3])):
        np.testing.assert_array_equal(o, r)
    outs = run_node("Split", {"x": x}, n_outputs=2, axis=1)
    np.testing.assert_array_equal(outs[1], x[:, 2:])
    s = run_node("Slice", {"x": x, "st": np.array([1, 0], np.int64), "en": np.array([5, 4], np.int64),
                           "ax": np.array([0, 1], np.int64), "sp": np.array([2, 1], np.int64)})[0]
    np.testing.assert_array_equal(s, x[1:5:2])
    s = run_node("Slice", {"x": x, "st": np.array([-1], np.int64), "en": np.array([-7], np.int64),
                           "ax": np.array([0], np.int64), "sp": np.array([-1], np.int64)})[0]
    np.testing.assert_array_equal(s, x[::-1])
    s = run_node("Slice", {"x": x}, opset=9, starts=[1], ends=[100], axes=[1])[0]
    np.testing.assert_array_equal(s, x[:, 1:])


def test_gather_scatter_family():
    x = f32(5, 4)
    idx = np.array([[0, -1], [2, 2]], np.int64)
    np.testing.assert_array_equal(run_node("Gather", {"x": x, "i": idx}, axis=0)[0], x[idx])
    np.testing.assert_array_equal(run_node("Gather", {"x": x, "i": np.array([1, 3], np.int64)}, axis=1)[0], x[:, [1, 3]])
    ge = np.array([[0, 1, 2, 3], [4, 3, 2, 1]], np.int64)
    np.testing.assert_array_equal(run_node("GatherElements", {"x": x, "i": ge}, axis=0)[0], np.take_along_axis(x, ge, 0))
    nd = np.array([[0, 1], [4, 3]], np.int64)
    np.testing.assert_array_equal(run_node("GatherND", {"x": x, "i": nd})[0], x[[0, 4], [1, 3]])
    upd = f32(2, 4)
    ref = x.copy()
    ref[[1, 3]] = upd
    np.testing.assert_array_equal(run_node("ScatterND", {"x": x, "i": np.array([[1], [3]], np.int64), "u": upd})[0], ref)
    ref = x.copy()
    np.put_along_axis(ref, ge, f32(2, 4) * 0 + 7, 0)
    np.testing.assert_array_equal(run_node("ScatterElements", {"x": x, "i": ge, "u": np.full((2, 4), 7, np.float32)}, axis=0)[0], ref)


def test_misc_tensor_ops():
    x = f32(3, 4)
    np.testing.assert_array_equal(run_node("Trilu", {"x": x}, upper=0)[0], np.tril(x))
    np.testing.assert_array_equal(run_node("Trilu", {"x": x, "k": np.array(1, np.int64)})[0], np.triu(x, 1))
    np.testing.assert_allclose(run_node("CumSum", {"x": x, "a": np.array(1, np.int64)})[0], np.cumsum(x, 1), rtol=1e-6)
    np.testing.assert_allclose(run_node("CumSum", {"x": x, "a": np.array(0, np.int64)}, reverse=1, exclusive=1)[0],
                               np.flip(np.cumsum(np.flip(x, 0), 0), 0) - x, rtol=1e-5, atol=1e-6)
    v, i = run_node("TopK", {"x": x, "k": np.array([2], np.int64)}, n_outputs=2, axis=1)
    np.testing.assert_allclose(v, np.sort(x, 1)[:, ::-1][:, :2])
    np.testing.assert_array_equal(run_node("Range", {"s": np.array(2, np.int64), "l": np.array(11, np.int64), "d": np.array(3, np.int64)})[0], np.arange(2, 11, 3))
    np.testing.assert_array_equal(run_node("ConstantOfShape", {"s": np.array([2, 2], np.int64)}, value=np.array([5], np.int32))[0], np.full((2, 2), 5, np.int32))
    np.testing.assert_array_equal(run_node("NonZero", {"x": (x > 0)})[0], np.array(np.nonzero(x > 0)))
    oh = run_node("OneHot", {"i": np.array([0, 2], np.int64), "d": np.array(3, np.int64), "v": np.array([0, 1], np.float32)})[0]
    np.testing.assert_array_equal(oh, np.eye(3, dtype=np.float32)[[0, 2]])
    pads = np.array([0, 1, 0, 2], np.int64)
    np.testing.assert_array_equal(run_node("Pad", {"x": x, "p": pads, "v": np.array(9, np.float32)})[0],
                                  np.pad(x, ((0, 0), (1, 2)), constant_values=9))
    np.testing.assert_array_equal(run_node("Pad", {"x": x, "p": pads}, mode="reflect")[0], np.pad(x, ((0, 0), (1, 2)), mode="reflect"))
    d2s = f32(1, 8, 2, 3)
    np.testing.assert_array_equal(run_node("DepthToSpace", {"x": d2s}, blocksize=2)[0],
                                  torch.nn.functional.pixel_shuffle(torch.from_numpy(d2s).reshape(1, 2, 2, 2, 2, 3).permute(0, 3, 1, 2, 4, 5).reshape(1, 8, 2, 3), 2).numpy())


def test_layernorm_family():
    x, g, b = f32(2, 5, 16), f32(16), f32(16)
    ref = torch.nn.functional.layer_norm(torch.from_numpy(x), (16,), torch.from_numpy(g), torch.from_numpy(b), 1e-5).numpy()
    np.testing.assert_allclose(run_node("LayerNormalization", {"x": x, "g": g, "b": b}, axis=-1, epsilon=1e-5)[0], ref, rtol=1e-4, atol=1e-5)
    rms = x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6) * g
    np.testing.assert_allclose(run_node("SimplifiedLayerNormalization", {"x": x, "g": g}, axis=-1, epsilon=1e-6)[0], rms, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(run_node("RMSNormalization", {"x": x, "g": g}, opset=23, axis=-1, epsilon=1e-6)[0], rms, rtol=1e-4, atol=1e-5)
    xb, sc, bi, mean, var = f32(2, 3, 4, 4), f32(3), f32(3), f32(3), np.abs(f32(3)) + 0.5
    refbn = torch.nn.functional.batch_norm(torch.from_numpy(xb), torch.from_numpy(mean), torch.from_numpy(var), torch.from_numpy(sc), torch.from_numpy(bi), False, 0.0, 1e-5).numpy()
    np.testing.assert_allclose(run_node("BatchNormalization", {"x": xb, "s": sc, "b": bi, "m": mean, "v": var})[0], refbn, rtol=1e-4, atol=1e-5)


def test_conv_pool_resize():
    x, w, b = f32(1, 3, 8, 8), f32(4, 3, 3, 3), f32(4)
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b), stride=2, padding=1).numpy()
    np.testing.assert_allclose(run_node("Conv", {"x": x, "w": w, "b": b}, strides=[2, 2], pads=[1, 1, 1, 1], kernel_shape=[3, 3])[0], ref, rtol=1e-4, atol=1e-4)
    same = run_node("Conv", {"x": x, "w": w}, auto_pad="SAME_UPPER", kernel_shape=[3, 3])[0]
    assert same.shape == (1, 4, 8, 8)
    asym = run_node("Conv", {"x": x, "w": w}, pads=[0, 1, 2, 1], kernel_shape=[3, 3])[0]
    refa = torch.nn.functional.conv2d(torch.nn.functional.pad(torch.from_numpy(x), (1, 1, 0, 2)), torch.from_numpy(w)).numpy()
    np.testing.assert_allclose(asym, refa, rtol=1e-4, atol=1e-4)
    wt = f32(3, 2, 3, 3)
    reft = torch.nn.functional.conv_transpose2d(torch.from_numpy(x), torch.from_numpy(wt), stride=2, padding=1, output_padding=1).numpy()
    np.testing.assert_allclose(run_node("ConvTranspose", {"x": x, "w": wt}, strides=[2, 2], pads=[1, 1, 1, 1], output_padding=[1, 1])[0], reft, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(run_node("MaxPool", {"x": x}, kernel_shape=[2, 2], strides=[2, 2])[0],
                               torch.nn.functional.max_pool2d(torch.from_numpy(x), 2).numpy())
    np.testing.assert_allclose(run_node("AveragePool", {"x": x}, kernel_shape=[3, 3], strides=[1, 1], pads=[1, 1, 1, 1])[0],
                               torch.nn.functional.avg_pool2d(torch.from_numpy(x), 3, 1, 1, count_include_pad=False).numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(run_node("GlobalAveragePool", {"x": x})[0], x.mean((2, 3), keepdims=True), rtol=1e-5, atol=1e-6)
    up = run_node("Resize", {"x": x, "roi": None, "scales": np.array([1, 1, 2, 2], np.float32)}, opset=13, mode="nearest",
                  coordinate_transformation_mode="asymmetric", nearest_mode="floor")[0]
    np.testing.assert_array_equal(up, x.repeat(2, 2).repeat(2, 3))
    lin = run_node("Resize", {"x": x, "roi": None, "scales": None, "sizes": np.array([1, 3, 16, 16], np.int64)}, opset=13, mode="linear")[0]
    np.testing.assert_allclose(lin, torch.nn.functional.interpolate(torch.from_numpy(x), size=(16, 16), mode="bilinear", align_corners=False).numpy(), rtol=1e-4, atol=1e-5)


def test_quantize_dequantize():
    x = f32(3, 4) * 3
    scale, zp = np.array(0.05, np.float32), np.array(128, np.uint8)
    q = run_node("QuantizeLinear", {"x": x, "s": scale, "z": zp})[0]
    np.testing.assert_array_equal(q, np.clip(np.round(x / 0.05) + 128, 0, 255).astype(np.uint8))
    np.testing.assert_allclose(run_node("DequantizeLinear", {"x": q, "s": scale, "z": zp})[0], (q.astype(np.float32) - 128) * 0.05, rtol=1e-6)
    sc = np.array([0.1, 0.2, 0.3], np.float32)
    qi = rng.randint(-100, 100, (3, 4)).astype(np.int8)
    np.testing.assert_allclose(run_node("DequantizeLinear", {"x": qi, "s": sc}, axis=0)[0], qi.astype(np.float32) * sc[:, None], rtol=1e-6)
    y, s, z = run_node("DynamicQuantizeLinear", {"x": x}, n_outputs=3)
    assert y.dtype == np.uint8 and np.abs((y.astype(np.float32) - z) * s - x).max() <= s * 0.51


def test_control_flow_if_loop_scan():
    from onnxruntime_b200 import onnx_lite as ol
    import onnxruntime_b200 as ort
    T = ol.TensorProto
    then_g = ol.make_graph([ol.make_node("Add", ["x", "one"], ["t"])], "then", [], [ol.make_tensor_value_info("t", T.FLOAT, None)])
    else_g = ol.make_graph([ol.make_node("Sub", ["x", "one"], ["e"])], "else", [], [ol.make_tensor_value_info("e", T.FLOAT, None)])
    g = ol.make_graph([ol.make_node("If", ["c"], ["y"], then_branch=then_g, else_branch=else_g)], "g",
                      [ol.make_tensor_value_info("c", T.BOOL, []), ol.make_tensor_value_info("x", T.FLOAT, [2])],
                      [ol.make_tensor_value_info("y", T.FLOAT, [2])], [ol.make_tensor("one", np.array([1, 1], np.float32))])
    s = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    x = np.array([3, 4], np.float32)
    np.testing.assert_array_equal(s.run(None, {"c": np.array(True), "x": x})[0], x + 1)
    np.testing.assert_array_equal(s.run(None, {"c": np.array(False), "x": x})[0], x - 1)
    # Loop: sum 0..n-1 carried, scan output collects the running sum
    body = ol.make_graph(
        [ol.make_node("Cast", ["i"], ["fi"], to=T.FLOAT), ol.make_node("Add", ["acc", "fi"], ["acc_out"]),
         ol.make_node("Identity", ["cond_in"], ["cond_out"]), ol.make_node("Identity", ["acc_out"], ["scan"])],
        "body", [ol.make_tensor_value_info("i", T.INT64, []), ol.make_tensor_value_info("cond_in", T.BOOL, []),
                 ol.make_tensor_value_info("acc", T.FLOAT, [])],
        [ol.make_tensor_value_info("cond_out", T.BOOL, []), ol.make_tensor_value_info("acc_out", T.FLOAT, []),
         ol.make_tensor_value_info("scan", T.FLOAT, [])])
    g = ol.make_graph([ol.make_node("Loop", ["n", "", "init"], ["final", "hist"], body=body)], "g",
                      [ol.make_tensor_value_info("n", T.INT64, []), ol.make_tensor_value_info("init", T.FLOAT, [])],
                      [ol.make_tensor_value_info("final", T.FLOAT, []), ol.make_tensor_value_info("hist", T.FLOAT, ["n"])])
    s = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    final, hist = s.run(None, {"n": np.array(5, np.int64), "init": np.array(0, np.float32)})
    assert final == 10 and hist.tolist() == [0, 1, 3, 6, 10]
    # Scan: running sum over rows
    sbody = ol.make_graph([ol.make_node("Add", ["st", "row"], ["st_out"]), ol.make_node("Identity", ["st_out"], ["o"])], "sb",
                          [ol.make_tensor_value_info("st", T.FLOAT, [3]), ol.make_tensor_value_info("row", T.FLOAT, [3])],
                          [ol.make_tensor_value_info("st_out", T.FLOAT, [3]), ol.make_tensor_value_info("o", T.FLOAT, [3])])
    g = ol.make_graph([ol.make_node("Scan", ["s0", "xs"], ["sf", "ys"], body=sbody, num_scan_inputs=1)], "g",
                      [ol.make_tensor_value_info("s0", T.FLOAT, [3]), ol.make_tensor_value_info("xs", T.FLOAT, [4, 3])],
                      [ol.make_tensor_value_info("sf", T.FLOAT, [3]), ol.make_tensor_value_info("ys", T.FLOAT, [4, 3])])
    s = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CPUExecutionProvider"])
    xs = f32(4, 3)
    sf, ys = s.run(None, {"s0": np.zeros(3, np.float32), "xs": xs})
    np.testing.assert_allclose(ys, np.cumsum(xs, 0), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(sf, xs.sum(0), rtol=1e-5, atol=1e-6)


def _qmoe_case(bits=4, block=0, E=4, H=32, I=64, T=6, k=2, dtype=np.float32, seed=0):
    """Quantised expert weights for QMoE plus their dequantised form (what MoE must reproduce)."""
    rng = np.random.RandomState(seed)
    qmax, mid = (15, 8) if bits == 4 else (255, 128)

    def quant(w):  # w [E, rows, K] -> packed, scales, dequantised
        Ee, rows, K = w.shape
        if block:
            wb = w.reshape(Ee, rows, K // block, block)
            s = np.abs(wb).max(-1) / (mid - 1) + 1e-8
            q = np.clip(np.rint(wb / s[..., None]) + mid, 0, qmax).astype(np.uint8).reshape(Ee, rows, K)
            deq = ((q.reshape(Ee, rows, K // block, block).astype(np.float32) - mid) * s[..., None]).reshape(Ee, rows, K)
        else:
            s = np.abs(w).max(-1) / (mid - 1) + 1e-8
            q = np.clip(np.rint(w / s[..., None]) + mid, 0, qmax).astype(np.uint8)
            deq = (q.astype(np.float32) - mid) * s[..., None]
        packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8) if bits == 4 else q
        return packed, s.astype(dtype), deq.astype(dtype)
    fc1 = rng.randn(E, I, H).astype(np.float32) * 0.2
    fc2 = rng.randn(E, H, I).astype(np.float32) * 0.2
    fc3 = rng.randn(E, I, H).astype(np.float32) * 0.2
    x = rng.randn(T, H).astype(dtype)
    logits = (np.argsort(rng.rand(T, E), axis=1) * 0.37 - 1.0).astype(dtype)
    return x, logits, quant(fc1), quant(fc2), quant(fc3)


@pytest.mark.parametrize("bits,block", [(4, 0), (8, 0), (4, 16)])
def test_qmoe_matches_moe_on_dequantised_weights(bits, block):
    x, logits, (p1, s1, d1), (p2, s2, d2), (p3, s3, d3) = _qmoe_case(bits, block)
    attrs = dict(k=2, activation_type="silu", normalize_routing_weights=1)
    q = run_node("QMoE", {"x": x, "r": logits, "w1": p1, "s1": s1, "b1": None, "w2": p2, "s2": s2, "b2": None, "w3": p3, "s3": s3},
                 domain="com.microsoft", expert_weight_bits=bits, block_size=block, **attrs)[0]
    m = run_node("MoE", {"x": x, "r": logits, "w1": d1, "b1": None, "w2": d2, "b2": None, "w3": d3}, domain="com.microsoft", **attrs)[0]
    np.testing.assert_allclose(q, m, rtol=1e-4, atol=1e-5)
