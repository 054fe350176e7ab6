"""ONNX-domain operators of the extended set and integer-quantised contrib operators against torch / numpy
restatements of the ONNX specifications."""
import numpy as np
import pytest
import torch

from helpers import run_node

MS = "com.microsoft"
rng = np.random.default_rng(0)


def _onnx_lstm_weights(m: torch.nn.LSTM, reverse=False):
    sfx = "_reverse" if reverse else ""
    H = m.hidden_size
    def reorder(w):   # torch gate order i f g o -> ONNX i o f c
        i, f, g, o = w.split(H, 0)
        return torch.cat([i, o, f, g], 0)
    W = reorder(getattr(m, "weight_ih_l0" + sfx)).detach()
    R = reorder(getattr(m, "weight_hh_l0" + sfx)).detach()
    B = torch.cat([reorder(getattr(m, "bias_ih_l0" + sfx)), reorder(getattr(m, "bias_hh_l0" + sfx))]).detach()
    return W, R, B


@pytest.mark.parametrize("direction", ["forward", "reverse", "bidirectional"])
def test_lstm_matches_torch(direction):
    torch.manual_seed(0)
    S, B, I, H = 5, 3, 4, 6
    bi = direction == "bidirectional"
    m = torch.nn.LSTM(I, H, bidirectional=bi)
    x = torch.randn(S, B, I)
    h0, c0 = torch.randn(2 if bi else 1, B, H), torch.randn(2 if bi else 1, B, H)
    if direction == "reverse":
        y_ref, (hn, cn) = m(x.flip(0), (h0, c0))
        y_ref = y_ref.flip(0)
    else:
        y_ref, (hn, cn) = m(x, (h0, c0))
    parts = [_onnx_lstm_weights(m)] + ([_onnx_lstm_weights(m, True)] if bi else [])
    W, R, Bb = (torch.stack([p[k] for p in parts]).numpy() for k in range(3))
    y, yh, yc = run_node("LSTM", {"X": x.numpy(), "W": W, "R": R, "B": Bb, "lens": None, "h0": h0.numpy(), "c0": c0.numpy()},
                         n_outputs=3, hidden_size=H, direction=direction)
    D = 2 if bi else 1
    np.testing.assert_allclose(y, y_ref.detach().reshape(S, B, D, H).permute(0, 2, 1, 3).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(yh, hn.detach().numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(yc, cn.detach().numpy(), rtol=1e-4, atol=1e-5)


def test_gru_and_rnn_match_torch():
    torch.manual_seed(1)
    S, B, I, H = 4, 2, 3, 5
    g = torch.nn.GRU(I, H)
    x = torch.randn(S, B, I)
    y_ref, hn = g(x)
    def reorder(w):   # torch r z n -> ONNX z r h
        r, z, n = w.split(H, 0)
        return torch.cat([z, r, n], 0)
    W, R = reorder(g.weight_ih_l0).detach()[None].numpy(), reorder(g.weight_hh_l0).detach()[None].numpy()
    Bb = torch.cat([reorder(g.bias_ih_l0), reorder(g.bias_hh_l0)]).detach()[None].numpy()
    y, yh = run_node("GRU", {"X": x.numpy(), "W": W, "R": R, "B": Bb}, n_outputs=2, hidden_size=H, linear_before_reset=1)
    np.testing.assert_allclose(y[:, 0], y_ref.detach().numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(yh, hn.detach().numpy(), rtol=1e-4, atol=1e-5)
    r = torch.nn.RNN(I, H)
    y_ref, hn = r(x)
    W, R = r.weight_ih_l0.detach()[None].numpy(), r.weight_hh_l0.detach()[None].numpy()
    Bb = torch.cat([r.bias_ih_l0, r.bias_hh_l0]).detach()[None].numpy()
    y, yh = run_node("RNN", {"X": x.numpy(), "W": W, "R": R, "B": Bb}, n_outputs=2, hidden_size=H)
    np.testing.assert_allclose(y[:, 0], y_ref.detach().numpy(), rtol=1e-4, atol=1e-5)


def test_quantised_linear_ops():
    a = rng.integers(0, 255, (3, 8)).astype(np.uint8)
    b = rng.integers(0, 255, (8, 5)).astype(np.uint8)
    sa, sb, sy = np.float32(0.02), np.float32(0.03), np.float32(0.5)
    za, zb, zy = np.uint8(120), np.uint8(128), np.uint8(100)
    (y,) = run_node("QLinearMatMul", {"a": a, "sa": sa, "za": za, "b": b, "sb": sb, "zb": zb, "sy": sy, "zy": zy})
    real = ((a.astype(np.float32) - 120) * sa) @ ((b.astype(np.float32) - 128) * sb)
    want = np.clip(np.rint(real / sy) + 100, 0, 255).astype(np.uint8)
    assert y.dtype == np.uint8 and np.abs(y.astype(int) - want.astype(int)).max() <= 1
    (f,) = run_node("MatMulIntegerToFloat", {"a": a, "b": b, "sa": sa, "sb": sb, "za": za, "zb": zb}, domain=MS)
    np.testing.assert_allclose(f, real, rtol=1e-5, atol=1e-4)
    (q,) = run_node("QLinearAdd", {"a": a, "sa": sa, "za": za, "b": a, "sb": sb, "zb": zb, "sc": sy, "zc": zy}, domain=MS)
    want = np.clip(np.rint(((a.astype(np.float32) - 120) * sa + (a.astype(np.float32) - 128) * sb) / sy) + 100, 0, 255)
    assert np.abs(q.astype(int) - want.astype(int)).max() <= 1
    x = rng.standard_normal((4, 8)).astype(np.float32)
    w8 = rng.integers(-127, 127, (8, 6)).astype(np.int8)
    ws = (rng.random(6) * 0.05 + 0.01).astype(np.float32)
    (d,) = run_node("DynamicQuantizeMatMul", {"x": x, "b": w8, "bs": ws}, domain=MS)
    ref = x @ (w8.astype(np.float32) * ws)
    assert np.abs(d - ref).max() < 0.05 * np.abs(ref).max() + 0.05


def test_windows_dft_and_pools():
    (h,) = run_node("HannWindow", {"n": np.array(8, np.int64)}, periodic=1)
    np.testing.assert_allclose(h, np.hanning(9)[:8], rtol=1e-5, atol=1e-6)
    (hm,) = run_node("HammingWindow", {"n": np.array(8, np.int64)}, periodic=0)
    np.testing.assert_allclose(hm, 25 / 46 - 21 / 46 * np.cos(2 * np.pi * np.arange(8) / 7), rtol=1e-5, atol=1e-6)
    sig = rng.standard_normal((2, 16, 1)).astype(np.float32)
    (f,) = run_node("DFT", {"x": sig}, axis=1, onesided=1)
    ref = np.fft.rfft(sig[..., 0], axis=1)
    np.testing.assert_allclose(f[..., 0], ref.real, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(f[..., 1], ref.imag, rtol=1e-4, atol=1e-4)
    x = rng.standard_normal((1, 2, 6, 6)).astype(np.float32)
    (lp,) = run_node("LpPool", {"x": x}, kernel_shape=[2, 2], strides=[2, 2], p=2)
    ref = np.sqrt((x.reshape(1, 2, 3, 2, 3, 2) ** 2).sum(axis=(3, 5)))
    np.testing.assert_allclose(lp, ref, rtol=1e-5, atol=1e-6)
    (gl,) = run_node("GlobalLpPool", {"x": x}, p=1)
    np.testing.assert_allclose(gl, np.abs(x).sum(axis=(2, 3), keepdims=True), rtol=1e-5)
    (mvn,) = run_node("MeanVarianceNormalization", {"x": x})
    np.testing.assert_allclose(mvn, (x - x.mean((0, 2, 3), keepdims=True)) / x.std((0, 2, 3), keepdims=True), rtol=1e-4, atol=1e-5)
    m = rng.standard_normal((3, 4, 4)).astype(np.float32)
    (det,) = run_node("Det", {"x": m})
    np.testing.assert_allclose(det, np.linalg.det(m), rtol=1e-4, atol=1e-5)


def test_unique_nms_losses_and_scatter():
    x = np.array([2, 1, 1, 3, 4, 3], np.float32)
    y, idx, inv, cnt = run_node("Unique", {"x": x}, n_outputs=4, sorted=0)
    np.testing.assert_array_equal(y, [2, 1, 3, 4])
    np.testing.assert_array_equal(idx, [0, 1, 3, 4])
    np.testing.assert_array_equal(inv, [0, 1, 1, 2, 3, 2])
    np.testing.assert_array_equal(cnt, [1, 2, 2, 1])
    y, idx, inv, cnt = run_node("Unique", {"x": x}, n_outputs=4, sorted=1)
    np.testing.assert_array_equal(y, [1, 2, 3, 4])
    np.testing.assert_array_equal(idx, [1, 0, 3, 4])
    boxes = np.array([[[0, 0, 1, 1], [0, 0.1, 1, 1.1], [0, -0.1, 1, 0.9], [0, 10, 1, 11], [0, 10.1, 1, 11.1], [0, 100, 1, 101]]], np.float32)
    scores = np.array([[[0.9, 0.75, 0.6, 0.95, 0.5, 0.3]]], np.float32)
    (sel,) = run_node("NonMaxSuppression", {"b": boxes, "s": scores, "m": np.array([3], np.int64), "iou": np.array([0.5], np.float32),
                                            "st": np.array([0.0], np.float32)})
    np.testing.assert_array_equal(sel, [[0, 0, 3], [0, 0, 0], [0, 0, 5]])   # the ONNX specification's example
    logits = rng.standard_normal((4, 5)).astype(np.float32)
    labels = np.array([1, 0, 4, 2], np.int64)
    loss, logp = run_node("SoftmaxCrossEntropyLoss", {"x": logits, "y": labels}, n_outputs=2, reduction="mean")
    ref = torch.nn.functional.cross_entropy(torch.from_numpy(logits), torch.from_numpy(labels))
    np.testing.assert_allclose(loss, ref.numpy(), rtol=1e-5)
    np.testing.assert_allclose(logp, torch.log_softmax(torch.from_numpy(logits), 1).numpy(), rtol=1e-5, atol=1e-6)
    past = np.zeros((2, 1, 4, 2), np.float32)
    upd = np.ones((2, 1, 1, 2), np.float32) * np.array([5, 7], np.float32).reshape(2, 1, 1, 1)
    (out,) = run_node("TensorScatter", {"p": past, "u": upd, "w": np.array([1, 3], np.int64)}, opset=24, axis=-2)
    assert out[0, 0, 1].tolist() == [5, 5] and out[1, 0, 3].tolist() == [7, 7] and out.sum() == 24
    (crop,) = run_node("CenterCropPad", {"x": np.arange(20, dtype=np.float32).reshape(4, 5), "s": np.array([2, 7], np.int64)}, opset=18)
    assert crop.shape == (2, 7) and crop[0, 1] == 5 and crop[0, 0] == 0


def test_quantised_convolutions():
    x = rng.integers(0, 255, (1, 2, 6, 6)).astype(np.uint8)
    w = rng.integers(0, 255, (3, 2, 3, 3)).astype(np.uint8)
    xs, ws, ys = np.float32(0.05), np.array([0.02, 0.03, 0.04], np.float32), np.float32(0.6)
    xz, wz, yz = np.uint8(128), np.uint8(127), np.uint8(110)
    bias = rng.integers(-50, 50, 3).astype(np.int32)
    (y,) = run_node("QLinearConv", {"x": x, "xs": xs, "xz": xz, "w": w, "ws": ws, "wz": wz, "ys": ys, "yz": yz, "b": bias}, pads=[1, 1, 1, 1])
    xf = torch.from_numpy((x.astype(np.float32) - 128) * xs)
    wf = torch.from_numpy((w.astype(np.float32) - 127) * ws.reshape(3, 1, 1, 1))
    ref = torch.nn.functional.conv2d(xf, wf, torch.from_numpy(bias.astype(np.float32) * xs * ws), padding=1).numpy()
    want = np.clip(np.rint(ref / ys) + 110, 0, 255)
    assert y.dtype == np.uint8 and np.abs(y.astype(int) - want.astype(int)).max() <= 1
    (ci,) = run_node("ConvInteger", {"x": x, "w": w, "xz": xz, "wz": wz})
    ref = torch.nn.functional.conv2d(torch.from_numpy(x.astype(np.float64) - 128), torch.from_numpy(w.astype(np.float64) - 127)).numpy()
    np.testing.assert_array_equal(ci, ref.astype(np.int32))


def _bilinear_roialign(img, y, x):
    """One RoiAlign sample on img [C, H, W] following the operator's definition."""
    C, H, W = img.shape
    if y < -1.0 or y > H or x < -1.0 or x > W:
        return np.zeros(C, np.float32), [np.zeros(C, np.float32)] * 4
    y, x = max(y, 0.0), max(x, 0.0)
    y0, x0 = int(y), int(x)
    if y0 >= H - 1:
        y0 = y1 = H - 1
        y = float(y0)
    else:
        y1 = y0 + 1
    if x0 >= W - 1:
        x0 = x1 = W - 1
        x = float(x0)
    else:
        x1 = x0 + 1
    ly, lx = y - y0, x - x0
    parts = [img[:, y0, x0] * (1 - ly) * (1 - lx), img[:, y0, x1] * (1 - ly) * lx, img[:, y1, x0] * ly * (1 - lx), img[:, y1, x1] * ly * lx]
    return sum(parts), parts


@pytest.mark.parametrize("mode", ["avg", "max"])
@pytest.mark.parametrize("sampling_ratio", [2, 0])
def test_roi_align(mode, sampling_ratio):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 3, 10, 12)).astype(np.float32)
    rois = np.array([[1.0, 1.5, 9.0, 8.0], [0.0, 0.0, 23.0, 19.0], [4.2, 3.1, 6.9, 5.5]], np.float32)
    bidx = np.array([0, 1, 1], np.int64)
    oh, ow, scale = 3, 4, 0.5
    (y,) = run_node("RoiAlign", {"x": x, "r": rois, "b": bidx}, opset=16, mode=mode, output_height=oh, output_width=ow,
                    sampling_ratio=sampling_ratio, spatial_scale=scale)
    want = np.zeros((3, 3, oh, ow), np.float32)
    for r in range(3):
        x1, y1, x2, y2 = rois[r] * scale - 0.5
        rw, rh = x2 - x1, y2 - y1
        bh, bw = rh / oh, rw / ow
        gh = sampling_ratio if sampling_ratio > 0 else int(np.ceil(rh / oh))
        gw = sampling_ratio if sampling_ratio > 0 else int(np.ceil(rw / ow))
        gh, gw = max(gh, 1), max(gw, 1)
        for p in range(oh):
            for q in range(ow):
                vals = []
                for i in range(gh):
                    for j in range(gw):
                        s, parts = _bilinear_roialign(x[bidx[r]], y1 + p * bh + (i + 0.5) * bh / gh, x1 + q * bw + (j + 0.5) * bw / gw)
                        vals.append(np.max(parts, 0) if mode == "max" else s)
                want[r, :, p, q] = np.max(vals, 0) if mode == "max" else np.mean(vals, 0)
    np.testing.assert_allclose(y, want, rtol=1e-4, atol=1e-5)


def test_deform_conv_zero_offsets_is_conv_and_random_offsets_match_naive():
    import torch
    rng = np.random.default_rng(12)
    N, C, H, W, M, kh, kw = 1, 4, 6, 7, 6, 3, 3
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = rng.standard_normal((M, C // 2, kh, kw)).astype(np.float32)
    b = rng.standard_normal(M).astype(np.float32)
    oH, oW = H, W
    off = np.zeros((N, 2 * kh * kw * 2, oH, oW), np.float32)
    (y,) = run_node("DeformConv", {"x": x, "w": w, "o": off, "b": b}, opset=19, group=2, offset_group=2, pads=[1, 1, 1, 1], kernel_shape=[kh, kw])
    want = torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), torch.tensor(b), padding=1, groups=2).numpy()
    np.testing.assert_allclose(y, want, rtol=1e-4, atol=1e-4)
    off = rng.uniform(-1.5, 1.5, off.shape).astype(np.float32)
    mask = rng.uniform(0, 1, (N, 2 * kh * kw, oH, oW)).astype(np.float32)
    (y,) = run_node("DeformConv", {"x": x, "w": w, "o": off, "b": b, "m": mask}, opset=19, group=2, offset_group=2, pads=[1, 1, 1, 1], kernel_shape=[kh, kw])

    def sample(img, py, px):   # img [H, W], zero outside, bilinear
        y0, x0 = int(np.floor(py)), int(np.floor(px))
        v = 0.0
        for yy, wy in ((y0, 1 - (py - y0)), (y0 + 1, py - y0)):
            for xx, wx in ((x0, 1 - (px - x0)), (x0 + 1, px - x0)):
                if 0 <= yy < H and 0 <= xx < W:
                    v += img[yy, xx] * wy * wx
        return v
    want = np.zeros((N, M, oH, oW), np.float32)
    cg = C // 2
    for m in range(M):
        g = m // (M // 2)
        for oy in range(oH):
            for ox in range(oW):
                acc = b[m]
                for c in range(C // 2):
                    ch = g * (C // 2) + c
                    ogi = ch // cg
                    for k in range(kh * kw):
                        ky, kx = divmod(k, kw)
                        py = oy - 1 + ky + off[0, (ogi * kh * kw + k) * 2, oy, ox]
                        px = ox - 1 + kx + off[0, (ogi * kh * kw + k) * 2 + 1, oy, ox]
                        acc += w[m, c, ky, kx] * sample(x[0, ch], py, px) * mask[0, ogi * kh * kw + k, oy, ox]
                want[0, m, oy, ox] = acc
    np.testing.assert_allclose(y, want, rtol=1e-3, atol=1e-4)


def test_label_encoder_numeric():
    x = np.array([[3, 7, 5], [9, 3, 1]], np.int64)
    (y,) = run_node("LabelEncoder", {"x": x}, domain="ai.onnx.ml", keys_int64s=[7, 3, 9], values_floats=[0.7, 0.3, 0.9], default_float=-1.0)
    np.testing.assert_allclose(y, [[0.3, 0.7, -1.0], [0.9, 0.3, -1.0]], rtol=1e-6)
    xf = np.array([0.5, 2.0, 1.5], np.float32)
    (z,) = run_node("LabelEncoder", {"x": xf}, domain="ai.onnx.ml", keys_floats=[1.5, 0.5], values_int64s=[15, 5], default_int64=-7)
    np.testing.assert_array_equal(z, [5, -7, 15])


def test_sparse_initializer_and_sparse_to_dense_matmul():
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    A = np.zeros((5, 6), np.float32)
    A[0, 2], A[3, 3], A[4, 0] = 1.5, -2.0, 4.0
    B = rng.standard_normal((6, 3)).astype(np.float32)
    g = ol.make_graph([ol.make_node("SparseToDenseMatMul", ["A", "B"], ["Y"], domain=MS, alpha=0.5)], "g",
                      [ol.make_tensor_value_info("B", ol.TensorProto.FLOAT, [6, 3])], [ol.make_tensor_value_info("Y", ol.TensorProto.FLOAT, None)])
    g.sparse_initializers.append(ol.make_sparse_tensor("A", A))
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(sess.run(None, {"B": B})[0], 0.5 * A @ B, rtol=1e-6)
    # linear-index form of the indices
    sp = ol.SparseTensor(ol.make_tensor("A", np.array([1.5, -2.0, 4.0], np.float32)), ol.make_tensor("", np.array([2, 21, 24], np.int64)), (5, 6))
    g.sparse_initializers[0] = sp
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), providers=["CPUExecutionProvider"])
    np.testing.assert_allclose(sess.run(None, {"B": B})[0], 0.5 * A @ B, rtol=1e-6)


def test_sequence_map_runs_the_body_per_element():
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    body = ol.make_graph([ol.make_node("Mul", ["elem", "scale"], ["scaled"]), ol.make_node("Add", ["scaled", "other"], ["out0"]),
                          ol.make_node("Shape", ["elem"], ["out1"])], "body",
                         [ol.make_tensor_value_info("elem", T.FLOAT, None), ol.make_tensor_value_info("other", T.FLOAT, None)],
                         [ol.make_tensor_value_info("out0", T.FLOAT, None), ol.make_tensor_value_info("out1", T.INT64, None)])
    nodes = [ol.make_node("SplitToSequence", ["x", "split"], ["xs"], axis=0), ol.make_node("SplitToSequence", ["y", "split"], ["ys"], axis=0),
             ol.make_node("SequenceMap", ["xs", "ys"], ["s0", "s1"], body=body),
             ol.make_node("ConcatFromSequence", ["s0"], ["z"], axis=0), ol.make_node("ConcatFromSequence", ["s1"], ["shapes"], axis=0, new_axis=1)]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("x", T.FLOAT, [6, 3]), ol.make_tensor_value_info("y", T.FLOAT, [6, 3])],
                      [ol.make_tensor_value_info("z", T.FLOAT, None), ol.make_tensor_value_info("shapes", T.INT64, None)],
                      [ol.make_tensor("split", np.array([1, 2, 3], np.int64)), ol.make_tensor("scale", np.array(2.0, np.float32))])
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), providers=["CPUExecutionProvider"])
    x, y = rng.standard_normal((6, 3)).astype(np.float32), rng.standard_normal((6, 3)).astype(np.float32)
    z, shapes = sess.run(None, {"x": x, "y": y})
    np.testing.assert_allclose(z, 2 * x + y, rtol=1e-6)
    np.testing.assert_array_equal(shapes, [[1, 3], [2, 3], [3, 3]])


def test_image_decoder_png_and_jpeg():
    import io
    from PIL import Image
    img = (rng.random((9, 7, 3)) * 255).astype(np.uint8)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    png = np.frombuffer(buf.getvalue(), np.uint8).copy()
    (y,) = run_node("ImageDecoder", {"x": png}, opset=20, pixel_format="RGB")
    np.testing.assert_array_equal(y, img)
    (y,) = run_node("ImageDecoder", {"x": png}, opset=20, pixel_format="BGR")
    np.testing.assert_array_equal(y, img[:, :, ::-1])
    (y,) = run_node("ImageDecoder", {"x": png}, opset=20, pixel_format="Grayscale")
    assert y.shape == (9, 7, 1) and y.dtype == np.uint8
    buf = io.BytesIO()
    Image.fromarray(np.full((8, 8, 3), 200, np.uint8)).save(buf, format="JPEG", quality=95)
    (y,) = run_node("ImageDecoder", {"x": np.frombuffer(buf.getvalue(), np.uint8).copy()}, opset=20)
    assert y.shape == (8, 8, 3) and abs(int(y.mean()) - 200) <= 2
