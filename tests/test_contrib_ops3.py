"""com.microsoft contrib operators of the third batch (fused / channels-last convolutions, QLinear* family, integer
helpers, NVFP4 weight-only MatMul, small utilities) against numpy / torch restatements of their definitions in
docs/ContribOperators.md of the reference."""
import numpy as np
import pytest
import torch

from helpers import run_node

MS = "com.microsoft"
rng = np.random.default_rng(3)


def _q(x, scale, zp, dtype=np.uint8):
    info = np.iinfo(dtype)
    return np.clip(np.rint(x / scale) + zp, info.min, info.max).astype(dtype)


def test_fused_conv_with_residual_and_activation():
    x = rng.standard_normal((2, 3, 8, 8)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    b = rng.standard_normal(4).astype(np.float32)
    z = rng.standard_normal((2, 4, 8, 8)).astype(np.float32)
    (y,) = run_node("FusedConv", {"x": x, "w": w, "b": b, "z": z}, domain=MS, activation="LeakyRelu",
                    activation_params=[0.1], pads=[1, 1, 1, 1], kernel_shape=[3, 3])
    want = torch.nn.functional.leaky_relu(torch.nn.functional.conv2d(torch.tensor(x), torch.tensor(w), torch.tensor(b), padding=1)
                                          + torch.tensor(z), 0.1).numpy()
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)


def test_nhwc_conv_and_nhwc_max_pool():
    x = rng.standard_normal((1, 6, 7, 4)).astype(np.float32)          # N H W C
    w = rng.standard_normal((5, 3, 3, 4)).astype(np.float32)          # M kH kW C
    (y,) = run_node("NhwcConv", {"x": x, "w": w}, domain=MS, pads=[1, 1, 1, 1], strides=[2, 2])
    want = torch.nn.functional.conv2d(torch.tensor(x).permute(0, 3, 1, 2), torch.tensor(w).permute(0, 3, 1, 2),
                                      padding=1, stride=2).permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)
    xq = rng.integers(0, 255, (1, 6, 6, 3)).astype(np.uint8)
    (p,) = run_node("NhwcMaxPool", {"x": xq}, domain=MS, kernel_shape=[2, 2], strides=[2, 2])
    want = xq.reshape(1, 3, 2, 3, 2, 3).max(axis=(2, 4))
    np.testing.assert_array_equal(p, want)


def test_fused_matmul_activation_and_gemm_fast_gelu():
    a = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.standard_normal((4, 5)).astype(np.float32)
    (y,) = run_node("FusedMatMulActivation", {"a": a, "b": b}, domain=MS, activation="Relu", transB=1, alpha=0.5)
    np.testing.assert_allclose(y, np.maximum(0.5 * a @ b.T, 0), rtol=1e-5, atol=1e-6)
    bias = rng.standard_normal(4).astype(np.float32)
    (g,) = run_node("GemmFastGelu", {"x": a, "w": b.T.copy(), "b": bias}, domain=MS)
    v = a @ b.T + bias
    want = 0.5 * v * (1 + np.tanh(0.7978845608 * (v + 0.044715 * v ** 3)))
    np.testing.assert_allclose(g, want, rtol=1e-4, atol=1e-5)


def test_expand_dims_is_all_finite_cdist():
    x = rng.standard_normal((2, 3)).astype(np.float32)
    (y,) = run_node("ExpandDims", {"x": x, "axis": np.array(-1, np.int32)}, domain=MS)
    assert y.shape == (2, 3, 1)
    (ok,) = run_node("IsAllFinite", {"a": x, "b": x}, domain=MS)
    assert bool(ok)
    bad = x.copy()
    bad[0, 0] = np.inf
    assert not bool(run_node("IsAllFinite", {"a": x, "b": bad}, domain=MS)[0])
    assert bool(run_node("IsAllFinite", {"a": bad}, domain=MS, isnan_only=1)[0])
    a = rng.standard_normal((4, 6)).astype(np.float32)
    b = rng.standard_normal((5, 6)).astype(np.float32)
    want = ((a[:, None, :] - b[None, :, :]) ** 2).sum(-1)
    np.testing.assert_allclose(run_node("CDist", {"a": a, "b": b}, domain=MS, metric="sqeuclidean")[0], want, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(run_node("CDist", {"a": a, "b": b}, domain=MS, metric="euclidean")[0], np.sqrt(want), rtol=1e-4, atol=1e-5)


def test_murmur_hash3_known_vectors():
    # x86_32 values for the 4-byte little-endian keys 0, 1, 2 with seed 0 (from the algorithm's definition)
    def ref(key: int, seed: int) -> int:
        def rotl(v, r): return ((v << r) | (v >> (32 - r))) & 0xffffffff
        k = (key * 0xcc9e2d51) & 0xffffffff
        k = rotl(k, 15)
        k = (k * 0x1b873593) & 0xffffffff
        h = seed ^ k
        h = rotl(h, 13)
        h = (h * 5 + 0xe6546b64) & 0xffffffff
        h ^= 4
        h ^= h >> 16
        h = (h * 0x85ebca6b) & 0xffffffff
        h ^= h >> 13
        h = (h * 0xc2b2ae35) & 0xffffffff
        h ^= h >> 16
        return h
    keys = np.array([0, 1, 2, 123456], np.int32)
    (h,) = run_node("MurmurHash3", {"x": keys}, domain=MS, seed=7, positive=1)
    assert [int(v) for v in h] == [ref(int(k), 7) for k in keys]
    (s,) = run_node("MurmurHash3", {"x": keys}, domain=MS, seed=7, positive=0)
    assert [int(v) & 0xffffffff for v in s] == [ref(int(k), 7) for k in keys]


def test_maxpool_with_mask_stops_at_masked_position():
    x = np.array([[[1.0, 5.0, 3.0, 9.0, 2.0, 8.0]]], np.float32)
    m = np.array([[[1, 1, 1, 0, 1, 1]]], np.int32)
    (y,) = run_node("MaxpoolWithMask", {"x": x, "m": m}, domain=MS, kernel_shape=[3], strides=[3])
    np.testing.assert_array_equal(y, [[[5.0, np.finfo(np.float32).min]]])   # second window starts on a masked element


def test_crop_and_resize_bilinear_identity_box():
    x = rng.standard_normal((2, 3, 5, 7)).astype(np.float32)
    rois = np.array([[0, 0, 1, 1], [0, 0, 1, 1]], np.float32)
    idx = np.array([1, 0], np.int32)
    (y,) = run_node("CropAndResize", {"x": x, "r": rois, "i": idx, "c": np.array([5, 7], np.int32)}, domain=MS, mode="bilinear")
    np.testing.assert_allclose(y, x[[1, 0]], rtol=1e-5, atol=1e-5)
    rois = np.array([[0.25, 0.0, 1.5, 1.0]], np.float32)    # reaches below the image: extrapolation value
    (z,) = run_node("CropAndResize", {"x": x, "r": rois, "i": np.array([0], np.int32), "c": np.array([3, 7], np.int32)},
                    domain=MS, mode="nearest", extrapolation_value=-1.0)
    assert np.all(z[0, :, 2, :] == -1.0) and np.allclose(z[0, :, 0, :], x[0, :, 1, :])


def test_qlinear_pools_concat_softmax_reduce_where():
    x = rng.uniform(-2, 2, (1, 2, 4, 4)).astype(np.float32)
    xs, xz, ys, yz = np.float32(0.02), np.uint8(120), np.float32(0.015), np.uint8(100)
    xq = _q(x, xs, xz)
    xd = (xq.astype(np.float32) - xz) * xs
    (p,) = run_node("QLinearAveragePool", {"x": xq, "xs": xs, "xz": xz, "ys": ys, "yz": yz}, domain=MS, kernel_shape=[2, 2], strides=[2, 2])
    np.testing.assert_array_equal(p, _q(xd.reshape(1, 2, 2, 2, 2, 2).mean(axis=(3, 5)), ys, yz))
    (g,) = run_node("QLinearGlobalAveragePool", {"x": xq.transpose(0, 2, 3, 1).copy(), "xs": xs, "xz": xz, "ys": ys, "yz": yz}, domain=MS, channels_last=1)
    np.testing.assert_array_equal(g, _q(xd.mean(axis=(2, 3), keepdims=True), ys, yz).transpose(0, 2, 3, 1))
    (c,) = run_node("QLinearConcat", {"ys": ys, "yz": yz, "a": xq, "as": xs, "az": xz, "b": xq, "bs": xs, "bz": xz}, domain=MS, axis=1)
    np.testing.assert_array_equal(c, _q(np.concatenate([xd, xd], 1), ys, yz))
    sm_s, sm_z = np.float32(1 / 256), np.uint8(0)
    (s,) = run_node("QLinearSoftmax", {"x": xq, "xs": xs, "xz": xz, "ys": sm_s, "yz": sm_z}, domain=MS, axis=-1, opset=13)
    e = np.exp(xd - xd.max(-1, keepdims=True))
    assert np.abs(s.astype(np.int32) - _q(e / e.sum(-1, keepdims=True), sm_s, sm_z).astype(np.int32)).max() <= 1
    (r,) = run_node("QLinearReduceMean", {"x": xq, "xs": xs, "xz": xz, "ys": ys, "yz": yz}, domain=MS, axes=[1], keepdims=0)
    np.testing.assert_array_equal(r, _q(xd.mean(1), ys, yz))
    cond = rng.integers(0, 2, x.shape).astype(bool)
    (w,) = run_node("QLinearWhere", {"c": cond, "x": xq, "xs": xs, "xz": xz, "y": xq[::-1].copy(), "ys2": ys, "yz2": yz, "zs": ys, "zz": yz}, domain=MS)
    yd = (xq[::-1].astype(np.float32) - yz) * ys
    np.testing.assert_array_equal(w, _q(np.where(cond, xd, yd), ys, yz))


def test_integer_helpers():
    a = rng.integers(0, 255, (3, 4)).astype(np.uint8)
    b = rng.integers(-128, 127, (4,)).astype(np.int8)
    (m,) = run_node("MulInteger", {"a": a, "az": np.uint8(3), "b": b, "bz": np.int8(-2)}, domain=MS)
    np.testing.assert_array_equal(m, (a.astype(np.int32) - 3) * (b.astype(np.int32) + 2))
    (s,) = run_node("ReduceSumInteger", {"a": a}, domain=MS, axes=[1], keepdims=0)
    np.testing.assert_array_equal(s, a.astype(np.int32).sum(1))
    x16 = rng.integers(-30000, 30000, (3, 6)).astype(np.int16)
    y16 = rng.integers(-300, 300, (6, 2)).astype(np.int16)
    (mm,) = run_node("MatMulInteger16", {"a": x16, "b": y16}, domain=MS)
    np.testing.assert_array_equal(mm, x16.astype(np.int64) @ y16.astype(np.int64))


def test_matmul_block_quantized_fp4_weight():
    N, K, block = 6, 32, 16
    lut = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    nib = rng.integers(0, 16, (N, K)).astype(np.uint8)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    sc = torch.tensor(rng.uniform(0.5, 2.0, (N, K // block)).astype(np.float32)).to(torch.float8_e4m3fn)
    sc_bytes = sc.view(torch.uint8).numpy()
    g = np.array(0.25, np.float32)
    w = lut[nib] * np.repeat(sc.float().numpy(), block, 1) * g
    a = rng.standard_normal((3, K)).astype(np.float16)
    bias = rng.standard_normal(N).astype(np.float16)
    (y,) = run_node("MatMulBlockQuantizedFp4Weight", {"a": a, "b": packed, "s": sc_bytes, "g": g, "in_scale": None, "bias": bias}, domain=MS, block_size=block)
    np.testing.assert_allclose(y.astype(np.float32), a.astype(np.float32) @ w.T + bias.astype(np.float32), rtol=2e-3, atol=2e-2)


def test_dynamic_quantize_lstm_matches_float_lstm_on_dequantised_weights():
    S, B, I, H = 4, 2, 3, 5
    x = rng.standard_normal((S, B, I)).astype(np.float32)
    wq = rng.integers(-100, 100, (1, I, 4 * H)).astype(np.int8)
    rq = rng.integers(-100, 100, (1, H, 4 * H)).astype(np.int8)
    ws, rs = np.array([0.01], np.float32), np.array([0.02], np.float32)
    wz, rz = np.array([0], np.int8), np.array([0], np.int8)
    bias = rng.standard_normal((1, 8 * H)).astype(np.float32)
    y, yh, yc = run_node("DynamicQuantizeLSTM", {"x": x, "w": wq, "r": rq, "b": bias, "sl": None, "h0": None, "c0": None, "p": None,
                                                   "ws": ws, "wz": wz, "rs": rs, "rz": rz}, n_outputs=3, domain=MS, hidden_size=H)
    w = (wq.astype(np.float32) * ws[0]).transpose(0, 2, 1).copy()
    r = (rq.astype(np.float32) * rs[0]).transpose(0, 2, 1).copy()
    y2, yh2, yc2 = run_node("LSTM", {"x": x, "w": w, "r": r, "b": bias}, n_outputs=3, hidden_size=H)
    np.testing.assert_allclose(y, y2, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(yc, yc2, rtol=1e-5, atol=1e-6)
