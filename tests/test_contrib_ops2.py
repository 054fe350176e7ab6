"""com.microsoft contrib operators of the second batch against numpy / torch restatements of their definitions
(docs/ContribOperators.md of the reference; the reference's own unit tests live under
onnxruntime/test/contrib_ops/)."""
import math

import numpy as np
import pytest
import torch

from helpers import run_node

MS = "com.microsoft"
rng = np.random.default_rng(0)


def test_remove_and_restore_padding():
    B, S, H = 3, 5, 4
    x = rng.standard_normal((B, S, H)).astype(np.float32)
    counts = np.array([2, 5, 1], dtype=np.int32)
    out, off, cum, mx = run_node("RemovePadding", {"x": x, "c": counts}, n_outputs=4, domain=MS)
    want = np.concatenate([x[b, :counts[b]] for b in range(B)])
    np.testing.assert_array_equal(out, want)
    assert off.shape == (B, S) and sorted(off.reshape(-1).tolist()) == list(range(B * S))
    np.testing.assert_array_equal(off.reshape(-1)[:8], [0, 1, 5, 6, 7, 8, 9, 10])
    np.testing.assert_array_equal(cum, [0, 2, 7, 8])
    assert int(mx[0]) == 5
    (back,) = run_node("RestorePadding", {"x": out, "off": off}, domain=MS)
    mask = (np.arange(S)[None, :] < counts[:, None])[..., None]
    np.testing.assert_array_equal(back, x * mask)


@pytest.mark.parametrize("bidirectional", [0, 1])
def test_relative_position_bias_matches_t5_buckets(bidirectional):
    heads, buckets, S, max_distance = 3, 32, 20, 128
    table = rng.standard_normal((heads, buckets)).astype(np.float32)   # memory order: heads outermost

    def bucket(rel):   # T5's _relative_position_bucket, scalar form
        nb, ret = buckets, 0
        if bidirectional:
            nb //= 2
            if rel > 0:
                ret += nb
            n = abs(rel)
        else:
            n = max(-rel, 0)
        max_exact = nb // 2
        if n < max_exact:
            return ret + n
        v = max_exact + int(math.log(n / max_exact) / math.log(max_distance / max_exact) * (nb - max_exact))
        return ret + min(v, nb - 1)
    want = np.zeros((1, heads, S, S), np.float32)
    for q in range(S):
        for k in range(S):
            want[0, :, q, k] = table[:, bucket(k - q)]
    (got,) = run_node("RelativePositionBias", {"t": table.reshape(buckets, heads), "q": np.array([S], np.int64), "k": np.array([S], np.int64)},
                      domain=MS, max_distance=max_distance, is_bidirectional=bidirectional)
    np.testing.assert_allclose(got, want, rtol=0, atol=0)


def test_ngram_repeat_block():
    ids = np.array([[1, 2, 3, 1, 2], [4, 4, 4, 4, 4]], dtype=np.int64)
    scores = np.zeros((2, 6), np.float32)
    (out,) = run_node("NGramRepeatBlock", {"ids": ids, "s": scores}, domain=MS, ngram_size=3)
    # sequence 0 ends with (1, 2): the trigram (1, 2, 3) exists, so 3 is banned; sequence 1: (4, 4) -> 4 banned
    assert np.isneginf(out[0, 3]) and np.isfinite(np.delete(out[0], 3)).all()
    assert np.isneginf(out[1, 4]) and np.isfinite(np.delete(out[1], 4)).all()


def test_skip_group_norm():
    N, H, W, C, G = 2, 3, 3, 8, 4
    x = rng.standard_normal((N, H, W, C)).astype(np.float32)
    skip = rng.standard_normal((N, C)).astype(np.float32)
    bias = rng.standard_normal(C).astype(np.float32)
    gamma, beta = rng.standard_normal(C).astype(np.float32), rng.standard_normal(C).astype(np.float32)
    y, s = run_node("SkipGroupNorm", {"x": x, "g": gamma, "b": beta, "skip": skip, "bias": bias}, n_outputs=2, domain=MS,
                    groups=G, activation=1, epsilon=1e-5, channels_last=1)
    s_ref = x + skip[:, None, None, :] + bias
    t = torch.from_numpy(s_ref).permute(0, 3, 1, 2)
    ref = torch.nn.functional.group_norm(t, G, torch.from_numpy(gamma), torch.from_numpy(beta), 1e-5)
    ref = (ref * torch.sigmoid(ref)).permute(0, 2, 3, 1).numpy()
    np.testing.assert_allclose(s, s_ref, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(y, ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("quant_type", [0, 1])
def test_matmul_bnb4(quant_type):
    fp4 = [0, 0.0052083333, 0.66666667, 1, 0.33333333, 0.5, 0.16666667, 0.25]
    table = np.array(fp4 + [-v for v in fp4], np.float32) if quant_type == 0 else np.array(
        [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334,
         -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
         0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], np.float32)
    N, K, bs = 6, 32, 16
    codes = rng.integers(0, 16, N * K).astype(np.uint8)
    packed = (codes[0::2] << 4 | codes[1::2]).astype(np.uint8)
    absmax = (rng.random(N * K // bs) + 0.5).astype(np.float32)
    w = (table[codes] * np.repeat(absmax, bs)).reshape(N, K)
    a = rng.standard_normal((3, K)).astype(np.float32)
    (y,) = run_node("MatMulBnb4", {"a": a, "b": packed, "m": absmax}, domain=MS, K=K, N=N, block_size=bs, quant_type=quant_type)
    np.testing.assert_allclose(y, a @ w.T, rtol=1e-5, atol=1e-5)


def test_dynamic_time_warping():
    cost = np.array([[1, 9, 9], [1, 9, 9], [9, 1, 1]], np.float32)
    (path,) = run_node("DynamicTimeWarping", {"c": cost}, domain=MS)
    np.testing.assert_array_equal(path, [[0, 1, 2, 2], [0, 0, 1, 2]])


def test_gated_rms_norm_and_gated_add():
    x = rng.standard_normal((2, 3, 8)).astype(np.float32)
    gate = rng.standard_normal((2, 3, 8)).astype(np.float32)
    scale = rng.standard_normal(4).astype(np.float32)
    (y,) = run_node("GatedRMSNorm", {"x": x, "s": scale, "g": gate}, domain=MS, epsilon=1e-6)
    xg = x.reshape(2, 3, 2, 4)
    ref = xg / np.sqrt((xg ** 2).mean(-1, keepdims=True) + 1e-6) * scale * (gate / (1 + np.exp(-gate))).reshape(2, 3, 2, 4)
    np.testing.assert_allclose(y, ref.reshape(2, 3, 8), rtol=1e-5, atol=1e-5)
    g1 = rng.standard_normal((2, 3, 1)).astype(np.float32)
    (z,) = run_node("GatedAdd", {"x": x, "y": gate, "g": g1}, domain=MS)
    np.testing.assert_allclose(z, x + gate * g1, rtol=1e-6, atol=1e-6)


def test_gemma_rotary_embedding():
    B, N, S, D = 1, 2, 3, 4
    emb = rng.standard_normal((B, S, D)).astype(np.float32)
    q, qr, k, kr = (rng.standard_normal((B, N, S, D)).astype(np.float32) for _ in range(4))
    o1, o2 = run_node("GemmaRotaryEmbedding", {"e": emb, "q": q, "qr": qr, "k": k, "kr": kr}, n_outputs=2, domain=MS)
    np.testing.assert_allclose(o1, q * np.cos(emb)[:, None] + qr * np.sin(emb)[:, None], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(o2, k * np.cos(emb)[:, None] + kr * np.sin(emb)[:, None], rtol=1e-5, atol=1e-6)


def test_inference_dropouts_pass_through():
    x = rng.standard_normal((2, 5)).astype(np.float32)
    b = rng.standard_normal(5).astype(np.float32)
    r = rng.standard_normal((2, 5)).astype(np.float32)
    y, m = run_node("BiasDropout", {"x": x, "b": b, "r": r}, n_outputs=2, domain=MS)
    np.testing.assert_allclose(y, x + b + r, rtol=1e-6)
    assert m.dtype == np.bool_ and m.all()
    y2, m2 = run_node("BitmaskDropout", {"x": x}, n_outputs=2, domain=MS)
    np.testing.assert_array_equal(y2, x)
    assert m2.dtype == np.uint32 and m2.tolist() == [(1 << 10) - 1]


def test_unfold_fft_complex():
    x = rng.standard_normal((2, 10)).astype(np.float32)
    (u,) = run_node("UnfoldTensor", {"x": x}, domain=MS, dim=1, size=4, step=3)
    np.testing.assert_array_equal(u, torch.from_numpy(x).unfold(1, 4, 3).numpy())
    sig = rng.standard_normal((3, 16)).astype(np.float32)
    (f,) = run_node("Rfft", {"x": sig}, domain=MS, signal_ndim=1, onesided=1, normalized=0)
    ref = np.fft.rfft(sig)
    np.testing.assert_allclose(f[..., 0], ref.real, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(f[..., 1], ref.imag, rtol=1e-4, atol=1e-4)
    (back,) = run_node("Irfft", {"x": f}, domain=MS, signal_ndim=1, onesided=1, normalized=0)
    np.testing.assert_allclose(back, sig, rtol=1e-4, atol=1e-4)
    a, b = rng.standard_normal((4, 2)).astype(np.float32), rng.standard_normal((4, 2)).astype(np.float32)
    ca, cb = a[:, 0] + 1j * a[:, 1], b[:, 0] + 1j * b[:, 1]
    (m,) = run_node("ComplexMul", {"a": a, "b": b}, domain=MS)
    np.testing.assert_allclose(m[:, 0] + 1j * m[:, 1], ca * cb, rtol=1e-5, atol=1e-6)
    (mc,) = run_node("ComplexMulConj", {"a": a, "b": b}, domain=MS)
    np.testing.assert_allclose(mc[:, 0] + 1j * mc[:, 1], ca * np.conj(cb), rtol=1e-5, atol=1e-6)


def test_block_scaled_fp8_weight_matmul():
    N, K, bs = 8, 256, 128
    w8 = (torch.randn(N, K) * 2).to(torch.float8_e4m3fn)
    scale = (torch.rand(N, K // bs) + 0.5).float()
    a = torch.randn(3, K).to(torch.bfloat16)
    bias = torch.randn(N).to(torch.bfloat16)
    w = (w8.float() * scale.repeat_interleave(bs, 1)).to(torch.bfloat16)
    ref = (a.float() @ w.float().T + bias.float())
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    node = ol.make_node("MatMulBlockQuantizedFp8Weight", ["a", "b", "s", "", "bias"], ["y"], domain=MS, block_size=bs)
    g = ol.make_graph([node], "g", [ol.make_tensor_value_info("a", T.BFLOAT16, [3, K])], [ol.make_tensor_value_info("y", T.BFLOAT16, [3, N])],
                      [ol.make_tensor("b", w8), ol.make_tensor("s", scale), ol.make_tensor("bias", bias)])
    sess = ort.InferenceSession(ol.make_model(g, opset=17).serialize(), providers=["CPUExecutionProvider"])
    (y,) = sess.run(None, {"a": a})
    y = torch.as_tensor(y).float() if not isinstance(y, torch.Tensor) else y.float()
    assert (y - ref).abs().max() / ref.abs().max() < 2e-2


def test_packed_multi_head_attention():
    heads, H = 2, 4
    lens = [1, 3, 2]
    cum = np.cumsum([0] + lens).astype(np.int32)
    Ttot = int(cum[-1])
    q, k, v = (rng.standard_normal((Ttot, heads * H)).astype(np.float32) for _ in range(3))
    off = np.arange(3 * 3, dtype=np.int32).reshape(3, 3)   # not used by the math
    (out,) = run_node("PackedMultiHeadAttention", {"q": q, "k": k, "v": v, "bias": None, "off": off, "cum": cum}, domain=MS, num_heads=heads)
    ref = np.zeros_like(out)
    for b in range(3):
        lo, hi = cum[b], cum[b + 1]
        qb, kb, vb = (torch.from_numpy(t[lo:hi]).reshape(hi - lo, heads, H).transpose(0, 1) for t in (q, k, v))
        o = torch.softmax(qb @ kb.transpose(1, 2) / math.sqrt(H), -1) @ vb
        ref[lo:hi] = o.transpose(0, 1).reshape(hi - lo, heads * H).numpy()
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)


def test_legacy_image_ops():
    x = rng.standard_normal((1, 2, 5, 6)).astype(np.float32)
    (a,) = run_node("Affine", {"x": x}, alpha=2.0, beta=-1.0)
    np.testing.assert_allclose(a, 2 * x - 1, rtol=1e-6)
    (s,) = run_node("ImageScaler", {"x": x}, scale=0.5, bias=[1.0, -1.0])
    np.testing.assert_allclose(s, x * 0.5 + np.array([1.0, -1.0], np.float32).reshape(1, 2, 1, 1), rtol=1e-6)
    (c,) = run_node("Crop", {"x": x}, border=[1, 2, 1, 0])
    np.testing.assert_array_equal(c, x[:, :, 2:5, 1:5])
    (t,) = run_node("ScaledTanh", {"x": x}, alpha=1.5, beta=0.5)
    np.testing.assert_allclose(t, 1.5 * np.tanh(0.5 * x), rtol=1e-5, atol=1e-6)
    (p,) = run_node("ParametricSoftplus", {"x": x}, alpha=1.5, beta=0.5)
    np.testing.assert_allclose(p, 1.5 * np.log1p(np.exp(0.5 * x)), rtol=1e-5, atol=1e-6)
    (d,) = run_node("DynamicSlice", {"x": x, "s": np.array([1, 2], np.int64), "e": np.array([4, 6], np.int64), "ax": np.array([2, 3], np.int64)})
    np.testing.assert_array_equal(d, x[:, :, 1:4, 2:6])


def _gqa(inputs, n_outputs=3, **attrs):
    return run_node("GroupQueryAttention", inputs, n_outputs=n_outputs, domain=MS, num_heads=4, kv_num_heads=2, **attrs)


def test_gqa_quantised_kv_cache_and_qk_norm():
    """int8 KV cache with per-tensor scales: prompt then one decode step track the float-cache run within the
    quantisation error, and the cache comes back as int8 in the shared buffer; q / k norm weights equal to an explicit
    per-head RMS norm applied before the operator."""
    B, S, N, Nk, H, cap = 2, 5, 4, 2, 8, 16
    qkv = rng.standard_normal((B, S, (N + 2 * Nk) * H)).astype(np.float32)
    step = rng.standard_normal((B, 1, (N + 2 * Nk) * H)).astype(np.float32)
    sl0, tot0 = np.full(B, S - 1, np.int32), np.array(S, np.int32)
    sl1, tot1 = np.full(B, S, np.int32), np.array(S + 1, np.int32)
    zeros_f = np.zeros((B, Nk, cap, H), np.float32)
    base = {"q": qkv, "k": None, "v": None, "pk": zeros_f, "pv": zeros_f.copy(), "sl": sl0, "tot": tot0}
    y0, pk, pv = _gqa(base)
    y1, _, _ = _gqa({**base, "q": step, "pk": pk, "pv": pv, "sl": sl1, "tot": tot1})
    ks, vs = np.array([0.03], np.float32), np.array([0.03], np.float32)
    zeros_q = np.zeros((B, Nk, cap, H), np.int8)
    qbase = {"q": qkv, "k": None, "v": None, "pk": zeros_q, "pv": zeros_q.copy(), "sl": sl0, "tot": tot0, "cos": None, "sin": None,
             "pos": None, "bias": None, "sink": None, "ks": ks, "vs": vs}
    q0, qk, qv = _gqa(qbase, k_quant_type="PER_TENSOR", v_quant_type="PER_TENSOR", kv_cache_bit_width=8)
    assert qk.dtype == np.int8 and qk.shape == (B, Nk, cap, H)
    np.testing.assert_allclose(qk[:, :, :S].astype(np.float32) * 0.03, pk[:, :, :S], atol=0.016)
    np.testing.assert_allclose(q0, y0, atol=1e-5)     # the prompt attends to its own unquantised keys
    q1, qk1, _ = _gqa({**qbase, "q": step, "pk": qk, "pv": qv, "sl": sl1, "tot": tot1},
                      k_quant_type="PER_TENSOR", v_quant_type="PER_TENSOR", kv_cache_bit_width=8)
    assert np.abs(q1 - y1).max() < 0.05 and qk1.dtype == np.int8
    # q / k norm
    wq, wk = rng.standard_normal(H).astype(np.float32), rng.standard_normal(H).astype(np.float32)
    def norm(x, heads, w):
        x = x.reshape(B, S, heads, H)
        return (x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6) * w).reshape(B, S, heads * H)
    qn = np.concatenate([norm(qkv[..., :N * H], N, wq), norm(qkv[..., N * H:(N + Nk) * H], Nk, wk), qkv[..., (N + Nk) * H:]], -1)
    want, _, _ = _gqa({**base, "q": qn.astype(np.float32)})
    got, _, _ = _gqa({**base, "cos": None, "sin": None, "pos": None, "bias": None, "sink": None, "ks": None, "vs": None, "qn": wq, "kn": wk},
                     qk_norm_epsilon=1e-6)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
