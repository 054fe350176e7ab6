"""QOrdered* operators (ORDER_ROW activations, ORDER_ROW / ORDER_COL weights) against numpy restatements of the
reference's documented semantics (docs/ContribOperators.md; test/contrib_ops/qordered_*_test.cc for the MatMul formula)."""
import numpy as np
import pytest

from helpers import run_node

MS = "com.microsoft"
ROW, COL = 1, 0
rng = np.random.default_rng(3)


def q8(x, s):
    return np.clip(np.rint(x / s), -128, 127).astype(np.int8)


def f32(v):
    return np.array(v, np.float32)


def test_quantize_dequantize_with_order():
    x = (rng.standard_normal((2, 5, 16)) * 3).astype(np.float32)
    (q,) = run_node("QuantizeWithOrder", {"x": x, "s": f32(0.05)}, domain=MS, order_input=ROW, order_output=ROW)
    np.testing.assert_array_equal(q, q8(x, 0.05))
    (d,) = run_node("DequantizeWithOrder", {"q": q, "s": f32(0.05)}, domain=MS, order_input=ROW, order_output=ROW, to=1)
    np.testing.assert_allclose(d, q.astype(np.float32) * 0.05, rtol=1e-6)
    (h,) = run_node("DequantizeWithOrder", {"q": q, "s": f32(0.05)}, domain=MS, order_input=ROW, order_output=ROW, to=10)
    assert h.dtype == np.float16
    with pytest.raises(Exception, match="ORDER_ROW"):
        run_node("QuantizeWithOrder", {"x": x, "s": f32(0.05)}, domain=MS, order_input=ROW, order_output=2)


@pytest.mark.parametrize("order_b", [ROW, COL])
@pytest.mark.parametrize("per_column", [False, True])
def test_qordered_matmul(order_b, per_column):
    Bn, M, K, N = 2, 16, 32, 64
    A = rng.integers(-128, 128, (Bn, M, K)).astype(np.int8)
    Bm = rng.integers(-128, 128, (K, N)).astype(np.int8)             # logical [K, N]
    C = rng.integers(-128, 128, (1, M, N)).astype(np.int8)
    bias = (rng.standard_normal(N) * 2).astype(np.float32)
    sA, sY, sC = 0.02, 0.9, 0.1
    sB = (rng.random(N) * 0.02 + 0.01).astype(np.float32) if per_column else f32(0.015)
    acc = A.astype(np.int64) @ Bm.astype(np.int64)
    ref = np.float32(sA) * sB / np.float32(sY) * acc.astype(np.float32) + bias / np.float32(sY) + np.float32(sC / sY) * C.astype(np.float32)
    ref = np.clip(np.rint(ref), -128, 127).astype(np.int8)
    # ORDER_COL: the declared shape stays [K, N], the buffer holds the matrix column by column
    stored = Bm if order_b == ROW else np.ascontiguousarray(Bm.T).reshape(K, N)
    (y,) = run_node("QOrderedMatMul", {"A": A, "sA": f32(sA), "B": stored, "sB": sB, "sY": f32(sY), "bias": bias, "C": C, "sC": f32(sC)},
                    domain=MS, order_A=ROW, order_B=order_b, order_Y=ROW)
    assert y.dtype == np.int8
    assert np.abs(y.astype(np.int32) - ref.astype(np.int32)).max() <= 1       # ties of the rounding may fall either way
    assert (y != ref).mean() < 0.01


def test_qordered_gelu_and_layernorm():
    import torch
    x = rng.integers(-128, 128, (2, 6, 32)).astype(np.int8)
    (y,) = run_node("QOrderedGelu", {"x": x, "sx": f32(0.03), "sy": f32(0.02)}, domain=MS, order_X=ROW, order_Y=ROW)
    ref = q8(torch.nn.functional.gelu(torch.from_numpy(x.astype(np.float32) * 0.03)).numpy(), 0.02)
    assert np.abs(y.astype(np.int32) - ref.astype(np.int32)).max() <= 1 and (y != ref).mean() < 0.01
    gamma = (rng.random(32) + 0.5).astype(np.float16)
    beta = rng.standard_normal(32).astype(np.float16)
    (z,) = run_node("QOrderedLayerNormalization", {"x": x, "sx": f32(0.03), "g": gamma, "b": beta, "sy": f32(0.025)}, domain=MS,
                    order_X=ROW, order_Y=ROW, axis=-1, epsilon=1e-5)
    xf = torch.from_numpy(x.astype(np.float32) * 0.03)
    ln = torch.nn.functional.layer_norm(xf, (32,), torch.from_numpy(gamma.astype(np.float32)), torch.from_numpy(beta.astype(np.float32)), 1e-5)
    ref = q8(ln.numpy(), 0.025)
    assert np.abs(z.astype(np.int32) - ref.astype(np.int32)).max() <= 1 and (z != ref).mean() < 0.01


def _fake(x, s):
    return np.clip(np.rint(x / s), -128, 127) * s


@pytest.mark.parametrize("order_w", [ROW, COL])
def test_qordered_attention(order_w):
    B, S, hidden, heads = 2, 8, 32, 4
    H = hidden // heads
    x = rng.integers(-128, 128, (B, S, hidden)).astype(np.int8)
    W = [rng.integers(-128, 128, (hidden, hidden)).astype(np.int8) for _ in range(3)]
    bias = [(rng.standard_normal(hidden) * 0.1).astype(np.float32) for _ in range(3)]
    s_in, s_w, s_g = 0.02, 0.004, [0.05, 0.05, 0.04]
    s_qk, s_soft, s_out = 0.08, 1.0 / 127, 0.03
    mask = np.ones((B, S), np.int32)
    mask[1, 6:] = 0
    xf = x.astype(np.float32) * s_in
    q, k, v = (_fake(xf @ (W[i].astype(np.float32) * s_w) + bias[i], s_g[i]).reshape(B, S, heads, H).transpose(0, 2, 1, 3) for i in range(3))
    sc = _fake(q @ k.transpose(0, 1, 3, 2), s_qk) / np.sqrt(H) + np.where(mask[:, None, None, :] == 0, -10000.0, 0.0)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    p = _fake(p / p.sum(-1, keepdims=True), s_soft)
    ref = q8((p @ v).transpose(0, 2, 1, 3).reshape(B, S, hidden), s_out)
    stored = [w if order_w == ROW else np.ascontiguousarray(w.T).reshape(hidden, hidden) for w in W]
    inputs = {"input": x, "scale_input": f32(s_in), "sq": f32(s_g[0]), "sk": f32(s_g[1]), "sv": f32(s_g[2]), "wq": stored[0], "wk": stored[1],
              "wv": stored[2], "swq": f32(s_w), "swk": f32(s_w), "swv": f32(s_w), "bq": bias[0], "bk": bias[1], "bv": bias[2],
              "s_qk": f32(s_qk), "s_soft": f32(s_soft), "s_out": f32(s_out), "mask": mask}
    (y,) = run_node("QOrderedAttention", inputs, domain=MS, num_heads=heads, order_input=ROW, order_output=ROW, order_weight=order_w, unidirectional=0)
    assert y.shape == (B, S, hidden) and y.dtype == np.int8
    diff = np.abs(y.astype(np.int32) - ref.astype(np.int32))
    assert diff.max() <= 2 and (diff > 0).mean() < 0.05


def test_qordered_longformer_attention_matches_float_operator_on_dequantised_inputs():
    B, S, hidden, heads, window = 1, 16, 16, 2, 2
    x = rng.integers(-128, 128, (B, S, hidden)).astype(np.int8)
    W = rng.integers(-128, 128, (hidden, 3 * hidden)).astype(np.int8)
    GW = rng.integers(-128, 128, (hidden, 3 * hidden)).astype(np.int8)
    b = (rng.standard_normal(3 * hidden) * 0.1).astype(np.float32)
    gb = (rng.standard_normal(3 * hidden) * 0.1).astype(np.float32)
    s_in, s_w, s_gw, s_qkv, s_g, s_out = 0.02, 0.004, 0.003, 0.05, 0.05, 0.02
    mask = np.zeros((B, S), np.float32)
    mask[0, 14:] = -10000.0
    glob = np.zeros((B, S), np.int32)
    glob[0, 0] = 1
    (y,) = run_node("QOrderedLongformerAttention",
                    {"input": x, "scale_input": f32(s_in), "weight": W, "scale_weight": f32(s_w), "bias": b, "scale_bias": f32(1.0),
                     "scale_qkv_gemm": f32(s_qkv), "mask": mask, "global_weight": GW, "scale_global_weight": f32(s_gw), "global_bias": gb,
                     "scale_global_gemm": f32(s_g), "global": glob, "scale_output": f32(s_out)},
                    domain=MS, num_heads=heads, window=window, order_input=ROW, order_output=ROW, order_weight=ROW, order_global_weight=ROW)
    # the float operator on weights chosen so that its projections land on the same grids: feed the already
    # fake-quantised projections through identity weights
    xf = x.astype(np.float32) * s_in
    qkv = _fake(xf @ (W.astype(np.float32) * s_w) + b, s_qkv).astype(np.float32)
    gqkv = _fake(xf @ (GW.astype(np.float32) * s_gw) + gb, s_g).astype(np.float32)
    H = hidden // heads
    def heads_of(t, part):
        return t[:, :, part * hidden:(part + 1) * hidden].reshape(B, S, heads, H).transpose(0, 2, 1, 3)
    def attend(t, allowed):
        sc = heads_of(t, 0) @ heads_of(t, 1).transpose(0, 1, 3, 2) / np.sqrt(H) + mask[:, None, None, :]
        sc = np.where(allowed, sc, -np.inf)
        p = np.exp(sc - sc.max(-1, keepdims=True))
        return (p / p.sum(-1, keepdims=True)) @ heads_of(t, 2)
    pos = np.arange(S)
    allowed = (np.abs(pos[:, None] - pos[None, :]) <= window)[None, None] | (glob[:, None, None, :] != 0)
    out = np.where((glob != 0)[:, None, :, None], attend(gqkv, np.ones_like(allowed)), attend(qkv, allowed))
    ref = q8(out.transpose(0, 2, 1, 3).reshape(B, S, hidden), s_out)
    diff = np.abs(y.astype(np.int32) - ref.astype(np.int32))
    assert diff.max() <= 1 and (diff > 0).mean() < 0.02
