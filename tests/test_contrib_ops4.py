"""com.microsoft contrib operators of the fourth batch (decoder-masked attentions, LongformerAttention,
SparseAttention, GatedRelativePositionBias, MRotaryEmbedding, linear-attention family, QAttention) against numpy
restatements of the definitions in docs/ContribOperators.md of the reference."""
import numpy as np
import pytest

from helpers import run_node

MS = "com.microsoft"
rng = np.random.default_rng(4)


def _softmax(x, axis=-1):
    e = np.exp(x - x.max(axis, keepdims=True))
    return e / e.sum(axis, keepdims=True)


def test_decoder_masked_mha_self_attention_with_shared_cache_and_beams():
    batch, beam, N, H, cap, past = 2, 2, 2, 4, 8, 3
    B = batch * beam
    q = rng.standard_normal((B, 1, N * H)).astype(np.float32)
    k = rng.standard_normal((B, 1, N * H)).astype(np.float32)
    v = rng.standard_normal((B, 1, N * H)).astype(np.float32)
    pk = rng.standard_normal((B, N, cap, H)).astype(np.float32)
    pv = rng.standard_normal((B, N, cap, H)).astype(np.float32)
    ind = rng.integers(0, beam, (batch, beam, cap)).astype(np.int32)
    mask = np.ones((B, past + 1), np.int32)
    mask[1, 0] = 0
    out, nk, nv = run_node("DecoderMaskedMultiHeadAttention",
                           {"q": q, "k": k, "v": v, "mask": mask, "ab": None, "pk": pk, "pv": pv, "pl": np.array([past], np.int32),
                            "bw": np.array([beam], np.int32), "ci": ind}, n_outputs=3, domain=MS, num_heads=N, past_present_share_buffer=1)
    want = np.zeros((B, 1, N * H), np.float32)
    for r in range(B):
        b, j = divmod(r, beam)
        for h in range(N):
            keys = np.stack([pk[b * beam + ind[b, j, t], h, t] for t in range(past)] + [k[r, 0, h * H:(h + 1) * H]])
            vals = np.stack([pv[b * beam + ind[b, j, t], h, t] for t in range(past)] + [v[r, 0, h * H:(h + 1) * H]])
            s = keys @ q[r, 0, h * H:(h + 1) * H] / np.sqrt(H) + np.where(mask[r] != 0, 0.0, -10000.0)
            want[r, 0, h * H:(h + 1) * H] = _softmax(s) @ vals
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(nk[:, :, past], k.reshape(B, N, H), rtol=0, atol=0)
    np.testing.assert_array_equal(nk[:, :, :past], pk[:, :, :past])
    np.testing.assert_allclose(nv[:, :, past], v.reshape(B, N, H), rtol=0, atol=0)


def test_decoder_masked_mha_cross_attention_and_qk_output():
    B, N, H, L = 2, 2, 4, 5
    q = rng.standard_normal((B, 1, N * H)).astype(np.float32)
    k = rng.standard_normal((B, N, L, H)).astype(np.float32)
    v = rng.standard_normal((B, N, L, H)).astype(np.float32)
    out, _, _, qk = run_node("DecoderMaskedMultiHeadAttention", {"q": q, "k": k, "v": v}, n_outputs=4, domain=MS, num_heads=N, output_qk=1)
    s = np.einsum("bnh,bnlh->bnl", q.reshape(B, N, H), k) / np.sqrt(H)
    np.testing.assert_allclose(qk.reshape(B, N, L), s, rtol=1e-4, atol=1e-5)
    want = np.einsum("bnl,bnlh->bnh", _softmax(s), v).reshape(B, 1, N * H)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)


def test_decoder_masked_self_attention_matches_attention_with_past():
    B, N, H, past = 2, 2, 4, 3
    hidden = N * H
    x = rng.standard_normal((B, 1, hidden)).astype(np.float32)
    w = (rng.standard_normal((hidden, 3 * hidden)) * 0.3).astype(np.float32)
    b = rng.standard_normal(3 * hidden).astype(np.float32)
    pst = rng.standard_normal((2, B, N, past, H)).astype(np.float32)
    out, present = run_node("DecoderMaskedSelfAttention", {"x": x, "w": w, "b": b, "m": None, "past": pst}, n_outputs=2, domain=MS, num_heads=N)
    ref, ref_present = run_node("Attention", {"x": x, "w": w, "b": b, "m": None, "past": pst}, n_outputs=2, domain=MS, num_heads=N, unidirectional=1)
    np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(present, ref_present, rtol=1e-5, atol=1e-6)


def test_longformer_attention_dense_restatement():
    B, S, N, H, w = 1, 12, 2, 4, 2
    hidden = N * H
    x = rng.standard_normal((B, S, hidden)).astype(np.float32)
    W = (rng.standard_normal((hidden, 3 * hidden)) * 0.3).astype(np.float32)
    bias = rng.standard_normal(3 * hidden).astype(np.float32)
    GW = (rng.standard_normal((hidden, 3 * hidden)) * 0.3).astype(np.float32)
    gb = rng.standard_normal(3 * hidden).astype(np.float32)
    mask = np.zeros((B, S), np.float32)
    mask[0, -2:] = -10000.0
    glob = np.zeros((B, S), np.int32)
    glob[0, 0] = 1
    (out,) = run_node("LongformerAttention", {"x": x, "w": W, "b": bias, "m": mask, "gw": GW, "gb": gb, "g": glob}, domain=MS, num_heads=N, window=w)
    qkv, gqkv = x @ W + bias, x @ GW + gb
    want = np.zeros((B, S, hidden), np.float32)
    for h in range(N):
        sl = lambda t, part: t[0, :, part * hidden + h * H: part * hidden + (h + 1) * H]
        for i in range(S):
            if glob[0, i]:
                s = sl(gqkv, 1) @ sl(gqkv, 0)[i] / np.sqrt(H) + mask[0]
                want[0, i, h * H:(h + 1) * H] = _softmax(s) @ sl(gqkv, 2)
            else:
                allowed = (np.abs(np.arange(S) - i) <= w) | (glob[0] != 0)
                s = np.where(allowed, sl(qkv, 1) @ sl(qkv, 0)[i] / np.sqrt(H) + mask[0], -np.inf)
                want[0, i, h * H:(h + 1) * H] = _softmax(s) @ sl(qkv, 2)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)


def test_gated_relative_position_bias():
    B, S, N, H, D = 2, 5, 3, 4, 8
    q = rng.standard_normal((B, S, N * H)).astype(np.float32)
    qb = rng.standard_normal(N * H).astype(np.float32)
    rel = rng.standard_normal((1, N, S, S)).astype(np.float32)
    w = rng.standard_normal((H, D)).astype(np.float32)
    b = rng.standard_normal(D).astype(np.float32)
    eco = rng.standard_normal((1, N, 1, 1)).astype(np.float32)
    (out,) = run_node("GatedRelativePositionBias", {"q": q, "qb": qb, "rel": rel, "w": w, "b": b, "eco": eco}, domain=MS, num_heads=N)
    ql = (q + qb).reshape(B, S, N, H).transpose(0, 2, 1, 3)
    g = 1 / (1 + np.exp(-((ql @ w + b).reshape(B, N, S, 2, D // 2).sum(-1))))
    gate = g[..., 0] * (g[..., 1] * eco.reshape(1, N, 1) - 1.0) + 2.0
    np.testing.assert_allclose(out, gate[..., None] * rel, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("layout", [0, 1])
def test_mrotary_embedding_sections(layout):
    B, S, N, H = 1, 6, 2, 8
    half, sec = H // 2, [2, 1, 1]
    x = rng.standard_normal((B, S, N * H)).astype(np.float32)
    pos = rng.integers(0, 16, (3, B, S)).astype(np.int64)
    ang = np.arange(16)[:, None] * (1.0 / 10000 ** (np.arange(half) / half))[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    (out,) = run_node("MRotaryEmbedding", {"x": x, "p": pos, "c": cos, "s": sin}, domain=MS, mrope_section=sec, mrope_layout=layout, num_heads=N)
    if layout == 0:
        stream = [0] * sec[0] + [1] * sec[1] + [2] * sec[2]
    else:
        stream = [0] * half
        for d in range(1, min(half, sec[1] * 3), 3):
            stream[d] = 1
        for d in range(2, min(half, sec[2] * 3), 3):
            stream[d] = 2
    want = np.zeros((B, S, N, H), np.float32)
    xs = x.reshape(B, S, N, H)
    for s in range(S):
        c = np.array([cos[pos[stream[d], 0, s], d] for d in range(half)])
        sn = np.array([sin[pos[stream[d], 0, s], d] for d in range(half)])
        a, b = xs[0, s, :, :half], xs[0, s, :, half:]
        want[0, s] = np.concatenate([a * c - b * sn, b * c + a * sn], -1)
    np.testing.assert_allclose(out, want.reshape(B, S, N * H), rtol=1e-5, atol=1e-5)


def test_causal_conv_with_state_chunked_equals_whole():
    B, C, L, k = 2, 3, 7, 4
    x = rng.standard_normal((B, C, L)).astype(np.float32)
    w = rng.standard_normal((C, 1, k)).astype(np.float32)
    b = rng.standard_normal(C).astype(np.float32)
    y, st = run_node("CausalConvWithState", {"x": x, "w": w, "b": b}, n_outputs=2, domain=MS, activation="silu")
    xp = np.concatenate([np.zeros((B, C, k - 1), np.float32), x], 2)
    pre = np.stack([(xp[:, :, t:t + k] * w[None, :, 0]).sum(-1) + b for t in range(L)], -1)
    np.testing.assert_allclose(y, pre / (1 + np.exp(-pre)), rtol=1e-4, atol=1e-5)
    np.testing.assert_array_equal(st, xp[:, :, -(k - 1):])
    y1, s1 = run_node("CausalConvWithState", {"x": x[:, :, :4].copy(), "w": w, "b": b}, n_outputs=2, domain=MS, activation="silu")
    y2, s2 = run_node("CausalConvWithState", {"x": x[:, :, 4:].copy(), "w": w, "b": b, "p": s1}, n_outputs=2, domain=MS, activation="silu")
    np.testing.assert_allclose(np.concatenate([y1, y2], 2), y, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(s2, st, rtol=0, atol=0)
    _, sw = run_node("CausalConvWithState", {"x": x, "w": w, "b": b}, n_outputs=2, domain=MS, state_window=2)
    assert sw.shape == (2, B, C, k - 1)
    np.testing.assert_array_equal(sw[1], st)
    np.testing.assert_array_equal(sw[0], xp[:, :, L - 2 + 1: L - 2 + k])


@pytest.mark.parametrize("rule", ["linear", "gated", "delta", "gated_delta"])
def test_linear_attention_recurrence(rule):
    B, T, Hq, Hkv, dk, dv = 2, 5, 4, 2, 3, 4
    q = rng.standard_normal((B, T, Hq * dk)).astype(np.float32)
    k = rng.standard_normal((B, T, Hkv * dk)).astype(np.float32)
    k /= np.linalg.norm(k.reshape(B, T, Hkv, dk), axis=-1, keepdims=True).repeat(dk, -1).reshape(B, T, Hkv * dk)
    v = rng.standard_normal((B, T, Hkv * dv)).astype(np.float32)
    past = rng.standard_normal((B, Hkv, dk, dv)).astype(np.float32)
    decay = -np.abs(rng.standard_normal((B, T, Hkv))).astype(np.float32)
    beta = rng.uniform(0, 1, (B, T, Hkv)).astype(np.float32)
    feeds = {"q": q, "k": k, "v": v, "past": past,
             "decay": decay if "gated" in rule else None, "beta": beta if "delta" in rule else None}
    out, state = run_node("LinearAttention", feeds, n_outputs=2, domain=MS, q_num_heads=Hq, kv_num_heads=Hkv, update_rule=rule)
    S = past.astype(np.float64).copy()
    want = np.zeros((B, T, Hq, dv))
    for t in range(T):
        kt, vt = k[:, t].reshape(B, Hkv, dk), v[:, t].reshape(B, Hkv, dv)
        if "gated" in rule:
            S = S * np.exp(decay[:, t])[:, :, None, None]
        if "delta" in rule:
            pred = np.einsum("bhkv,bhk->bhv", S, kt)
            S = S + beta[:, t][:, :, None, None] * kt[..., None] * (vt - pred)[:, :, None, :]
        else:
            S = S + kt[..., None] * vt[:, :, None, :]
        qt = q[:, t].reshape(B, Hq, dk)
        want[:, t] = np.einsum("bhk,bhkv->bhv", qt, np.repeat(S, Hq // Hkv, 1)) / np.sqrt(dk)
    np.testing.assert_allclose(out, want.reshape(B, T, Hq * dv), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(state, S, rtol=1e-4, atol=1e-4)


def test_linear_attention_gate():
    a = rng.standard_normal((2, 3, 4)).astype(np.float16)
    b = rng.standard_normal((2, 3, 4)).astype(np.float16)
    dt = rng.standard_normal(4).astype(np.float32)
    sc = -np.exp(rng.standard_normal(4)).astype(np.float32)
    decay, beta = run_node("LinearAttentionGate", {"a": a, "dt": dt, "sc": sc, "b": b}, n_outputs=2, domain=MS)
    z = a.astype(np.float32) + dt
    np.testing.assert_allclose(decay.astype(np.float32), sc * np.log1p(np.exp(z)), rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(beta.astype(np.float32), 1 / (1 + np.exp(-b.astype(np.float32))), rtol=2e-3, atol=2e-3)


def test_sparse_attention_block_layout():
    B, S, N, Nk, H, bs, blocks = 1, 8, 2, 1, 4, 2, 4
    q = rng.standard_normal((B, S, N * H)).astype(np.float32)
    k = rng.standard_normal((B, S, Nk * H)).astype(np.float32)
    v = rng.standard_normal((B, S, Nk * H)).astype(np.float32)
    cache = np.zeros((B, Nk, blocks * bs, H), np.float32)
    layout = np.array([[[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 1, 1, 1]],
                       [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 0, 1, 1]]], bool)
    rows = np.array([[0, 1, 3, 5, 8], [0, 1, 3, 6, 9]], np.int32)
    cols = np.array([[0, 0, 1, 1, 2, 1, 2, 3, -1], [0, 0, 1, 0, 1, 2, 0, 2, 3]], np.int32)
    out, pk, pv = run_node("SparseAttention", {"q": q, "k": k, "v": v, "pk": cache, "pv": cache.copy(), "r": rows, "c": cols,
                                                "t": np.array([S], np.int32), "kl": np.array([S], np.int32)},
                           n_outputs=3, domain=MS, num_heads=N, kv_num_heads=Nk, sparse_block_size=bs)
    want = np.zeros((B, S, N, H), np.float32)
    for h in range(N):
        for i in range(S):
            ok = np.array([j <= i and layout[h % 2, i // bs, j // bs] for j in range(S)])
            s = np.where(ok, k[0].reshape(S, H) @ q[0, i, h * H:(h + 1) * H] / np.sqrt(H), -np.inf)
            want[0, i, h] = _softmax(s) @ v[0].reshape(S, H)
    np.testing.assert_allclose(out, want.reshape(B, S, N * H), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(pk[0, 0, :S], k[0], rtol=0, atol=0)


def test_qattention_matches_float_attention_on_dequantised_operands():
    B, S, N, H = 2, 4, 2, 4
    hidden = N * H
    xs, ws = np.float32(0.05), np.float32(0.02)
    xq = rng.integers(0, 255, (B, S, hidden)).astype(np.uint8)
    wq = rng.integers(-127, 127, (hidden, 3 * hidden)).astype(np.int8)
    bias = rng.standard_normal(3 * hidden).astype(np.float32)
    mask = np.array([4, 2], np.int32)
    (out,) = run_node("QAttention", {"x": xq, "w": wq, "b": bias, "xs": xs, "ws": ws, "m": mask, "xz": np.uint8(128), "wz": np.int8(0)},
                      domain=MS, num_heads=N)
    x = (xq.astype(np.float32) - 128) * xs
    w = wq.astype(np.float32) * ws
    (ref,) = run_node("Attention", {"x": x, "w": w, "b": bias, "m": mask}, domain=MS, num_heads=N)
    np.testing.assert_allclose(out, ref, rtol=1e-3, atol=1e-3)


def _quant4(w, block=32):
    """Symmetric-zero-point (8) 4-bit block quantisation in the MatMulNBits layout: B [N, blocks, block / 2], scales [N, blocks]."""
    N, K = w.shape
    blocks = K // block
    wb = w.reshape(N, blocks, block)
    scales = (np.abs(wb).max(-1) / 7.0).astype(np.float32)
    q = np.clip(np.rint(wb / scales[..., None]) + 8, 0, 15).astype(np.uint8)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)
    deq = (q.astype(np.float32) - 8) * scales[..., None]
    return packed, scales, deq.reshape(N, K)


def test_matmul_nbits_mlp_and_qkv_with_rms_norm():
    T, K, N = 3, 64, 32
    a = rng.standard_normal((T, K)).astype(np.float32)
    skip = rng.standard_normal((T, K)).astype(np.float32)
    gamma = rng.standard_normal(K).astype(np.float32)
    gB, gs, gw = _quant4(rng.standard_normal((N, K)).astype(np.float32))
    uB, us, uw = _quant4(rng.standard_normal((N, K)).astype(np.float32))
    gb = rng.standard_normal(N).astype(np.float32)
    y, ssum = run_node("MatMulNBitsMlp", {"a": a, "skip": skip, "g": gamma, "gB": gB, "gs": gs, "gb": gb, "uB": uB, "us": us, "ub": None},
                       n_outputs=2, domain=MS, K=K, N=N, bits=4, block_size=32, activation="silu", epsilon=1e-5)
    x = a + skip
    xn = x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-5) * gamma
    gate = xn @ gw.T + gb
    np.testing.assert_allclose(y, gate / (1 + np.exp(-gate)) * (xn @ uw.T), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(ssum, x, rtol=1e-6, atol=1e-6)
    Nq, Nkv = 32, 16
    qB, qs, qw = _quant4(rng.standard_normal((Nq, K)).astype(np.float32))
    kB, ks, kw = _quant4(rng.standard_normal((Nkv, K)).astype(np.float32))
    vB, vs, vw = _quant4(rng.standard_normal((Nkv, K)).astype(np.float32))
    q, k, v = run_node("MatMulNBitsQkv", {"a": a, "skip": None, "g": gamma, "qB": qB, "qs": qs, "qb": None, "kB": kB, "ks": ks, "kb": None,
                                          "vB": vB, "vs": vs, "vb": None}, n_outputs=3, domain=MS, K=K, Nq=Nq, Nkv=Nkv, bits=4, block_size=32)
    an = a / np.sqrt((a ** 2).mean(-1, keepdims=True) + 1e-5) * gamma
    np.testing.assert_allclose(q, an @ qw.T, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(k, an @ kw.T, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(v, an @ vw.T, rtol=1e-4, atol=1e-4)


def test_decoder_attention_self_then_cached_step():
    S, B, N, H = 3, 2, 2, 4
    hidden = N * H
    x = rng.standard_normal((S, B, hidden)).astype(np.float32)
    qw = (rng.standard_normal((hidden, hidden)) * 0.3).astype(np.float32)
    kvw = (rng.standard_normal((hidden, 2 * hidden)) * 0.3).astype(np.float32)
    bias = rng.standard_normal(3 * hidden).astype(np.float32)
    f, t = np.array(False), np.array(True)
    out, kc, vc = run_node("DecoderAttention", {"q": x, "k": x, "qw": qw, "kvw": kvw, "b": bias, "m": None, "kc": None, "vc": None,
                                                "static_kv": f, "use_past": f, "has_layer_state": f, "has_mask": f}, n_outputs=3, domain=MS, num_heads=N)

    def heads(z):
        return z.reshape(z.shape[0], B, N, H).transpose(1, 2, 0, 3)
    q = heads(x @ qw + bias[:hidden])
    kv = x @ kvw + bias[hidden:]
    k, v = heads(kv[..., :hidden]), heads(kv[..., hidden:])
    want = (_softmax(q @ k.transpose(0, 1, 3, 2) / np.sqrt(H)) @ v).transpose(2, 0, 1, 3).reshape(S, B, hidden)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(kc, k, rtol=1e-5, atol=1e-6)
    x1 = rng.standard_normal((1, B, hidden)).astype(np.float32)
    out1, kc1, _ = run_node("DecoderAttention", {"q": x1, "k": x1, "qw": qw, "kvw": kvw, "b": bias, "m": None, "kc": kc, "vc": vc,
                                                 "static_kv": f, "use_past": t, "has_layer_state": t, "has_mask": f}, n_outputs=3, domain=MS, num_heads=N)
    assert kc1.shape == (B, N, S + 1, H)
    q1 = heads(x1 @ qw + bias[:hidden])
    kv1 = x1 @ kvw + bias[hidden:]
    k1 = np.concatenate([k, heads(kv1[..., :hidden])], 2)
    v1 = np.concatenate([v, heads(kv1[..., hidden:])], 2)
    want1 = (_softmax(q1 @ k1.transpose(0, 1, 3, 2) / np.sqrt(H)) @ v1).transpose(2, 0, 1, 3).reshape(1, B, hidden)
    np.testing.assert_allclose(out1, want1, rtol=1e-4, atol=1e-5)


def test_bifurcation_detector():
    src = np.array([10, 11, 12, 13, 14, 15, 11, 20], np.int64)
    cur = np.array([1, 2], np.int64)
    pred = np.array([12, 13, 99, 15, 11, 20, 7], np.int64)     # leaves the source at index 2 (prev = 2)
    tokens, idx = run_node("BifurcationDetector", {"s": src, "c": cur, "p": np.array([2], np.int64), "pred": pred},
                           n_outputs=2, domain=MS, min_ngram_size=1, max_ngram_size=3)
    np.testing.assert_array_equal(tokens, [1, 2, 12, 13, 99])
    assert int(idx[0]) == -1                                    # 99 does not occur in the source
    tokens, idx = run_node("BifurcationDetector", {"s": src, "c": np.array([5, 13, 14], np.int64), "p": np.array([0], np.int64)},
                           n_outputs=2, domain=MS, min_ngram_size=1, max_ngram_size=3)
    np.testing.assert_array_equal(tokens, [5, 13, 14])
    assert int(idx[0]) == 5                                     # "13 14" is unique in the source and ends before index 5
    _, idx = run_node("BifurcationDetector", {"s": src, "c": np.array([11], np.int64), "p": np.array([0], np.int64)},
                      n_outputs=2, domain=MS, min_ngram_size=1, max_ngram_size=3)
    assert int(idx[0]) == -1                                    # 11 occurs twice


def test_word_conv_embedding_reference_vectors():
    """Inputs and expected outputs of the reference's own test (onnxruntime/test/contrib_ops/word_conv_embedding_test.cc)."""
    import numpy as np
    import pytest
    from helpers import run_node
    seq = np.array([[1, 2, 3, 4, 0], [4, 3, 2, 1, 0]], np.int32)
    C = np.array([[0.1, 0.2, 0.3], [0.2, 0.3, 0.1], [0.3, 0.1, 0.2], [0.4, 0.5, 0.6], [0.7, 0.8, 0.9]], np.float32)
    W = np.array([0.1, 0.2, 0.3, 0.2, 0.3, 0.1, 0.3, 0.1, 0.2, 1.0, 1.1, 1.2], np.float32).reshape(2, 1, 2, 3)
    B = np.array([0.1, 0.2], np.float32)
    (y,) = run_node("WordConvEmbedding", {"Sequence": seq, "W": W, "B": B, "C": C}, domain="com.microsoft")
    np.testing.assert_allclose(y, [[0.711393774, 0.996334076], [0.711393774, 0.981612563]], rtol=1e-5)
    (y,) = run_node("WordConvEmbedding", {"Sequence": seq, "W": W, "B": B, "C": C}, domain="com.microsoft", embedding_size=2, conv_window_size=2,
                    char_embedding_size=3)
    assert y.shape == (2, 2)
    with pytest.raises(Exception, match="embedding_size"):
        run_node("WordConvEmbedding", {"Sequence": seq, "W": W, "B": B, "C": C}, domain="com.microsoft", embedding_size=3)
    # an id outside the character table counts as padding: one window over (char 1, zero vector)
    (y,) = run_node("WordConvEmbedding", {"Sequence": np.array([[1, 99]], np.int32), "W": np.ones((1, 1, 2, 1), np.float32), "B": np.zeros(1, np.float32),
                                          "C": np.array([[123.0], [2.0]], np.float32)}, domain="com.microsoft")
    np.testing.assert_allclose(y, [[np.tanh(2.0)]], rtol=1e-6)
    with pytest.raises(Exception, match="must not exceed word length"):
        run_node("WordConvEmbedding", {"Sequence": np.array([[1, 2]], np.int32), "W": np.ones((1, 1, 3, 1), np.float32), "B": np.zeros(1, np.float32),
                                       "C": np.array([[0.0], [1.0], [2.0]], np.float32)}, domain="com.microsoft")


def test_contrib_aliases_of_onnx_operators_and_unique():
    import numpy as np
    from helpers import run_node
    MS = "com.microsoft"
    (r,) = run_node("Range", {"s": np.array(1.0, np.float32), "l": np.array(4.0, np.float32), "d": np.array(0.5, np.float32)}, domain=MS)
    np.testing.assert_allclose(r, np.arange(1.0, 4.0, 0.5, dtype=np.float32))
    data = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    (g,) = run_node("GatherND", {"data": data, "idx": np.array([[0, 1], [1, 2]], np.int64)}, domain=MS)
    np.testing.assert_array_equal(g, data[[0, 1], [1, 2]])
    (p,) = run_node("Pad", {"x": np.ones((2, 2), np.float32), "pads": np.array([0, 1, 0, 1], np.int64), "v": np.array(7.0, np.float32)}, domain=MS, mode="constant")
    np.testing.assert_array_equal(p, [[7, 1, 1, 7], [7, 1, 1, 7]])
    y, idx, counts = run_node("Unique", {"x": np.array([5, 2, 5, 9, 2, 5], np.int64)}, n_outputs=3, domain=MS)
    np.testing.assert_array_equal(y, [5, 2, 9])
    np.testing.assert_array_equal(idx, [0, 1, 0, 2, 1, 0])
    np.testing.assert_array_equal(counts, [3, 2, 1])


def test_attn_lstm_against_a_numpy_restatement():
    """AttnLSTM (LSTM cell wrapped by Bahdanau attention) against the documented equations, forward and bidirectional,
    with sequence lengths, memory lengths, peepholes and the attention layer."""
    import numpy as np
    from helpers import run_node
    rng = np.random.RandomState(0)
    S, B, I, H, steps, depth, att, aw = 5, 3, 4, 6, 7, 5, 8, 3

    def sig(x):
        return 1 / (1 + np.exp(-x))

    def run_dir(X, W, R, Bb, P, QW, MW, V, M, mlens, AW, lens, reverse):
        mask = np.arange(steps)[None, :] < mlens[:, None]
        values = M * mask[..., None]
        keys = values @ MW
        h, c = np.zeros((B, H)), np.zeros((B, H))
        attn = np.zeros((B, AW.shape[1]))
        Y = np.zeros((S, B, H))
        bias = Bb[:4 * H] + Bb[4 * H:]
        for step in range(S):
            for b in range(B):
                if step >= lens[b]:
                    continue
                t = lens[b] - 1 - step if reverse else step
                g = np.concatenate([X[t, b], attn[b]]) @ W.T + h[b] @ R.T + bias
                gi, go, gf, gc = g[:H], g[H:2 * H], g[2 * H:3 * H], g[3 * H:]
                it, ft = sig(gi + P[:H] * c[b]), sig(gf + P[2 * H:] * c[b])
                cn = ft * c[b] + it * np.tanh(gc)
                hn = sig(go + P[H:2 * H] * cn) * np.tanh(cn)
                score = (np.tanh(keys[b] + hn @ QW) * V).sum(-1)
                score = np.where(mask[b], score, -np.inf)
                al = np.exp(score - score.max())
                al = al / al.sum()
                attn[b] = np.concatenate([hn, al @ values[b]]) @ AW
                h[b], c[b] = hn, cn
                Y[t, b] = hn
        return Y, h, c

    for direction, D in (("forward", 1), ("bidirectional", 2)):
        X = rng.randn(S, B, I)
        W, R, Bb = rng.randn(D, 4 * H, I + aw) * 0.3, rng.randn(D, 4 * H, H) * 0.3, rng.randn(D, 8 * H) * 0.1
        P, QW, MW, V = rng.randn(D, 3 * H) * 0.2, rng.randn(D, H, att) * 0.3, rng.randn(D, depth, att) * 0.3, rng.randn(D, att)
        M, AW = rng.randn(B, steps, depth), rng.randn(D, depth + H, aw) * 0.3
        lens, mlens = np.array([5, 3, 4], np.int32), np.array([7, 4, 6], np.int32)
        f = lambda a: a.astype(np.float32)
        y, yh, yc = run_node("AttnLSTM", {"X": f(X), "W": f(W), "R": f(R), "B": f(Bb), "sequence_lens": lens, "initial_h": None, "initial_c": None,
                                          "P": f(P), "QW": f(QW), "MW": f(MW), "V": f(V), "M": f(M), "memory_seq_lens": mlens, "AW": f(AW)},
                             n_outputs=3, domain="com.microsoft", hidden_size=H, direction=direction)
        assert y.shape == (S, D, B, H)
        for d in range(D):
            Y, hl, cl = run_dir(X, W[d], R[d], Bb[d], P[d], QW[d], MW[d], V[d], M, mlens, AW[d], lens, reverse=(d == 1))
            np.testing.assert_allclose(y[:, d], Y, rtol=2e-4, atol=2e-5)
            np.testing.assert_allclose(yh[d], hl, rtol=2e-4, atol=2e-5)
            np.testing.assert_allclose(yc[d], cl, rtol=2e-4, atol=2e-5)
