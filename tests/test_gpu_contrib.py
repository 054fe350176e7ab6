"""GPU kernels behind the quantised / paged / encoder-attention contrib ops: kernel-level numerics against PyTorch
fp32 references, and session-level runs (GPU provider with fallback disabled) against the CPU provider."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from onnxruntime_b200.ops import _kernels
    _kernels.lib()
    return _kernels


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


def _quantize(N, Kd, bits, bs, dtype, zp_mode, seed=0):
    """Random block-quantised weights in the MatMulNBits layout plus their fp32 expansion."""
    g = torch.Generator().manual_seed(seed)
    nb = (Kd + bs - 1) // bs
    q = torch.randint(0, 1 << bits, (N, nb, bs), generator=g)
    scales = (torch.rand(N, nb, generator=g) * 0.02 + 0.005).to(dtype)
    if zp_mode == "none":
        zp_vals = torch.full((N, nb), 1 << (bits - 1))
        zp = None
    else:
        zp_vals = torch.randint(0, 1 << bits, (N, nb), generator=g)
        if zp_mode == "packed":
            if bits == 4:
                z = torch.nn.functional.pad(zp_vals, (0, nb % 2))
                zp = (z[:, 0::2] | (z[:, 1::2] << 4)).to(torch.uint8)
            else:
                zp = zp_vals.to(torch.uint8)
        else:
            zp = zp_vals.to(dtype)
    w = ((q - zp_vals.unsqueeze(-1)).float() * scales.float().unsqueeze(-1)).reshape(N, nb * bs)[:, :Kd]
    if bits == 4:
        B = (q[:, :, 0::2] | (q[:, :, 1::2] << 4)).to(torch.uint8)
    else:
        B = q.to(torch.uint8)
    return B, scales, zp, w


@pytest.mark.parametrize("bits,bs", [(4, 32), (4, 128), (8, 32), (4, 16)])
@pytest.mark.parametrize("zp_mode", ["none", "packed", "typed"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_nbits_dequant(K, bits, bs, zp_mode, dtype):
    N, Kd = 300, 1000 if bs == 32 else 1024
    B, scales, zp, w = _quantize(N, Kd, bits, bs, dtype, zp_mode)
    out = K.nbits_dequant(B.cuda(), scales.cuda(), None if zp is None else zp.cuda(), N, Kd, bits, bs)
    assert torch.equal(out.cpu(), w.to(dtype))


@pytest.mark.parametrize("H,N,Nk", [(128, 8, 2), (64, 4, 4)])
@pytest.mark.parametrize("block_size", [16, 64])
def test_paged_decode_matches_dense(K, H, N, Nk, block_size):
    torch.manual_seed(0)
    B, max_len = 3, 500
    max_blocks = (max_len + block_size - 1) // block_size
    num_blocks = B * max_blocks + 5
    past = torch.tensor([0, 137, 499], dtype=torch.int32, device="cuda")
    perm = torch.randperm(num_blocks)[:B * max_blocks].reshape(B, max_blocks).to(torch.int32).cuda()
    kc = torch.randn(num_blocks, block_size, Nk, H, device="cuda").bfloat16()
    vc = torch.randn(num_blocks, block_size, Nk, H, device="cuda").bfloat16()
    qkv = torch.randn(B, (N + 2 * Nk) * H, device="cuda").bfloat16()
    half = H // 2
    pos = torch.arange(1024, device="cuda").float().unsqueeze(1)
    inv = 1.0 / (10000 ** (torch.arange(half, device="cuda").float() / half))
    cos, sin = torch.cos(pos * inv).bfloat16(), torch.sin(pos * inv).bfloat16()
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc0, vc0 = kc.clone(), vc.clone()
    q_rot = K.paged_prep(qkv, kc, vc, cu, past, perm, N, Nk, cos, sin, status=status)
    out = K.gqa_decode(q_rot, kc, vc, past, block_table=perm)
    torch.cuda.synchronize()
    assert status.item() == 0

    def rope(x, p):  # x [heads, H]
        c, s = cos[p].float(), sin[p].float()
        x1, x2 = x[:, :half].float(), x[:, half:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    for b in range(B):
        p = int(past[b])
        q = rope(qkv[b, :N * H].view(N, H), p).bfloat16().float()
        k_new = rope(qkv[b, N * H:(N + Nk) * H].view(Nk, H), p).bfloat16()
        v_new = qkv[b, (N + Nk) * H:].view(Nk, H)
        blk, off = int(perm[b, p // block_size]), p % block_size
        assert torch.equal(kc[blk, off], k_new) and torch.equal(vc[blk, off], v_new)
        L = p + 1
        keys = torch.stack([kc[int(perm[b, j // block_size]), j % block_size] for j in range(L)]).float()   # L,Nk,H
        vals = torch.stack([vc[int(perm[b, j // block_size]), j % block_size] for j in range(L)]).float()
        keys = keys.repeat_interleave(N // Nk, 1)
        vals = vals.repeat_interleave(N // Nk, 1)
        s = torch.einsum("nh,lnh->nl", q, keys) / math.sqrt(H)
        ref = torch.einsum("nl,lnh->nh", torch.softmax(s, -1), vals)
        assert _rel(out[b].view(N, H), ref) < 2e-2, b
    # nothing but the B new slots was written
    changed = (kc != kc0).any(-1).any(-1).sum().item()
    assert changed <= B


def test_attn_prefill_key_mask(K):
    torch.manual_seed(0)
    B, S, N, H = 2, 300, 4, 64
    q = torch.randn(B, S, N, H, device="cuda").half()
    k = torch.randn(B, S, N, H, device="cuda").half()
    v = torch.randn(B, S, N, H, device="cuda").half()
    mask = (torch.rand(B, S, device="cuda") > 0.3).int()
    mask[:, 0] = 1
    out = K.attn_prefill(q, k, v, None, first_prompt=True, causal=False, kv_layout="bsnh", key_mask=mask)
    s = torch.einsum("bsnh,btnh->bnst", q.float(), k.float()) / math.sqrt(H)
    ref = torch.einsum("bnst,btnh->bsnh", torch.softmax(s.masked_fill(mask.view(B, 1, 1, S) == 0, float("-inf")), -1), v.float())
    assert _rel(out, ref) < 2e-2


# ------------------------------------------------------------------------------------------ session level
def _both(op, inputs, initializers=(), n_outputs=1, **attrs):
    """Run a one-node com.microsoft model on the CPU provider and on the GPU provider (fallback disabled)."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    names = list(inputs)
    node = ol.make_node(op, [n if inputs[n] is not None else "" for n in names], [f"o{i}" for i in range(n_outputs)],
                        domain="com.microsoft", **attrs)
    gin, inits = [], []
    for n in names:
        v = inputs[n]
        if v is None:
            continue
        if n in initializers:
            inits.append(ol.make_tensor(n, v))
        else:
            gin.append(ol.make_tensor_value_info(n, ol.np_dtype_to_onnx(v.dtype), list(v.shape)))
    model = ol.make_model(ol.make_graph([node], "g", gin, [ol.make_tensor_value_info(f"o{i}", 0, None) for i in range(n_outputs)], inits)).serialize()
    feeds = {n: inputs[n] for n in names if inputs[n] is not None and n not in initializers}
    cpu = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    gpu = ort.InferenceSession(model, providers=["CUDAExecutionProvider"], enable_fallback=False)
    assert {n["ep"] for n in gpu.graph_nodes() if n["op_type"] == op} == {"CUDAExecutionProvider"}
    before = gpu.kernel_launch_count()
    rc = cpu.run(None, feeds)
    rg = gpu.run(None, feeds)
    gpu.check_device_status()
    assert gpu.kernel_launch_count() > before, "the sm_100a kernel did not run"
    return rc, rg


def _np16(t):
    return t.view(torch.int16).numpy().view(np.float16) if t.dtype == torch.float16 else t


@pytest.mark.parametrize("M", [1, 8, 200])
def test_session_matmul_nbits(M):
    N, Kd, bs = 512, 1024, 32
    B, scales, zp, w = _quantize(N, Kd, 4, bs, torch.float16, "packed", seed=3)
    a = (torch.randn(2, M, Kd) * 0.5).half()
    rc, rg = _both("MatMulNBits", {"a": a.numpy(), "B": B.numpy(), "scales": scales.numpy(), "zp": zp.numpy(), "g": None,
                                   "bias": torch.randn(N).half().numpy()}, initializers=("B", "scales", "zp", "bias"),
                   K=Kd, N=N, bits=4, block_size=bs)
    ref = a.float() @ w.half().float().T
    assert np.abs(rg[0].astype(np.float32) - rc[0].astype(np.float32)).max() / np.abs(rc[0].astype(np.float32)).max() < 1e-2
    assert rg[0].shape == (2, M, N) and np.isfinite(rg[0].astype(np.float32)).all()
    assert ref.shape == (2, M, N)


@pytest.mark.parametrize("mask", ["none", "lengths", "raw"])
def test_session_bert_attention(mask):
    torch.manual_seed(0)
    B, S, N, H = 2, 200, 4, 64
    W = N * H
    x = (torch.randn(B, S, W) * 0.5).half()
    w = (torch.randn(W, 3 * W) * 0.05).half()
    b = (torch.randn(3 * W) * 0.1).half()
    m = None
    if mask == "lengths":
        m = np.array([200, 77], dtype=np.int32)
    elif mask == "raw":
        m = (np.random.RandomState(0).rand(B, S) > 0.3).astype(np.int32)
        m[:, 0] = 1
    rc, rg = _both("Attention", {"x": x.numpy(), "w": w.numpy(), "b": b.numpy(), "mask": m}, initializers=("w", "b"), num_heads=N)
    c, g = rc[0].astype(np.float32), rg[0].astype(np.float32)
    assert np.abs(c - g).max() / np.abs(c).max() < 2e-2


def test_session_multihead_attention_packed_and_separate():
    torch.manual_seed(0)
    B, S, N, H = 2, 160, 4, 64
    qkv = (torch.randn(B, S, N, 3, H) * 0.5).half()
    rc, rg = _both("MultiHeadAttention", {"q": qkv.numpy()}, num_heads=N)
    c, g = rc[0].astype(np.float32), rg[0].astype(np.float32)
    assert np.abs(c - g).max() / np.abs(c).max() < 2e-2
    q = (torch.randn(B, S, N * H) * 0.5).half()
    k = (torch.randn(B, 96, N * H) * 0.5).half()
    v = (torch.randn(B, 96, N * H) * 0.5).half()
    rc, rg = _both("MultiHeadAttention", {"q": q.numpy(), "k": k.numpy(), "v": v.numpy()}, num_heads=N)
    c, g = rc[0].astype(np.float32), rg[0].astype(np.float32)
    assert np.abs(c - g).max() / np.abs(c).max() < 2e-2


def test_session_paged_attention_decode():
    import onnxruntime_b200 as ort
    torch.manual_seed(0)
    B, N, Nk, H, bsz, max_blocks = 3, 8, 2, 128, 16, 8
    num_blocks = 40
    qkv = (torch.randn(B, (N + 2 * Nk) * H) * 0.5).half()
    kc = (torch.randn(num_blocks, bsz, Nk, H) * 0.5).half()
    vc = (torch.randn(num_blocks, bsz, Nk, H) * 0.5).half()
    table = torch.randperm(num_blocks)[:B * max_blocks].reshape(B, max_blocks).to(torch.int32)
    past = torch.tensor([5, 100, 64], dtype=torch.int32)
    cu = torch.arange(B + 1, dtype=torch.int32)
    half = H // 2
    pos = torch.arange(256).float().unsqueeze(1)
    inv = 1.0 / (10000 ** (torch.arange(half).float() / half))
    cos, sin = torch.cos(pos * inv).half(), torch.sin(pos * inv).half()
    rc, rg = _both("PagedAttention", {"q": qkv.numpy(), "k": None, "v": None, "kc": kc.numpy(), "vc": vc.numpy(), "cu": cu.numpy(),
                                      "past": past.numpy(), "table": table.numpy(), "cos": cos.numpy(), "sin": sin.numpy()},
                   n_outputs=3, initializers=("cos", "sin"), num_heads=N, kv_num_heads=Nk, do_rotary=1)
    for i in range(3):
        c, g = rc[i].astype(np.float32), rg[i].astype(np.float32)
        assert np.abs(c - g).max() / np.abs(c).max() < 2e-2, i


@pytest.mark.parametrize("T,E,k,act,fc3,bias", [(1, 8, 2, "silu", True, False), (16, 8, 2, "silu", True, False),
                                                (300, 8, 2, "silu", True, False), (64, 64, 4, "relu", False, True),
                                                (40, 16, 1, "gelu", False, False), (2048, 8, 2, "silu", True, False),
                                                (33, 6, 3, "identity", False, True)])
def test_session_moe(T, E, k, act, fc3, bias):
    torch.manual_seed(0)
    H, I = 256, 512
    x = (torch.randn(T, H) * 0.5).half()
    # distinct values per row, so that the choice of experts does not hinge on how ties are broken
    logits = (torch.argsort(torch.rand(T, E), dim=1).float() * 0.37 - 1.0).half()
    fc1 = (torch.randn(E, I, H) * 0.05).half()
    fc2 = (torch.randn(E, H, I) * 0.05).half()
    inputs = {"x": x.numpy(), "router": logits.numpy(), "fc1": fc1.numpy(), "b1": (torch.randn(E, I) * 0.1).half().numpy() if bias else None,
              "fc2": fc2.numpy(), "b2": (torch.randn(E, H) * 0.1).half().numpy() if bias else None}
    inits = ["fc1", "fc2", "b1", "b2"]
    if fc3:
        inputs["fc3"] = (torch.randn(E, I, H) * 0.05).half().numpy()
        inits.append("fc3")
    rc, rg = _both("MoE", inputs, initializers=inits, k=k, activation_type=act, normalize_routing_weights=1)
    c, g = rc[0].astype(np.float32), rg[0].astype(np.float32)
    assert np.isfinite(g).all()
    assert np.abs(c - g).max() / np.abs(c).max() < 2e-2


@pytest.mark.parametrize("M,N,Kd", [(8, 256, 512), (200, 1024, 1024), (1024, 2048, 4096), (130, 384, 144),
                                    (4096, 4096, 512), (2500, 3000, 1040)])   # the last two run on CTA pairs (kind::f8f6f4, cta_group::2)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_gemm_fp8_operands(K, M, N, Kd, out_dtype):
    torch.manual_seed(0)
    x = (torch.randn(M, Kd, device="cuda") * 0.5).to(torch.float8_e4m3fn)
    w = (torch.randn(N, Kd, device="cuda") * 0.5).to(torch.float8_e4m3fn)
    b = torch.randn(N, device="cuda").to(out_dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = K.gemm(x, w, bias=b, alpha=0.125, out_dtype=out_dtype, status=status)
    assert status.item() == 0
    ref = 0.125 * (x.float() @ w.float().T) + b.float()
    assert _rel(y, ref) < 1e-2


def test_session_gemm_float8():
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    torch.manual_seed(0)
    M, Kd, N = 64, 512, 384
    a16 = (torch.randn(M, Kd) * 0.5).half()
    w8 = (torch.randn(N, Kd) * 0.5).to(torch.float8_e4m3fn)
    nodes = [ol.make_node("Cast", ["a"], ["a8"], to=T.FLOAT8E4M3FN, saturate=1),
             ol.make_node("GemmFloat8", ["a8", "w", "", "sa", "sb"], ["y"], domain="com.microsoft", transB=1, dtype=T.FLOAT16, alpha=2.0)]
    g = ol.make_graph(nodes, "g", [ol.make_tensor_value_info("a", T.FLOAT16, [M, Kd])], [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                      [ol.make_tensor("w", w8), ol.make_tensor("sa", np.array([0.5], np.float32)), ol.make_tensor("sb", np.array([0.25], np.float32))])
    model = ol.make_model(g).serialize()
    so = ort.SessionOptions()
    so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    cpu = ort.InferenceSession(model, so, providers=["CPUExecutionProvider"])
    gpu = ort.InferenceSession(model, so, providers=["CUDAExecutionProvider"], enable_fallback=False)
    before = gpu.kernel_launch_count()
    c = cpu.run(None, {"a": a16.numpy()})[0].astype(np.float32)
    gq = gpu.run(None, {"a": a16.numpy()})[0].astype(np.float32)
    assert gpu.kernel_launch_count() > before
    ref = 2.0 * 0.5 * 0.25 * (a16.to(torch.float8_e4m3fn).float() @ w8.float().T)
    assert np.abs(gq - ref.numpy()).max() / np.abs(ref.numpy()).max() < 1e-2
    assert np.abs(c - ref.numpy()).max() / np.abs(ref.numpy()).max() < 1e-2


@pytest.mark.parametrize("M,N,Kd,bs", [(1, 512, 1024, 32), (8, 1280, 8192, 32), (33, 384, 2048, 64), (64, 1000, 1024, 128), (8, 4096, 4096, 32)])
@pytest.mark.parametrize("zp_mode", ["none", "packed"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_q4_in_kernel_expansion(K, M, N, Kd, bs, zp_mode, dtype):
    """Decode GEMM on 4-bit block-quantised weights: the kernel expands the nibbles in shared memory.  The result
    must match the GEMM on the explicitly dequantised weights (same rounding of the weights to 16 bits)."""
    B, scales, zp, w = _quantize(N, Kd, 4, bs, dtype, zp_mode, seed=5)
    zp_bytes = None
    if zp is not None:
        z = zp.to(torch.int32)
        zp_bytes = torch.stack([z & 0xF, (z >> 4) & 0xF], -1).reshape(N, -1)[:, :(Kd + bs - 1) // bs].to(torch.uint8).contiguous().cuda()
    blobs = K.nbits_build_blobs(B.cuda(), scales.cuda(), zp_bytes, N, Kd, bs)
    assert blobs.shape == ((N + 127) // 128, Kd // 64, 4864) and blobs.dtype == torch.uint8
    x = (torch.randn(M, Kd, device="cuda") * 0.5).to(dtype)
    bias = torch.randn(N, device="cuda").to(dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = K.gemm(x, blobs, bias=bias, n=N, q4=True, status=status)
    assert status.item() == 0
    ref = x.float() @ w.to(dtype).float().cuda().T + bias.float()
    assert _rel(y, ref) < 1e-2
    dense = K.gemm(x, K.nbits_dequant(B.cuda(), scales.cuda(), None if zp is None else zp.cuda(), N, Kd, 4, bs), bias=bias)
    assert _rel(y, dense) < 4e-3


@pytest.mark.parametrize("bits,block", [(4, 0), (4, 32)])
def test_session_qmoe(bits, block):
    """QMoE on the GPU provider (weights expanded once at session creation, then the grouped-GEMM MoE path)."""
    import sys
    sys.path.insert(0, __import__("os").path.dirname(__file__))
    from test_ops_cpu import _qmoe_case
    x, logits, (p1, s1, _), (p2, s2, _), (p3, s3, _) = _qmoe_case(bits, block, E=8, H=256, I=512, T=40, dtype=np.float16)
    rc, rg = _both("QMoE", {"x": x, "r": logits, "w1": p1, "s1": s1, "b1": None, "w2": p2, "s2": s2, "b2": None, "w3": p3, "s3": s3},
                   initializers=("w1", "s1", "w2", "s2", "w3", "s3"), k=2, activation_type="silu", normalize_routing_weights=1,
                   expert_weight_bits=bits, block_size=block)
    c, g = rc[0].astype(np.float32), rg[0].astype(np.float32)
    assert np.abs(c - g).max() / np.abs(c).max() < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N", [512, 500])
def test_block_scaled_fp8_weight_matmul_on_gpu(dtype, N):
    """MatMulBlockQuantizedFp8Weight: decode-shaped calls keep the weight in fp8 and expand it inside the tcgen05 decode
    GEMM (tensor-memory operand); larger ones use a 16-bit copy made once.  Both against the dequantised product."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    torch.manual_seed(0)
    K, bs = 1024, 128
    w8 = (torch.randn(N, K) * 2).to(torch.float8_e4m3fn)
    w8.view(torch.uint8)[:, :16] = torch.arange(16, dtype=torch.uint8)      # zero, the seven subnormals and small normals
    w8.view(torch.uint8)[:, 16:32] = torch.arange(16, dtype=torch.uint8) + 0x80
    scale = (torch.rand(N, K // bs) + 0.5).float() * 0.02
    bias = torch.randn(N).to(dtype)
    et = T.BFLOAT16 if dtype == torch.bfloat16 else T.FLOAT16
    node = ol.make_node("MatMulBlockQuantizedFp8Weight", ["a", "b", "s", "", "bias"], ["y"], domain="com.microsoft", block_size=bs)
    g = ol.make_graph([node], "g", [ol.make_tensor_value_info("a", et, ["m", K])], [ol.make_tensor_value_info("y", et, ["m", N])],
                      [ol.make_tensor("b", w8), ol.make_tensor("s", scale), ol.make_tensor("bias", bias)])
    model = ol.make_model(g, opset=17).serialize()
    sess = ort.InferenceSession(model, providers=["CUDAExecutionProvider"], enable_fallback=False)
    so = ort.SessionOptions()
    so.add_session_config_entry("ortb200.fp8_weight_in_kernel", "0")
    copy16 = ort.InferenceSession(model, so, providers=["CUDAExecutionProvider"], enable_fallback=False)
    w = (w8.float() * scale.repeat_interleave(bs, 1)).to(dtype).float()
    for m in (1, 8, 40, 300):
        a = torch.randn(m, K).to(dtype)
        before = sess.kernel_launch_count()
        y = torch.as_tensor(sess.run(None, {"a": a.cuda()})[0]).float().cpu()
        assert sess.kernel_launch_count() == before + 1
        ref = a.float() @ w.T + bias.float()
        assert (y - ref).abs().max() / ref.abs().max() < 1e-2, m
        y16 = torch.as_tensor(copy16.run(None, {"a": a.cuda()})[0]).float().cpu()
        assert (y - y16).abs().max() / ref.abs().max() < 1e-2, m
    sess.check_device_status()


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("with_segment", [True, False])
def test_embed_layer_normalization_kernel(dtype, with_segment):
    rng = np.random.default_rng(3)
    B, S, H, V = 3, 7, 256, 50
    ids = rng.integers(0, V, (B, S)).astype(np.int32)
    seg = rng.integers(0, 2, (B, S)).astype(np.int32)
    word = rng.standard_normal((V, H)).astype(dtype)
    pos = rng.standard_normal((16, H)).astype(dtype)
    segt = rng.standard_normal((2, H)).astype(dtype)
    gamma, beta = rng.standard_normal(H).astype(dtype), rng.standard_normal(H).astype(dtype)
    mask = (np.arange(S)[None, :] < np.array([7, 3, 5])[:, None]).astype(np.int32)
    inputs = {"ids": ids, "seg": seg if with_segment else None, "word": word, "pos": pos, "segt": segt if with_segment else None,
              "gamma": gamma, "beta": beta, "mask": mask}
    rc, rg = _both("EmbedLayerNormalization", inputs, initializers=("word", "pos", "segt", "gamma", "beta"), n_outputs=3, epsilon=1e-5)
    tol = 2e-2 if dtype == np.float16 else 1e-4
    np.testing.assert_allclose(np.asarray(rg[0], dtype=np.float32), np.asarray(rc[0], dtype=np.float32), rtol=tol, atol=tol)
    np.testing.assert_array_equal(rg[1], [7, 3, 5])
    np.testing.assert_allclose(np.asarray(rg[2], dtype=np.float32), np.asarray(rc[2], dtype=np.float32), rtol=tol, atol=tol)


def test_session_gemm_float8_with_runtime_scales_needs_no_host_read():
    """Scales that arrive as run-time inputs stay on the device: the kernel multiplies their product into alpha."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200 import onnx_lite as ol
    T = ol.TensorProto
    torch.manual_seed(0)
    M, Kd, N = 256, 512, 384
    a8 = (torch.randn(M, Kd) * 0.5).to(torch.float8_e4m3fn)
    w8 = (torch.randn(N, Kd) * 0.5).to(torch.float8_e4m3fn)
    node = ol.make_node("GemmFloat8", ["a", "w", "", "sa", "sb"], ["y"], domain="com.microsoft", transB=1, dtype=T.BFLOAT16, alpha=2.0)
    g = ol.make_graph([node], "g", [ol.make_tensor_value_info("a", T.FLOAT8E4M3FN, [M, Kd]), ol.make_tensor_value_info("sa", T.FLOAT, [1]),
                                    ol.make_tensor_value_info("sb", T.FLOAT, [1])], [ol.make_tensor_value_info("y", T.BFLOAT16, None)],
                      [ol.make_tensor("w", w8)])
    sess = ort.InferenceSession(ol.make_model(g).serialize(), providers=["CUDAExecutionProvider"], enable_fallback=False)
    for sa, sb in ((0.5, 0.25), (1.5, 0.125)):
        before = sess.kernel_launch_count()
        y = sess.run(None, {"a": a8.cuda(), "sa": torch.tensor([sa]).cuda(), "sb": torch.tensor([sb]).cuda()})[0]
        assert sess.kernel_launch_count() == before + 1
        ref = 2.0 * sa * sb * (a8.float() @ w8.float().T)
        assert (torch.as_tensor(y).float().cpu() - ref).abs().max() / ref.abs().max() < 1e-2
