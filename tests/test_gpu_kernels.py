"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from onnxruntime_b200.ops import _kernels
    _kernels.lib()  # fail loudly when the library is missing
    return _kernels


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


@pytest.mark.parametrize("M,N,Kd", [(8, 128, 64), (8, 4096, 4096), (1, 6144, 4096), (16, 1024, 14336), (32, 1024, 1024),
                                    (64, 1024, 1024), (128, 1024, 1024), (200, 1000, 1024), (1024, 4096, 1024),
                                    (8, 1000, 264)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm(K, M, N, Kd, dtype):
    torch.manual_seed(0)
    x = (torch.randn(M, Kd, device="cuda") * 0.5).to(dtype)
    w = (torch.randn(N, Kd, device="cuda") * 0.05).to(dtype)
    y = K.gemm(x, w)
    ref = x.float() @ w.float().T
    assert _rel(y, ref) < 1e-2


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_gemm_split_k_epilogue(K, splits):
    torch.manual_seed(1)
    x = (torch.randn(8, 4096, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(2048, 4096, device="cuda") * 0.05).bfloat16()
    b = torch.randn(2048, device="cuda").bfloat16()
    r = torch.randn(8, 2048, device="cuda").bfloat16()
    y = K.gemm(x, w, bias=b, residual=r, act="fastgelu", force_splits=splits)
    ref = torch.nn.functional.gelu(x.float() @ w.float().T + b.float(), approximate="tanh") + r.float()
    assert _rel(y, ref) < 1e-2


@pytest.mark.parametrize("M", [8, 300])
def test_gemm_swiglu(K, M):
    torch.manual_seed(2)
    I, H = 1536, 1024
    x = (torch.randn(M, H, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(2 * I, H, device="cuda") * 0.05).bfloat16()
    y = K.gemm(x, w, act="swiglu")
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    assert _rel(y, torch.nn.functional.silu(g) * u) < 1.5e-2


def test_gemm_deterministic(K):
    torch.manual_seed(3)
    x = (torch.randn(8, 14336, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(4096, 14336, device="cuda") * 0.05).bfloat16()
    a = K.gemm(x, w)
    b = K.gemm(x, w)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("H", [128, 1024, 4096, 8192])
@pytest.mark.parametrize("simplified", [True, False])
def test_norm(K, dtype, H, simplified):
    torch.manual_seed(0)
    rows = 37
    x = torch.randn(rows, H, device="cuda").to(dtype)
    skip = torch.randn(rows, H, device="cuda").to(dtype)
    bias = torch.randn(H, device="cuda").to(dtype)
    gamma = torch.randn(H, device="cuda").to(dtype)
    beta = None if simplified else torch.randn(H, device="cuda").to(dtype)
    out, s = K.norm(x, gamma, beta=beta, skip=skip, bias=bias, eps=1e-5, simplified=simplified, want_sum=True)
    sf = (x.float() + skip.float() + bias.float()).to(dtype).float()
    if simplified:
        ref = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
    else:
        ref = torch.nn.functional.layer_norm(sf, (H,), gamma.float(), beta.float(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert _rel(out, ref) < tol
    assert _rel(s, sf) < 1e-6


def _ref_attention(q, k, v, causal_offset, scale, window=-1, lens=None):
    # q [B,N,S,H], k/v [B,Nk,T,H] fp32; query s sits at position causal_offset[b] + s
    B, N, S, H = q.shape
    Nk, T = k.shape[1], k.shape[2]
    g = N // Nk
    kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = q @ kk.transpose(-1, -2) * scale
    qpos = causal_offset.view(B, 1, 1, 1) + torch.arange(S, device=q.device).view(1, 1, S, 1)
    kpos = torch.arange(T, device=q.device).view(1, 1, 1, T)
    allowed = kpos <= qpos
    if window > 0:
        allowed = allowed & (kpos > qpos - window)
    if lens is not None:
        allowed = allowed & (kpos < lens.view(B, 1, 1, 1))
    s = s.masked_fill(~allowed, float("-inf"))
    return torch.softmax(s, -1) @ vv


@pytest.mark.parametrize("H", [64, 128])
@pytest.mark.parametrize("N,Nk", [(4, 4), (8, 2), (32, 8), (8, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gqa_decode(K, H, N, Nk, dtype):
    torch.manual_seed(0)
    B, Smax = 3, 700
    lens = torch.tensor([1, 333, 700], dtype=torch.int32, device="cuda")
    q = torch.randn(B, N, H, device="cuda").to(dtype)
    kc = torch.randn(B, Nk, Smax, H, device="cuda").to(dtype)
    vc = torch.randn(B, Nk, Smax, H, device="cuda").to(dtype)
    out = K.gqa_decode(q, kc, vc, lens - 1)
    ref = _ref_attention(q.float().unsqueeze(2), kc.float(), vc.float(), (lens - 1).long(), 1 / math.sqrt(H),
                         lens=lens.long()).squeeze(2)
    assert _rel(out.view(B, N, H), ref) < 2e-2


def test_gqa_decode_window(K):
    torch.manual_seed(0)
    B, N, Nk, H, Smax = 2, 8, 2, 128, 512
    lens = torch.tensor([100, 512], dtype=torch.int32, device="cuda")
    q = torch.randn(B, N, H, device="cuda").bfloat16()
    kc = torch.randn(B, Nk, Smax, H, device="cuda").bfloat16()
    vc = torch.randn(B, Nk, Smax, H, device="cuda").bfloat16()
    out = K.gqa_decode(q, kc, vc, lens - 1, window=64)
    ref = _ref_attention(q.float().unsqueeze(2), kc.float(), vc.float(), (lens - 1).long(), 1 / math.sqrt(H), window=64,
                         lens=lens.long()).squeeze(2)
    assert _rel(out.view(B, N, H), ref) < 2e-2


@pytest.mark.parametrize("H", [64, 128])
@pytest.mark.parametrize("S,past", [(128, 0), (200, 0), (1024, 0), (77, 300)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attn_prefill(K, H, S, past, dtype):
    torch.manual_seed(0)
    B, N, Nk = 2, 4, 2
    T = past + S
    q = torch.randn(B, S, N, H, device="cuda").to(dtype)
    kc = torch.randn(B, Nk, T + 5, H, device="cuda").to(dtype)
    vc = torch.randn(B, Nk, T + 5, H, device="cuda").to(dtype)
    seqlens = torch.full((B,), T - 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = K.attn_prefill(q, kc, vc, seqlens, first_prompt=(past == 0), status=status)
    assert status.item() == 0
    ref = _ref_attention(q.float().transpose(1, 2), kc.float(), vc.float(),
                         torch.full((B,), past, device="cuda"), 1 / math.sqrt(H),
                         lens=torch.full((B,), T, device="cuda")).transpose(1, 2)
    assert _rel(out, ref) < 2e-2


def test_attn_prefill_noncausal_lengths(K):
    torch.manual_seed(0)
    B, S, N, H = 3, 384, 4, 64
    q = torch.randn(B, S, N, H, device="cuda").half()
    k = torch.randn(B, S, N, H, device="cuda").half()
    v = torch.randn(B, S, N, H, device="cuda").half()
    lens = torch.tensor([384, 100, 257], dtype=torch.int32, device="cuda")
    out = K.attn_prefill(q, k, v, lens - 1, first_prompt=True, causal=False, kv_layout="bsnh")
    s = torch.einsum("bsnh,btnh->bnst", q.float(), k.float()) / math.sqrt(H)
    mask = torch.arange(S, device="cuda").view(1, 1, 1, S) < lens.view(B, 1, 1, 1)
    ref = torch.einsum("bnst,btnh->bsnh", torch.softmax(s.masked_fill(~mask, float("-inf")), -1), v.float())
    assert _rel(out, ref) < 2e-2


def test_gqa_prep_rotary_append(K):
    torch.manual_seed(0)
    B, S, N, Nk, H, Smax = 2, 5, 4, 2, 64, 32
    qkv = torch.randn(B, S, (N + 2 * Nk) * H, device="cuda").bfloat16()
    half = H // 2
    inv = 1.0 / (10000 ** (torch.arange(half, device="cuda").float() / half))
    ang = torch.outer(torch.arange(Smax, device="cuda").float(), inv)
    cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    kc = torch.zeros(B, Nk, Smax, H, device="cuda").bfloat16()
    vc = torch.zeros_like(kc)
    seqlens = torch.tensor([7 + S - 1, 3 + S - 1], dtype=torch.int32, device="cuda")  # past lengths 7 and 3
    q_rot = K.gqa_prep(qkv, kc, vc, seqlens, cos, sin, N, Nk, H, first_prompt=False)
    qf = qkv.float().view(B, S, N + 2 * Nk, H)
    for b, past in enumerate([7, 3]):
        pos = torch.arange(past, past + S, device="cuda")
        c, s_ = cos.float()[pos].unsqueeze(1), sin.float()[pos].unsqueeze(1)

        def rot(x):
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat([x1 * c - x2 * s_, x2 * c + x1 * s_], -1)
        assert _rel(q_rot[b], rot(qf[b, :, :N])) < 1e-2
        assert _rel(kc[b, :, past:past + S].transpose(0, 1), rot(qf[b, :, N:N + Nk])) < 1e-2
        assert torch.equal(vc[b, :, past:past + S].transpose(0, 1), qkv.view(B, S, N + 2 * Nk, H)[b, :, N + Nk:])


def test_argmax_gather(K):
    torch.manual_seed(0)
    x = torch.randn(8, 128256, device="cuda").bfloat16()
    assert torch.equal(K.argmax(x), x.float().argmax(-1))
    table = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (4, 7), device="cuda")
    assert torch.equal(K.gather_rows(table, ids), table[ids])


@pytest.mark.parametrize("M,N,Kd,act", [(8, 1024, 4096, "none"), (1, 512, 512, "none"), (16, 2048, 1024, "swiglu"), (33, 768, 2048, "none"),
                                        (8, 4096, 14336, "none")])
def test_gemm_fused_rms_norm(K, M, N, Kd, act):
    """out = act((x / rms(x)) @ (W * gamma)^T): gamma is folded into the weights by the caller, 1 / rms in the epilogue."""
    torch.manual_seed(0)
    x = (torch.randn(M, Kd, device="cuda") * 2.0).bfloat16()
    rows = N * (2 if act == "swiglu" else 1)
    w = (torch.randn(rows, Kd, device="cuda") * 0.05).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16() if act == "none" else None
    y = K.gemm(x, w, act=act, residual=res, rms_eps=1e-5)
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    if act == "swiglu":
        ref = torch.nn.functional.silu(xn @ w[:N].float().T) * (xn @ w[N:].float().T)
    else:
        ref = xn @ w.float().T + res.float()
    assert _rel(y, ref) < 1e-2


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("H", [64, 128])
def test_gqa_decode_split_counts_agree(K, H, splits):
    """Every split count gives the fp32 reference's answer, also with a head sink and a soft cap in play."""
    torch.manual_seed(1)
    B, N, Nk, Smax = 4, 16, 2, 1100
    lens = torch.tensor([1, 31, 640, 1100], dtype=torch.int32, device="cuda")
    q = torch.randn(B, N, H, device="cuda").bfloat16()
    kc = torch.randn(B, Nk, Smax, H, device="cuda").bfloat16()
    vc = torch.randn(B, Nk, Smax, H, device="cuda").bfloat16()
    a = K.gqa_decode(q, kc, vc, lens - 1, splits=splits)
    ref = _ref_attention(q.float().unsqueeze(2), kc.float(), vc.float(), (lens - 1).long(), 1 / math.sqrt(H), lens=lens.long()).squeeze(2)
    assert _rel(a.view(B, N, H), ref) < 2e-2
    sink = torch.randn(N, device="cuda").bfloat16()
    a2 = K.gqa_decode(q, kc, vc, lens - 1, splits=splits, head_sink=sink, softcap=30.0)
    b2 = K.gqa_decode(q, kc, vc, lens - 1, splits=1, head_sink=sink, softcap=30.0)
    assert _rel(a2, b2) < 1e-2


@pytest.mark.parametrize("H,N,Nk", [(128, 32, 8), (64, 8, 2), (128, 4, 4), (128, 8, 1)])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gqa_decode_with_fused_rotary_and_append(K, H, N, Nk, interleaved, dtype):
    """One-token step with the unpack + rotary + KV append done inside the attention kernel equals the two-kernel
    sequence (prep kernel, then attention), output and cache contents alike."""
    torch.manual_seed(0)
    B, Smax = 4, 600
    lens = torch.tensor([1, 2, 300, 600], dtype=torch.int32, device="cuda")   # length including the new token
    qkv = torch.randn(B, 1, (N + 2 * Nk) * H, device="cuda").to(dtype)
    kc = torch.randn(B, Nk, Smax, H, device="cuda").to(dtype)
    vc = torch.randn(B, Nk, Smax, H, device="cuda").to(dtype)
    half = H // 2
    pos = torch.arange(1024, device="cuda").float().unsqueeze(1)
    inv = 1.0 / (10000 ** (torch.arange(half, device="cuda").float() / half))
    cos, sin = torch.cos(pos * inv).to(dtype), torch.sin(pos * inv).to(dtype)
    k1, v1 = kc.clone(), vc.clone()
    q_rot = K.gqa_prep(qkv, k1, v1, lens - 1, cos, sin, N, Nk, H, first_prompt=False, interleaved=interleaved)
    want = K.gqa_decode(q_rot.view(B, N, H), k1, v1, lens - 1)
    k2, v2 = kc.clone(), vc.clone()
    got = K.gqa_decode(None, k2, v2, lens - 1, qkv=qkv.view(B, -1), num_heads=N, cos=cos, sin=sin, interleaved=interleaved)
    torch.cuda.synchronize()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert _rel(got, want) < 1e-2


# ---------------------------------------------------------------- tcgen05 decode attention (head size 128)
@pytest.mark.parametrize("N,Nk", [(32, 8), (16, 2), (4, 4), (16, 1), (6, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gqa_decode_tensor_core_kernel(K, N, Nk, dtype):
    """The tensor-core kernel against the fp32 reference: lengths that end inside a tile, the cache beyond each
    length poisoned with NaN (a masked key must not leak through 0 * NaN), and scores that keep growing along the
    sequence so the reference maximum is raised (and O^T rescaled) several times."""
    torch.manual_seed(0)
    B, H, Smax = 4, 128, 1152
    lens = torch.tensor([1, 130, 1024, 1152], dtype=torch.int32, device="cuda")
    q = torch.randn(B, N, H, device="cuda").to(dtype)
    ramp = torch.linspace(0.2, 3.0, Smax, device="cuda").view(1, 1, Smax, 1)
    kc = (torch.randn(B, Nk, Smax, H, device="cuda") * ramp).to(dtype)
    vc = torch.randn(B, Nk, Smax, H, device="cuda").to(dtype)
    ref = _ref_attention(q.float().unsqueeze(2), kc.float(), vc.float(), (lens - 1).long(), 1 / math.sqrt(H),
                         lens=lens.long()).squeeze(2)
    for b in range(B):
        kc[b, :, int(lens[b]):] = float("nan")
        vc[b, :, int(lens[b]):] = float("nan")
    for splits in (0, 1, 3):
        out = K.gqa_decode(q, kc, vc, lens - 1, splits=splits, algo=2)
        assert torch.isfinite(out.float()).all()
        assert _rel(out.view(B, N, H), ref) < 2e-2, splits
    old = K.gqa_decode(q, kc, vc, lens - 1, algo=1)
    assert _rel(old.view(B, N, H), ref) < 2e-2


@pytest.mark.parametrize("block_size", [16, 128, 256])
def test_gqa_decode_tensor_core_kernel_paged(K, block_size):
    torch.manual_seed(1)
    B, N, Nk, H = 3, 8, 2, 128
    max_len = 768
    per_seq = max_len // block_size
    lens = torch.tensor([5, 300, 768], dtype=torch.int32, device="cuda")
    num_blocks = B * per_seq + 3
    perm = torch.randperm(num_blocks, device="cuda")[:B * per_seq].view(B, per_seq).int()
    k = torch.randn(B, Nk, max_len, H, device="cuda").bfloat16()
    v = torch.randn(B, Nk, max_len, H, device="cuda").bfloat16()
    kc = torch.full((num_blocks, block_size, Nk, H), float("nan"), device="cuda", dtype=torch.bfloat16)
    vc = torch.full((num_blocks, block_size, Nk, H), float("nan"), device="cuda", dtype=torch.bfloat16)
    for b in range(B):
        for j in range(per_seq):
            lo, hi = j * block_size, min((j + 1) * block_size, int(lens[b]))
            if hi > lo:
                kc[perm[b, j], :hi - lo] = k[b, :, lo:hi].transpose(0, 1)
                vc[perm[b, j], :hi - lo] = v[b, :, lo:hi].transpose(0, 1)
    # table entries past a sequence's last block are unset
    table = perm.clone()
    for b in range(B):
        used = (int(lens[b]) + block_size - 1) // block_size
        table[b, used:] = -1
    q = torch.randn(B, N, H, device="cuda").bfloat16()
    ref = _ref_attention(q.float().unsqueeze(2), k.float(), v.float(), (lens - 1).long(), 1 / math.sqrt(H),
                         lens=lens.long()).squeeze(2)
    for algo in (1, 2):
        tb = table if algo == 2 else perm   # the CUDA-core kernel is given a fully populated table
        out = K.gqa_decode(q, kc, vc, lens - 1, block_table=tb, algo=algo)
        assert torch.isfinite(out.float()).all(), algo
        assert _rel(out.view(B, N, H), ref) < 2e-2, algo


@pytest.mark.parametrize("interleaved", [False, True])
def test_gqa_decode_tensor_core_kernel_paged_fused_append(K, interleaved):
    """Paged cache + fused step 1 in the tcgen05 kernel: same result as rotating / appending first and attending after,
    and the new key / value land in the right slot of the block pool."""
    torch.manual_seed(2)
    B, N, Nk, H, bs = 3, 8, 2, 128, 16
    max_len = 256
    per_seq = max_len // bs
    lens = torch.tensor([1, 100, 256], dtype=torch.int32, device="cuda")     # totals including the new token
    num_blocks = B * per_seq
    table = torch.randperm(num_blocks, device="cuda").view(B, per_seq).int()
    kc = torch.randn(num_blocks, bs, Nk, H, device="cuda").bfloat16()
    vc = torch.randn(num_blocks, bs, Nk, H, device="cuda").bfloat16()
    qkv = torch.randn(B, (N + 2 * Nk) * H, device="cuda").bfloat16()
    pos = torch.arange(max_len, device="cuda").float()
    inv = 1.0 / (10000 ** (torch.arange(0, H // 2, device="cuda").float() / (H // 2)))
    cos, sin = torch.outer(pos, inv).cos().bfloat16(), torch.outer(pos, inv).sin().bfloat16()
    k1, v1 = kc.clone(), vc.clone()
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
    q_rot = K.paged_prep(qkv, k1, v1, cu, lens - 1, table, N, Nk, cos=cos, sin=sin, interleaved=interleaved)
    want = K.gqa_decode(q_rot.view(B, N, H), k1, v1, lens - 1, block_table=table, algo=2)
    k2, v2 = kc.clone(), vc.clone()
    got = K.gqa_decode(None, k2, v2, lens - 1, block_table=table, qkv=qkv, num_heads=N, cos=cos, sin=sin, interleaved=interleaved, algo=2)
    assert _rel(got, want) < 1e-2
    assert torch.equal(k1, k2) and torch.equal(v1, v2)


def test_fused_allreduce_gives_up_on_a_silent_peer(K):
    """Failure detection without a fault: rank 0 of a two-rank fused GEMM + all-reduce whose peer never writes (its
    'workspace' is a second local buffer that nothing fills).  The kernel's polling limit (header word 2, set small
    here) runs out, the status word reports the peer timeout, the kernel returns normally and the context stays
    usable - the next GEMM is correct."""
    torch.manual_seed(0)
    nbytes = 4 << 20
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    ws.view(torch.int32)[2] = 2000            # polling rounds before giving up (default: 4 M)
    x = torch.randn(8, 256, device="cuda").bfloat16()
    w = (torch.randn(128, 256, device="cuda") * 0.1).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    K.gemm(x, w, peers=[ws.data_ptr(), silent_peer.data_ptr()], rank=0, symm_bytes=nbytes, status=status)
    t1.record()
    torch.cuda.synchronize()
    assert status.item() == 4                  # kStatusTimeoutPeer
    assert t0.elapsed_time(t1) < 1000.0        # milliseconds: bounded, nowhere near a hang
    status.zero_()
    y = K.gemm(x, w, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert _rel(y, x.float() @ w.float().T) < 2e-2


def test_symmetric_collective_gives_up_on_a_silent_peer(K):
    """The same for the one-kernel collectives: rank 0 of a two-rank all-reduce whose peer never raises its flags (the
    peer 'workspace' is a second local buffer).  The polling limit (header word at byte 72, set small here) runs out,
    the status word reports the peer, the kernel returns, and a later single-GPU kernel is correct."""
    nbytes = 8 << 20
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    ws.view(torch.int32)[18] = 2000
    x = torch.randn(4096, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    K.symm_collective("allreduce", x, [ws.data_ptr(), silent_peer.data_ptr()], 0, nbytes, status=status)
    t1.record()
    torch.cuda.synchronize()
    assert status.item() == 4
    assert t0.elapsed_time(t1) < 1000.0
    status.zero_()
    a = torch.randn(8, 256, device="cuda").bfloat16()
    w = (torch.randn(128, 256, device="cuda") * 0.1).bfloat16()
    y = K.gemm(a, w, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0 and _rel(y, a.float() @ w.float().T) < 2e-2
