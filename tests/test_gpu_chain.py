"""gemm_chain_kernel: dependent decode GEMMs in one persistent launch, against a PyTorch fp32 restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from onnxruntime_b200.ops import _kernels
    _kernels.lib()
    return _kernels


def _ref_chain(x, stages, dtype):
    """fp32 math with the same rounding points as the kernel: every stage output is rounded to the 16-bit type."""
    outs = []
    cur = x.float()
    for st in stages:
        w = st["w"].float()
        xin = cur
        if st.get("rms_eps", 0.0) > 0:
            xin = cur * torch.rsqrt(cur.pow(2).mean(-1, keepdim=True) + st["rms_eps"])
        y = xin @ w.t()
        act = st.get("act", "none")
        if act == "swiglu":
            n = w.shape[0] // 2
            g, u = y[:, :n], y[:, n:]
            if st.get("bias") is not None:
                g = g + st["bias"].float()
            y = torch.nn.functional.silu(g) * u
        else:
            if st.get("bias") is not None:
                y = y + st["bias"].float()
            if act == "gelu":
                y = torch.nn.functional.gelu(y)
            elif act == "silu":
                y = torch.nn.functional.silu(y)
            elif act == "relu":
                y = torch.relu(y)
        res = st.get("residual")
        if isinstance(res, int):
            y = y + outs[res].float()
        elif res is not None:
            y = y + res.float()
        y = y.to(dtype)
        outs.append(y)
        cur = y.float()
    return outs


def _llama_like(H, F, QKV, M, dtype, dev="cuda", seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(dev)
    x = rnd(M, H, std=0.5)
    resid = rnd(M, H, std=0.5)
    stages = [
        {"w": rnd(H, H, std=H ** -0.5), "residual": resid},
        {"w": rnd(2 * F, H, std=H ** -0.5), "act": "swiglu", "rms_eps": 1e-5},
        {"w": rnd(H, F, std=F ** -0.5), "residual": 0},
        {"w": rnd(QKV, H, std=H ** -0.5), "rms_eps": 1e-5, "bias": rnd(QKV, std=0.1)},
    ]
    return x, stages


def _close(got, want, tol):
    for i, (a, b) in enumerate(zip(got, want)):
        err = (a.float() - b.float()).abs().max().item()
        ref = max(b.float().abs().max().item(), 1e-3)
        assert err <= tol * ref, f"stage {i}: max abs err {err} vs scale {ref}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("H,F,QKV", [(512, 1024, 768), (1024, 3584, 1536), (256, 320, 200)])
def test_chain_matches_reference(K, dtype, M, H, F, QKV):
    if F % 64:
        pytest.skip("K of the down projection must be a multiple of 64")
    x, stages = _llama_like(H, F, QKV, M, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = K.gemm_chain(x, stages, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    _close(got, _ref_chain(x, stages, dtype), 2e-2)


def test_chain_is_deterministic_and_reusable(K):
    x, stages = _llama_like(1024, 2048, 1536, 8, torch.bfloat16, seed=3)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = [t.clone() for t in K.gemm_chain(x, stages, status=status)]
    for prefetch in (0, 8, 8):
        again = K.gemm_chain(x, stages, status=status, prefetch_items=prefetch)
        torch.cuda.synchronize()
        for a, b in zip(first, again):
            assert torch.equal(a, b)
    assert status.item() == 0


def test_chain_with_few_ctas_and_one_stage(K):
    """Slices that span several tiles (few CTAs) and a single-stage chain with an odd N."""
    x, stages = _llama_like(512, 1024, 200, 5, torch.float16, seed=5)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = _ref_chain(x, stages, torch.float16)
    for ctas in (1, 3, 37):
        got = K.gemm_chain(x, stages, status=status, max_ctas=ctas)
        torch.cuda.synchronize()
        _close(got, want, 2e-2)
    one = K.gemm_chain(x, stages[:1], status=status)
    torch.cuda.synchronize()
    _close(one, want[:1], 2e-2)
    assert status.item() == 0
