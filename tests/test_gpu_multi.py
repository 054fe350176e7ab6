"""Multi-GPU (one process per GPU, NCCL + in-kernel peer stores).  Skipped with fewer than two GPUs."""
import pytest
import torch

from test_distributed_cpu import launch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


WORLDS = [2, 4, 8]


def _need(n):
    if _ngpu() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("n", WORLDS)
def test_fused_gemm_allreduce_kernel(tmp_path, n):
    _need(n)
    out = launch("gemm_allreduce", "cuda", n, tmp_path)
    for r in range(n):
        assert out[r]["status"] == 0
        for k, v in out[r].items():
            if k.startswith("case"):
                assert v["err"] < 1e-2 and v["stable"], (r, k, v["err"], v["stable"])
    for k in out[0]:
        if k.startswith("case"):
            for r in range(1, n):
                assert torch.equal(out[0][k]["out"], out[r][k]["out"])  # every rank holds the same reduced result
    if out[0]["nvls"]:  # the workspace has a multicast mapping: the prompt-sized cases also ran through the switch
        assert any(k.endswith("_nvls") for k in out[0])
    print("NVLS multicast mapping:", out[0]["nvls"])


@pytest.mark.parametrize("n", WORLDS)
@pytest.mark.parametrize("fused", ["1", "0"])
def test_llama_tp_gpu(tmp_path, fused, n):
    _need(n)
    out = launch("llama_tp", "cuda", n, tmp_path, extra_env={"ORTB200_TEST_FUSED": fused})
    assert out[0]["fused"] == (fused == "1")
    a, ref = out[0]["logits"], out[0]["ref"]
    for r in range(1, n):
        assert (a - out[r]["logits"]).abs().max() / a.abs().max() < 1e-6
    assert (a - ref).abs().max() / ref.abs().max() < 0.06


@pytest.mark.parametrize("n", WORLDS)
def test_symmetric_memory_collectives(tmp_path, n):
    _need(n)
    out = launch("symm_collectives", "cuda", n, tmp_path)
    for r in range(n):
        assert out[r]["status"] == 0
        for k, v in out[r].items():
            if k.startswith("ar_"):
                assert v < 1e-2, (r, k, v)
            elif k.startswith("ag_") or k.startswith("a2a_"):
                assert v is True, (r, k)


@pytest.mark.parametrize("n", WORLDS)
def test_sharded_moe_fused_combine(tmp_path, n):
    """Expert parallelism with the one-kernel cross-rank combine: every rank ends with the single-device MoE result."""
    _need(n)
    out = launch("sharded_moe_gpu", "cuda", n, tmp_path)
    for k in out[0]:
        ref = out[0][k]["ref"]
        scale = ref.abs().max()
        for r in range(n):
            assert out[r][k]["stable"]
            assert (out[r][k]["fused"] - ref).abs().max() / scale < 3e-2, (r, k)
            assert (out[r][k]["plain"] - ref).abs().max() / scale < 3e-2, (r, k)
            assert torch.equal(out[r][k]["fused"], out[0][k]["fused"])  # replicated bit for bit


@pytest.mark.parametrize("n", WORLDS)
def test_mixtral_shaped_decoder_expert_parallel_gpu(tmp_path, n):
    _need(n)
    out = launch("mixtral_ep", "cuda", n, tmp_path)
    ref = out[0]["ref"]
    for r in range(n):
        assert torch.equal(out[r]["logits"], out[0]["logits"])
        assert (out[r]["logits"] - ref).abs().max() / ref.abs().max() < 5e-2


@pytest.mark.parametrize("n", WORLDS)
def test_llama_tp_int4_reduces_in_kernel_and_is_captured(tmp_path, n):
    """4-bit weights under tensor parallelism: the row-parallel MatMulNBits nodes carry the all-reduce themselves, so the
    decode step holds no library collective (no AllReduce node is left) and runs as a captured graph."""
    _need(n)
    out = launch("llama_tp", "cuda", n, tmp_path, extra_env={"ORTB200_TEST_FUSED": "1", "ORTB200_TEST_QUANT": "4"})
    assert "AllReduce" not in out[0]["ops"] and "MatMulNBits" in out[0]["ops"] and "SwiGLU" in out[0]["ops"]
    a, ref = out[0]["logits"], out[0]["ref"]
    for r in range(1, n):
        assert (a - out[r]["logits"]).abs().max() / a.abs().max() < 1e-6
    assert (a - ref).abs().max() / ref.abs().max() < 0.06


@pytest.mark.parametrize("n", WORLDS)
def test_allgather_gemm_one_kernel(tmp_path, n):
    _need(n)
    out = launch("allgather_gemm", "cuda", n, tmp_path)
    for r in range(n):
        assert out[r]["status"] == 0
        for k, v in out[r].items():
            if k.startswith("agg_"):
                assert v < 2e-2, (r, k, v)
        assert out[r]["same"] < 0.25, out[r]["same"]
    fused, library, gemm = (max(out[r][k] for r in range(n)) for k in ("ms_fused", "ms_library", "ms_gemm_only"))
    print(f"allgather_gemm world={n} 8192x4096x8192: fused {fused:.3f} ms, all-gather + GEMM {library:.3f} ms, GEMM alone {gemm:.3f} ms")
