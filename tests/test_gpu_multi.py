"""Multi-GPU (one process per GPU, NCCL + in-kernel peer stores).  Skipped with fewer than two GPUs."""
import pytest
import torch

from test_distributed_cpu import launch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_gemm_allreduce_kernel(tmp_path):
    n = 2
    out = launch("gemm_allreduce", "cuda", n, tmp_path)
    for r in range(n):
        assert out[r]["status"] == 0
        for k, v in out[r].items():
            if k.startswith("case"):
                assert v["err"] < 1e-2 and v["stable"], (r, k, v["err"], v["stable"])
    for k in out[0]:
        if k.startswith("case"):
            assert torch.equal(out[0][k]["out"], out[1][k]["out"])  # every rank holds the same reduced result


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", ["1", "0"])
def test_llama_tp2_gpu(tmp_path, fused):
    out = launch("llama_tp", "cuda", 2, tmp_path, extra_env={"ORTB200_TEST_FUSED": fused})
    assert out[0]["fused"] == (fused == "1")
    a, b, ref = out[0]["logits"], out[1]["logits"], out[0]["ref"]
    assert (a - b).abs().max() / a.abs().max() < 1e-6
    assert (a - ref).abs().max() / ref.abs().max() < 0.06


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_symmetric_memory_collectives(tmp_path):
    out = launch("symm_collectives", "cuda", 2, tmp_path)
    for r in range(2):
        assert out[r]["status"] == 0
        for k, v in out[r].items():
            if k.startswith("ar_"):
                assert v < 1e-2, (r, k, v)
            elif k.startswith("ag_") or k.startswith("a2a_"):
                assert v is True, (r, k)
