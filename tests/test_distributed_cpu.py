"""Collective / tensor-parallel host logic on CPU ranks (gloo, world size 2): real processes, no GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(case, device, nproc, tmp_path, extra_env=None, timeout=300):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ)
    env.update({"OMP_NUM_THREADS": "1", "NCCL_NVLS_ENABLE": "0"})
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_worker.py"), case, device, str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(nproc)]


def test_collective_ops(tmp_path):
    out = launch("collectives", "cpu", 2, tmp_path)
    xs = [np.arange(8, dtype=np.float32).reshape(4, 2) + 10 * r for r in range(2)]
    for r in range(2):
        np.testing.assert_array_equal(out[r]["AllReduce"].numpy(), xs[0] + xs[1])
        np.testing.assert_array_equal(out[r]["AllGather0"].numpy(), np.concatenate(xs, 0))
        np.testing.assert_array_equal(out[r]["AllGather1"].numpy(), np.concatenate(xs, 1))
        # all-to-all with equal splits along the flattened leading dimension
        expect = np.concatenate([np.split(x, 2, 0)[r] for x in xs], 0)
        np.testing.assert_array_equal(out[r]["AllToAll"].numpy(), expect)
        wt = (np.arange(6, dtype=np.float32).reshape(2, 3) - 2) * 0.5
        np.testing.assert_allclose(out[r]["AllGatherMatMul"].numpy(), np.concatenate(xs, 0) @ wt + np.array([1, 2, 3], np.float32), rtol=1e-6)


def test_distributed_matmul_specs(tmp_path):
    out = launch("distributed_matmul", "cpu", 2, tmp_path)
    full = out[0]["full"].numpy()
    for r in range(2):
        np.testing.assert_allclose(out[r]["col"].numpy(), np.split(full, 2, 1)[r], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(out[r]["row"].numpy(), full, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(out[r]["reshard"].numpy(), full, rtol=1e-5, atol=1e-5)


def test_sharded_moe_matches_single_device_moe(tmp_path):
    out = launch("sharded_moe", "cpu", 2, tmp_path)
    for r in range(2):
        np.testing.assert_allclose(out[r]["y"].numpy(), out[r]["ref"].numpy(), rtol=1e-4, atol=1e-5)


def test_sharded_moe_with_sharded_tokens_dispatches_and_combines(tmp_path):
    """tokens_sharded = 1: every rank feeds different tokens; rows go to the ranks of their experts and the partial sums come
    back.  Each rank's result equals the single-device MoE over the full expert set on that rank's tokens."""
    out = launch("sharded_moe_tokens", "cpu", 2, tmp_path)
    for r in range(2):
        np.testing.assert_allclose(out[r]["y"].numpy(), out[r]["ref"].numpy(), rtol=1e-4, atol=1e-5)
    assert not np.allclose(out[0]["ref"].numpy(), out[1]["ref"].numpy())


def test_llama_tensor_parallel_matches_single_rank(tmp_path):
    out = launch("llama_tp", "cpu", 2, tmp_path)
    assert "AllReduce" in out[0]["ops"]
    assert out[0]["first_equal"]
    np.testing.assert_allclose(out[0]["logits"].numpy(), out[1]["logits"].numpy(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(out[0]["logits"].numpy(), out[0]["ref"].numpy(), rtol=2e-3, atol=2e-3)


def test_int4_llama_tensor_parallel_matches_single_rank(tmp_path, monkeypatch):
    """The 4-bit model shards its packed blocks (rows for column-parallel, block ranges for row-parallel
    projections); two ranks must reproduce the single-rank logits."""
    monkeypatch.setenv("ORTB200_TEST_QUANT", "4")
    out = launch("llama_tp", "cpu", 2, tmp_path)
    assert "MatMulNBits" in out[0]["ops"] and "AllReduce" in out[0]["ops"]
    np.testing.assert_allclose(out[0]["logits"].numpy(), out[0]["ref"].numpy(), rtol=2e-3, atol=2e-3)


def test_sharding_spec_algebra():
    from onnxruntime_b200 import _core as C
    d = C.parse_shard_spec("RS[0]", [0, 1, 2, 3], [4])
    assert d == {"spec": "RS[0]", "sharded_axis": 1, "num_shards": 4}
    assert C.shard_shape([8, 12], "RS[0]", [0, 1, 2, 3], [4]) == [8, 3]
    assert C.shard_shape([8, 12], "S[0]R", [0, 1], [2]) == [4, 12]
    assert C.parse_shard_spec("RRR", [0, 1], [2])["sharded_axis"] == -1
    import onnxruntime_b200 as ort
    with pytest.raises(ort.InvalidArgument):
        C.parse_shard_spec("S[0]S[0]", [0, 1], [2])
    with pytest.raises(ort.InvalidArgument):
        C.shard_shape([7, 12], "S[0]R", [0, 1], [2])


def test_mixtral_shaped_decoder_with_expert_parallelism(tmp_path):
    """Two gloo ranks, two local experts each: the expert-parallel decoder reproduces the single-rank mixture."""
    out = launch("mixtral_ep", "cpu", 2, tmp_path)
    assert "ShardedMoE" in out[0]["ops"]
    a, b, ref = out[0]["logits"], out[1]["logits"], out[0]["ref"]
    assert (a - b).abs().max() == 0
    assert (a - ref).abs().max() / ref.abs().max() < 1e-4


def test_data_parallel_training_follows_the_full_batch_run(tmp_path):
    """Training API with bucketed gradient all-reduce and ORTModule under DistributedDataParallel, 2 gloo ranks."""
    out = launch("data_parallel_training", "cpu", 2, tmp_path)
    for r in range(2):
        for k, ref in out[r]["ref"].items():
            np.testing.assert_allclose(out[r]["api"][k].numpy(), ref.numpy(), rtol=2e-3, atol=2e-4, err_msg=k)
            np.testing.assert_allclose(out[r]["ddp_grad"][k].numpy(), out[r]["full_grad"][k].numpy(), rtol=1e-4, atol=1e-6, err_msg=k)
    for k in out[0]["api"]:
        np.testing.assert_array_equal(out[0]["api"][k].numpy(), out[1]["api"][k].numpy())


def test_megatron_split_mlp_trains_with_the_gradients_of_the_whole(tmp_path):
    """MegatronF / MegatronG around a column- and a row-parallel weight: every rank holds its shard's gradient, and the
    replicated weight in front of the split gets the full gradient (the backward all-reduce of MegatronF)."""
    out = launch("megatron_training", "cpu", 2, tmp_path)
    for r in range(2):
        o = out[r]
        assert abs(o["loss"].item() - o["ref_loss"].item()) < 1e-5
        ref = o["ref_grads"]
        np.testing.assert_allclose(o["grads"]["w0"].numpy(), ref["w0"].numpy(), rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(o["grads"]["w1"].numpy(), np.split(ref["w1"].numpy(), 2, 1)[r], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(o["grads"]["b1"].numpy(), np.split(ref["b1"].numpy(), 2, 0)[r], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(o["grads"]["w2"].numpy(), np.split(ref["w2"].numpy(), 2, 0)[r], rtol=1e-4, atol=1e-6)
