"""Session-level behaviour on the GPU provider: fused-GEMM residual shapes, CUDA-graph replay without aliasing the
caller's tensors, arg-max tie rule."""
import numpy as np
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol
from helpers import graph_model, op_counts

pytestmark = pytest.mark.gpu
T = ol.TensorProto


def _matmul_add_model(res_shape, K=64, N=128):
    torch.manual_seed(0)
    W = (torch.randn(K, N) * 0.1).half()
    nodes = [ol.make_node("MatMul", ["x", "W"], ["mm"]), ol.make_node("Add", ["mm", "t"], ["y"])]
    return graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, ["b", "s", K]), ol.make_tensor_value_info("t", T.FLOAT16, res_shape)],
                       [ol.make_tensor_value_info("y", T.FLOAT16, None)], [ol.make_tensor("W", W)]), W


@pytest.mark.parametrize("res_shape", [[2, 5, 128], [2, 1, 128], [1, 5, 128], [128], [3, 2, 5, 128]])
def test_fused_gemm_residual_follows_add_broadcasting(res_shape):
    """MatMul + Add becomes one FusedGemm; an operand that is not exactly the product's shape must still broadcast as
    the Add did (the kernel epilogue only takes a full [M, N] residual)."""
    model, W = _matmul_add_model(res_shape)
    x = (torch.randn(2, 5, 64) * 0.5).half()
    t = torch.randn(*res_shape).half()
    sess = ort.InferenceSession(model, providers=["CUDAExecutionProvider"], enable_fallback=False)
    assert op_counts(sess).get("FusedGemm") == 1
    y = sess.run(None, {"x": x.numpy(), "t": t.numpy()})[0]
    ref = (x.float() @ W.float() + t.float()).numpy()
    assert y.shape == ref.shape
    np.testing.assert_allclose(y.astype(np.float32), ref, rtol=2e-2, atol=2e-2)
    sess.check_device_status()


def test_cuda_graph_replay_leaves_earlier_arguments_and_results_alone():
    """Plain run() under a captured graph: a second run with other tensors must neither overwrite the first call's
    input nor the output returned by the first call."""
    torch.manual_seed(1)
    W = (torch.randn(64, 64) * 0.1).half()
    nodes = [ol.make_node("MatMul", ["x", "W"], ["mm"]), ol.make_node("Relu", ["mm"], ["y"])]
    model = graph_model(nodes, [ol.make_tensor_value_info("x", T.FLOAT16, [4, 64])], [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                        [ol.make_tensor("W", W)])
    sess = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"enable_cuda_graph": "1"})], enable_fallback=False)
    x1 = ort.OrtValue.ortvalue_from_numpy(torch.randn(4, 64).half().numpy(), "cuda", 0)
    x2 = ort.OrtValue.ortvalue_from_numpy(torch.randn(4, 64).half().numpy(), "cuda", 0)
    x1_before = x1.numpy().copy()
    outs = []
    for _ in range(2):  # first call warms up and captures, the second replays
        outs.append(sess.run_with_ort_values(["y"], {"x": x1})[0])
    y1 = outs[-1].numpy().copy()
    y2 = sess.run_with_ort_values(["y"], {"x": x2})[0].numpy()
    np.testing.assert_array_equal(x1.numpy(), x1_before)
    np.testing.assert_array_equal(outs[-1].numpy(), y1)
    ref2 = torch.relu(torch.from_numpy(x2.numpy()).float() @ W.float()).numpy()
    np.testing.assert_allclose(y2.astype(np.float32), ref2, rtol=2e-2, atol=2e-2)
    assert not np.array_equal(y1, y2)


def test_argmax_treats_the_two_zeros_as_equal():
    from onnxruntime_b200.ops import _kernels as K
    K.lib()
    x = torch.full((3, 1000), -1.0, device="cuda", dtype=torch.float32)
    x[0, 10], x[0, 20] = -0.0, 0.0
    x[1, 10], x[1, 20] = 0.0, -0.0
    x[2, 7] = 0.5
    got = K.argmax(x).cpu()
    assert got.tolist() == torch.argmax(x, dim=-1).cpu().tolist() == [10, 10, 7]


def test_tunable_gemm_picks_a_configuration_and_results_travel():
    """tunable_op_enable + tunable_op_tuning_enable: the first run of a GEMM signature times the candidate launch
    configurations and keeps the fastest; results export / import in the reference's get / set_tuning_results shape and
    the tuned session computes the same product."""
    torch.manual_seed(1)
    K, N = 1024, 2048
    W = (torch.randn(K, N) * 0.05).to(torch.bfloat16)
    model = graph_model([ol.make_node("MatMul", ["x", "W"], ["y"])], [ol.make_tensor_value_info("x", T.BFLOAT16, ["m", K])],
                        [ol.make_tensor_value_info("y", T.BFLOAT16, None)], [ol.make_tensor("W", W)])
    opts = {"tunable_op_enable": "1", "tunable_op_tuning_enable": "1", "tunable_op_max_tuning_duration_ms": "100"}
    sess = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", opts)], enable_fallback=False)
    assert sess.get_tuning_results() == []
    for m in (8, 300):
        x = (torch.randn(m, K) * 0.5).to(torch.bfloat16).cuda()
        y = sess.run(None, {"x": x})[0]
        ref = x.float() @ W.float().cuda()
        assert (torch.as_tensor(y).float().cuda() - ref).abs().max() / ref.abs().max() < 2e-2
    sess.check_device_status()
    res = sess.get_tuning_results()
    assert len(res) == 1 and res[0]["ep"] == "CUDAExecutionProvider"
    gemm = res[0]["results"]["Gemm"]
    assert len(gemm) == 2 and all(k.startswith("Gemm_") and "splits=" in v for k, v in gemm.items())
    # a second session takes the results without tuning
    sess2 = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"tunable_op_enable": "1"})], enable_fallback=False)
    sess2.set_tuning_results(res)
    assert sess2.get_tuning_results()[0]["results"] == res[0]["results"]
    x = (torch.randn(8, K) * 0.5).to(torch.bfloat16).cuda()
    np.testing.assert_array_equal(torch.as_tensor(sess2.run(None, {"x": x})[0]).float().cpu().numpy(),
                                  torch.as_tensor(sess.run(None, {"x": x})[0]).float().cpu().numpy())
    bad = [dict(res[0], validators={"ORTB200_VERSION": "other"})]
    with pytest.raises(Exception):
        sess2.set_tuning_results(bad, error_on_invalid=True)


def test_sdpa_kernel_math_switches_the_fused_attention_kernels_off():
    """Provider option sdpa_kernel = 16 (MATH) and ORT_DISABLE_FLASH_ATTENTION: MultiHeadAttention runs unfused on
    ATen instead of the tcgen05 kernel, with the same result."""
    torch.manual_seed(2)
    B, S, N, H = 2, 96, 4, 64
    model = graph_model([ol.make_node("MultiHeadAttention", ["q", "k", "v"], ["y"], domain="com.microsoft", num_heads=N)],
                        [ol.make_tensor_value_info(n, T.FLOAT16, [B, S, N * H]) for n in ("q", "k", "v")],
                        [ol.make_tensor_value_info("y", T.FLOAT16, None)], [])
    feeds = {n: (torch.randn(B, S, N * H) * 0.5).half().numpy() for n in ("q", "k", "v")}
    fused = ort.InferenceSession(model, providers=["CUDAExecutionProvider"], enable_fallback=False)
    math = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"sdpa_kernel": "16"})], enable_fallback=False)
    y0 = fused.run(None, feeds)[0].astype(np.float32)
    n_fused = fused.kernel_launch_count()
    y1 = math.run(None, feeds)[0].astype(np.float32)
    assert n_fused >= 1 and math.kernel_launch_count() == 0          # none of this library's kernels ran
    np.testing.assert_allclose(y0, y1, rtol=2e-2, atol=2e-3)
