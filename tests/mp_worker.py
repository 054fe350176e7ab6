"""Worker launched by torch.distributed.run from the multi-process tests (one process per rank).

usage: mp_worker.py <case> <device: cpu|cuda> <out_dir>
Each case writes `<out_dir>/rank<r>.pt` with its results; the parent test compares them.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import onnxruntime_b200 as ort  # noqa: E402
from onnxruntime_b200 import onnx_lite as ol  # noqa: E402
from onnxruntime_b200.parallel.dist import init_distributed  # noqa: E402

T = ol.TensorProto


def session(model, info, device, **kw):
    providers = ["CPUExecutionProvider"] if device == "cpu" else [("CUDAExecutionProvider", {"device_id": str(info.local_rank)})]
    return ort.InferenceSession(model, providers=providers, dist=info, enable_fallback=False, **kw)


def case_collectives(info, device, out):
    r, w = info.rank, info.world_size
    x = np.arange(8, dtype=np.float32).reshape(4, 2) + 10 * r
    res = {}
    for op, attrs in (("AllReduce", {}), ("AllGather", {"axis": 0, "group_size": w}), ("AllGather", {"axis": 1, "group_size": w}),
                      ("AllToAll", {"group_size": w})):
        g = ol.make_graph([ol.make_node(op, ["x"], ["y"], domain="com.microsoft", **attrs)], "g",
                          [ol.make_tensor_value_info("x", T.FLOAT, [4, 2])], [ol.make_tensor_value_info("y", T.FLOAT, None)])
        s = session(ol.make_model(g).serialize(), info, device)
        res[f"{op}{attrs.get('axis', '')}"] = torch.from_numpy(s.run(None, {"x": x})[0])
    # the fused node's generic form: all-gather along axis 0, then MatMul + bias
    wt = (np.arange(6, dtype=np.float32).reshape(2, 3) - 2) * 0.5
    g = ol.make_graph([ol.make_node("AllGatherMatMul", ["x", "w", "b"], ["y"], domain="com.ortb200")], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [4, 2])], [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_tensor("w", wt), ol.make_tensor("b", np.array([1, 2, 3], np.float32))])
    s = session(ol.make_model(g).serialize(), info, device)
    res["AllGatherMatMul"] = torch.from_numpy(s.run(None, {"x": x})[0])
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_distributed_matmul(info, device, out):
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    A, B = rng.randn(4, 8).astype(np.float32), rng.randn(8, 6).astype(np.float32)
    mesh = "[" + ",".join(str(i) for i in range(w)) + "]"

    def run(a_spec, b_spec, y_spec, a, b):
        g = ol.make_graph([ol.make_node("DistributedMatMul", ["a", "b"], ["y"], domain="com.microsoft",
                                        input_device_mesh_elements=[mesh, mesh], input_device_mesh_shapes=[f"[{w}]", f"[{w}]"],
                                        input_shard_specs=[a_spec, b_spec], output_device_mesh_elements=[mesh],
                                        output_device_mesh_shapes=[f"[{w}]"], output_shard_specs=[y_spec])], "g",
                          [ol.make_tensor_value_info("a", T.FLOAT, list(a.shape)), ol.make_tensor_value_info("b", T.FLOAT, list(b.shape))],
                          [ol.make_tensor_value_info("y", T.FLOAT, None)])
        return torch.from_numpy(session(ol.make_model(g).serialize(), info, device).run(None, {"a": a, "b": b})[0])
    res = {
        "col": run("RR", "RS[0]", "RS[0]", A, np.split(B, w, 1)[r].copy()),
        "row": run("RS[0]", "S[0]R", "RR", np.split(A, w, 1)[r].copy(), np.split(B, w, 0)[r].copy()),
        "reshard": run("S[0]R", "RS[0]", "RR", np.split(A, w, 0)[r].copy(), np.split(B, w, 1)[r].copy()),
        "full": torch.from_numpy(A @ B),
    }
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_sharded_moe(info, device, out):
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    Tn, H, I, E, k = 16, 32, 64, 4 * w, 2
    x = rng.randn(Tn, H).astype(np.float32)
    logits = rng.randn(Tn, E).astype(np.float32)
    fc1, fc2, fc3 = rng.randn(E, H, I).astype(np.float32) * 0.1, rng.randn(E, I, H).astype(np.float32) * 0.1, rng.randn(E, H, I).astype(np.float32) * 0.1
    el = E // w
    sl = slice(r * el, (r + 1) * el)
    g = ol.make_graph([ol.make_node("ShardedMoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k,
                                    activation_type="silu", normalize_routing_weights=1, local_experts_start_index=r * el)], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT, [Tn, E])],
                      [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_tensor("fc1", fc1[sl]), ol.make_tensor("fc2", fc2[sl]), ol.make_tensor("fc3", fc3[sl])])
    y = session(ol.make_model(g).serialize(), info, device).run(None, {"x": x, "p": logits})[0]
    # single-device MoE on the full expert set (new weight layout [E, I, H] / [E, H, I])
    g2 = ol.make_graph([ol.make_node("MoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k,
                                     activation_type="silu", normalize_routing_weights=1)], "g",
                       [ol.make_tensor_value_info("x", T.FLOAT, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT, [Tn, E])],
                       [ol.make_tensor_value_info("y", T.FLOAT, None)],
                       [ol.make_tensor("fc1", fc1.transpose(0, 2, 1).copy()), ol.make_tensor("fc2", fc2.transpose(0, 2, 1).copy()),
                        ol.make_tensor("fc3", fc3.transpose(0, 2, 1).copy())])
    ref = ort.InferenceSession(ol.make_model(g2).serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x, "p": logits})[0]
    torch.save({"y": torch.from_numpy(y), "ref": torch.from_numpy(ref)}, os.path.join(out, f"rank{r}.pt"))


def case_sharded_moe_tokens(info, device, out):
    """ShardedMoE with tokens_sharded = 1: every rank feeds its own tokens; the rows travel to the experts' ranks and back."""
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    Tn, H, I, E, k = 10, 16, 24, 3 * w, 2
    x_all = rng.randn(w, Tn, H).astype(np.float32)
    logits_all = np.stack([np.stack([rng.permutation(np.linspace(-2.0, 2.0, E)) for _ in range(Tn)]) for _ in range(w)]).astype(np.float32)
    logits_all[0, :, :] = logits_all[0, :, ::-1] if w > 1 else logits_all[0]
    fc1, fc2, fc3 = rng.randn(E, H, I).astype(np.float32) * 0.2, rng.randn(E, I, H).astype(np.float32) * 0.2, rng.randn(E, H, I).astype(np.float32) * 0.2
    el = E // w
    sl = slice(r * el, (r + 1) * el)
    g = ol.make_graph([ol.make_node("ShardedMoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k, activation_type="silu",
                                    normalize_routing_weights=1, local_experts_start_index=r * el, tokens_sharded=1)], "g",
                      [ol.make_tensor_value_info("x", T.FLOAT, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT, [Tn, E])],
                      [ol.make_tensor_value_info("y", T.FLOAT, None)],
                      [ol.make_tensor("fc1", fc1[sl]), ol.make_tensor("fc2", fc2[sl]), ol.make_tensor("fc3", fc3[sl])])
    y = session(ol.make_model(g).serialize(), info, device).run(None, {"x": x_all[r], "p": logits_all[r]})[0]
    g2 = ol.make_graph([ol.make_node("MoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k, activation_type="silu",
                                     normalize_routing_weights=1)], "g",
                       [ol.make_tensor_value_info("x", T.FLOAT, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT, [Tn, E])],
                       [ol.make_tensor_value_info("y", T.FLOAT, None)],
                       [ol.make_tensor("fc1", fc1.transpose(0, 2, 1).copy()), ol.make_tensor("fc2", fc2.transpose(0, 2, 1).copy()),
                        ol.make_tensor("fc3", fc3.transpose(0, 2, 1).copy())])
    ref = ort.InferenceSession(ol.make_model(g2).serialize(), providers=["CPUExecutionProvider"]).run(None, {"x": x_all[r], "p": logits_all[r]})[0]
    torch.save({"y": torch.from_numpy(y), "ref": torch.from_numpy(ref)}, os.path.join(out, f"rank{r}.pt"))


def case_sharded_moe_gpu(info, device, out):
    """ShardedMoE in fp16 on GPUs, with the fused cross-rank combine (symmetric workspace) and with the library all-reduce,
    against the single-device MoE on the full expert set (the design of the reference's own parity test,
    onnxruntime/test/python/transformers/sharded_moe/test_sharded_moe.py:221-336)."""
    from onnxruntime_b200.parallel import symm
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    res = {}
    ws = symm.create_workspace(64 << 20)
    for case, (Tn, H, I, E, k) in enumerate([(64, 128, 512, 4 * w, 2), (1024, 1024, 512, 8 * w, 2), (37, 256, 256, 2 * w, 3)]):
        x = (rng.randn(Tn, H) * 0.5).astype(np.float16)
        # every row a permutation of distinct values: no ties, so the top-k choice cannot depend on a tie rule
        logits = np.stack([rng.permutation(np.linspace(-2.0, 2.0, E)) for _ in range(Tn)]).astype(np.float16)
        fc1, fc2, fc3 = [(rng.randn(*s) * 0.05).astype(np.float16) for s in ((E, H, I), (E, I, H), (E, H, I))]
        el = E // w
        sl = slice(r * el, (r + 1) * el)
        g = ol.make_graph([ol.make_node("ShardedMoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k,
                                        activation_type="silu", normalize_routing_weights=1, local_experts_start_index=r * el)], "g",
                          [ol.make_tensor_value_info("x", T.FLOAT16, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT16, [Tn, E])],
                          [ol.make_tensor_value_info("y", T.FLOAT16, None)],
                          [ol.make_tensor("fc1", fc1[sl]), ol.make_tensor("fc2", fc2[sl]), ol.make_tensor("fc3", fc3[sl])])
        model = ol.make_model(g).serialize()
        fused = session(model, info, device)
        symm.attach(fused, ws)
        ys = [fused.run(None, {"x": x, "p": logits})[0] for _ in range(3)]  # both parities of the staging areas
        fused.check_device_status()
        plain = session(model, info, device)
        yp = plain.run(None, {"x": x, "p": logits})[0]
        g2 = ol.make_graph([ol.make_node("MoE", ["x", "p", "fc1", "", "fc2", "", "fc3"], ["y"], domain="com.microsoft", k=k,
                                         activation_type="silu", normalize_routing_weights=1)], "g",
                           [ol.make_tensor_value_info("x", T.FLOAT, [Tn, H]), ol.make_tensor_value_info("p", T.FLOAT, [Tn, E])],
                           [ol.make_tensor_value_info("y", T.FLOAT, None)],
                           [ol.make_tensor("fc1", fc1.transpose(0, 2, 1).astype(np.float32)), ol.make_tensor("fc2", fc2.transpose(0, 2, 1).astype(np.float32)),
                            ol.make_tensor("fc3", fc3.transpose(0, 2, 1).astype(np.float32))])
        ref = ort.InferenceSession(ol.make_model(g2).serialize(), providers=["CPUExecutionProvider"]).run(
            None, {"x": x.astype(np.float32), "p": logits.astype(np.float32)})[0]
        res[f"case{case}"] = {"fused": torch.from_numpy(ys[-1].astype(np.float32)), "plain": torch.from_numpy(yp.astype(np.float32)),
                              "ref": torch.from_numpy(ref), "stable": all(np.array_equal(ys[0], y) for y in ys[1:])}
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_mixtral_ep(info, device, out):
    """Mixtral-shaped decoder with expert parallelism (ShardedMoE per layer) against the single-rank MoE form."""
    from onnxruntime_b200.models.generation import DecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama
    r, w = info.rank, info.world_size
    cfg = LlamaConfig.tiny(dtype="fp32" if device == "cpu" else "bf16", head_dim=64, hidden_size=128, ffn_size=256, num_layers=2, num_heads=4,
                           num_kv_heads=2, max_seq_len=64)
    dev = torch.device("cpu") if device == "cpu" else torch.device("cuda", info.local_rank)
    if device == "cuda":
        torch.cuda.set_device(info.local_rank)
    model, _ = build_llama(cfg, weight_std=0.05, moe_experts=2 * w, ep_rank=r, ep_size=w)
    sess = session(model, info, device)
    if device == "cuda":
        from onnxruntime_b200.parallel import symm
        symm.attach(sess, symm.create_workspace(16 << 20))
    ids = torch.randint(0, cfg.vocab_size, (2, 17), generator=torch.Generator().manual_seed(5))
    run = DecoderRunner(sess, cfg, batch=2, max_len=64, device=dev)
    run.prefill(ids)
    res = {"logits": run.prefill_logits.float().cpu().clone(), "ops": sorted({n["op_type"] for n in sess.graph_nodes()})}
    if r == 0:
        full, _ = build_llama(cfg, weight_std=0.05, moe_experts=2 * w)
        s1 = ort.InferenceSession(full, providers=["CPUExecutionProvider"] if device == "cpu" else [("CUDAExecutionProvider", {"device_id": str(info.local_rank)})])
        r1 = DecoderRunner(s1, cfg, batch=2, max_len=64, device=dev)
        r1.prefill(ids)
        res["ref"] = r1.prefill_logits.float().cpu().clone()
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_llama_tp(info, device, out):
    from onnxruntime_b200.models.generation import DecoderRunner
    from onnxruntime_b200.models.llama import LlamaConfig, build_llama
    r, w = info.rank, info.world_size
    dtype = "fp32" if device == "cpu" else "bf16"
    cfg = LlamaConfig.tiny(dtype=dtype, head_dim=64, hidden_size=256, ffn_size=512, num_layers=2, num_heads=max(8, w),
                           num_kv_heads=max(4, w), max_seq_len=128)
    quant = int(os.environ.get("ORTB200_TEST_QUANT", "0"))
    model, _ = build_llama(cfg, tp_rank=r, tp_size=w, weight_std=0.05, quant_bits=quant)
    opts = {}
    if device == "cuda":
        torch.cuda.set_device(info.local_rank)
    want_fused = device == "cuda" and os.environ.get("ORTB200_TEST_FUSED", "1") == "1"
    # graph capture only with the in-kernel reduction: the decode step then contains no library collective
    providers = ["CPUExecutionProvider"] if device == "cpu" else [
        ("CUDAExecutionProvider", {"device_id": str(info.local_rank), "enable_cuda_graph": "1" if want_fused else "0"})]
    sess = ort.InferenceSession(model, providers=providers, dist=info, enable_fallback=False, **opts)
    fused = False
    if want_fused:
        from onnxruntime_b200.parallel import symm
        ws = symm.create_workspace(16 << 20)
        symm.attach(sess, ws)
        fused = True
    dev = torch.device("cpu") if device == "cpu" else torch.device("cuda", info.local_rank)
    runner = DecoderRunner(sess, cfg, batch=2, max_len=96, tp_size=w, device=dev)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (2, 40))
    first = runner.prefill(ids)
    logits = []
    tok = first.clone()
    for _ in range(6):
        tok = runner.decode_step(tok).clone()
        logits.append(runner.step_logits.float().cpu().clone())
    if device == "cuda":
        torch.cuda.synchronize()
        sess.check_device_status()
    ops = sorted({n["op_type"] for n in sess.graph_nodes()})
    res = {"logits": torch.stack(logits), "ops": ops, "fused": fused}
    if r == 0:
        # single-rank run of the unsharded model for comparison
        full, _ = build_llama(cfg, weight_std=0.05, quant_bits=quant)
        s1 = ort.InferenceSession(full, providers=["CPUExecutionProvider"] if device == "cpu" else [("CUDAExecutionProvider", {"device_id": str(info.local_rank)})],
                                  enable_fallback=False)
        r1 = DecoderRunner(s1, cfg, batch=2, max_len=96, device=dev)
        t1 = r1.prefill(ids)
        ref = []
        tok = first.clone()
        for _ in range(6):
            r1.decode_step(tok)
            ref.append(r1.step_logits.float().cpu().clone())
            tok = torch.stack(logits)[len(ref) - 1].argmax(-1)  # follow the TP run's tokens so the caches stay comparable
            tok = tok.to(dev)
        res["ref"] = torch.stack(ref)
        res["first_equal"] = bool(torch.equal(t1.cpu(), first.cpu()))
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_gemm_allreduce(info, device, out):
    """The fused GEMM + all-reduce kernel against a process-group all-reduce of the per-rank products."""
    from onnxruntime_b200.ops import _kernels as K
    from onnxruntime_b200.parallel import symm
    r, w = info.rank, info.world_size
    torch.cuda.set_device(info.local_rank)
    ws = symm.create_workspace(64 << 20)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = {}
    # decode-sized problems reduce inside the GEMM kernel; the prompt-sized ones (M > 64) push their product into the
    # all-reduce scatter areas from the CTA-pair kernel's epilogue and a reduction kernel finishes them
    for i, (M, N, Kd) in enumerate([(8, 4096, 512), (8, 1024, 1792), (16, 2048, 256), (1, 512, 128), (33, 768, 512),
                                    (1024, 2048, 512), (700, 1000, 256), (2048, 512, 1024)]):
        g = torch.Generator(device="cuda").manual_seed(100 * i + r)
        x = (torch.randn(M, Kd, device="cuda", generator=g) * 0.5).bfloat16()
        wt = (torch.randn(N, Kd, device="cuda", generator=g) * 0.05).bfloat16()
        resid = torch.randn(M, N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7 + i)).bfloat16()
        outs = []
        for rep in range(3):  # consecutive launches exercise the epoch / double-buffer protocol
            outs.append(K.gemm(x, wt, residual=resid, status=status, peers=ws.peer_ptrs, rank=r, symm_bytes=ws.nbytes).clone())
        ref = (x.float() @ wt.float().T)
        dist.all_reduce(ref)
        ref = ref + resid.float()
        torch.cuda.synchronize()
        res[f"case{i}"] = {"err": float((outs[-1].float() - ref).abs().max() / ref.abs().max()),
                           "stable": bool(torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])), "out": outs[-1].cpu()}
        if M > 64 and ws.multicast_ptr:
            # the same problem reduced through the switch (multimem.ld_reduce / multimem.st)
            outs = [K.gemm(x, wt, residual=resid, status=status, peers=ws.peer_ptrs, rank=r, symm_bytes=ws.nbytes,
                           mc_ptr=ws.multicast_ptr).clone() for _ in range(3)]
            torch.cuda.synchronize()
            res[f"case{i}_nvls"] = {"err": float((outs[-1].float() - ref).abs().max() / ref.abs().max()),
                                    "stable": bool(torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])), "out": outs[-1].cpu()}
    res["nvls"] = bool(ws.multicast_ptr)
    res["status"] = int(status.item())
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_symm_collectives(info, device, out):
    """The one-kernel collectives over peer-mapped memory against the process group's results."""
    from onnxruntime_b200.ops import _kernels as K
    from onnxruntime_b200.parallel import symm
    r, w = info.rank, info.world_size
    torch.cuda.set_device(info.local_rank)
    ws = symm.create_workspace(32 << 20)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = {}
    g = torch.Generator(device="cuda").manual_seed(1000 + r)
    for rep in range(3):  # repeated calls walk through both parities of the staging areas
        for dtype in (torch.bfloat16, torch.float32):
            for n in (8, 4096, 100000, 262144):
                x = torch.randn(n, device="cuda", generator=g).to(dtype)
                y = K.symm_collective("allreduce", x, ws.peer_ptrs, r, ws.nbytes, status=status)
                ref = x.float().clone()
                dist.all_reduce(ref)
                res[f"ar_{rep}_{dtype}_{n}"] = float((y.float() - ref).abs().max() / ref.abs().max())
                if ws.multicast_ptr:
                    y = K.symm_collective("allreduce", x, ws.peer_ptrs, r, ws.nbytes, status=status, mc_ptr=ws.multicast_ptr)
                    res[f"ar_nvls_{rep}_{dtype}_{n}"] = float((y.float() - ref).abs().max() / ref.abs().max())
        for shape, axis in (((8, 16032), 1), ((4, 3, 64), 0), ((2, 5, 128), 2), ((1, 8), 0)):
            x = torch.randn(*shape, device="cuda", generator=g).bfloat16()
            y = K.symm_collective("allgather", x, ws.peer_ptrs, r, ws.nbytes, axis=axis, status=status)
            parts = [torch.empty_like(x) for _ in range(w)]
            dist.all_gather(parts, x)
            res[f"ag_{rep}_{shape}"] = bool(torch.equal(y, torch.cat(parts, axis)))
        x = torch.randn(w * 3, 40, device="cuda", generator=g).half()
        y = K.symm_collective("alltoall", x, ws.peer_ptrs, r, ws.nbytes, status=status)
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        res[f"a2a_{rep}"] = bool(torch.equal(y, ref))
    torch.cuda.synchronize()
    res["status"] = int(status.item())
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_allgather_gemm(info, device, out):
    """All-gather -> GEMM as one kernel against the process group's all-gather followed by a matmul, with device times
    of both (CUDA events, max over ranks is taken by the caller)."""
    from onnxruntime_b200.ops import _kernels as K
    from onnxruntime_b200.parallel import symm
    r, w = info.rank, info.world_size
    torch.cuda.set_device(info.local_rank)
    ws = symm.create_workspace(1 << 30)   # gather areas are an eighth of it: 8192 x 8192 bf16 rows fit
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = {}
    g = torch.Generator(device="cuda").manual_seed(7 + r)
    gw = torch.Generator(device="cuda").manual_seed(99 + r)
    for rep in range(2):   # both parities of the gather areas
        for rows, N, Kd, act in ((96, 384, 512, "none"), (320, 256, 1024, "gelu"), (1024, 2048, 4096, "none")):
            x = (torch.randn(rows, Kd, device="cuda", generator=g) * 0.5).bfloat16()
            wt = (torch.randn(N, Kd, device="cuda", generator=gw) * 0.05).bfloat16()
            bias = torch.randn(N, device="cuda", generator=gw).bfloat16()
            y = K.allgather_gemm(x, wt, ws.peer_ptrs, r, ws.nbytes, bias=bias, act=act, status=status)
            parts = [torch.empty_like(x) for _ in range(w)]
            dist.all_gather(parts, x)
            ref = torch.cat(parts).float() @ wt.float().t() + bias.float()
            if act == "gelu":
                ref = torch.nn.functional.gelu(ref)
            res[f"agg_{rep}_{rows}_{N}_{Kd}"] = float((y.float() - ref).abs().max() / ref.abs().max())
    # timing: the shape of a sequence-parallel projection (8192 tokens in all, hidden 8192, this rank's 4096 output features)
    rows, N, Kd = 8192 // w, 4096, 8192
    x = (torch.randn(rows, Kd, device="cuda", generator=g) * 0.5).bfloat16()
    wt = (torch.randn(N, Kd, device="cuda", generator=gw) * 0.05).bfloat16()
    full = torch.empty(w * rows, Kd, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / iters

    def fused():
        return K.allgather_gemm(x, wt, ws.peer_ptrs, r, ws.nbytes, status=status)

    def library():
        dist.all_gather_into_tensor(full, x)
        return K.gemm(full, wt)

    res["ms_fused"] = timed(fused)
    res["ms_library"] = timed(library)
    res["ms_gemm_only"] = timed(lambda: K.gemm(full, wt))
    res["same"] = float((fused().float() - library().float()).abs().max())
    torch.cuda.synchronize()
    res["status"] = int(status.item())
    torch.save(res, os.path.join(out, f"rank{r}.pt"))


def case_data_parallel_training(info, device, out):
    """Each rank trains on its shard of the batch: (a) the training API with bucketed gradient all-reduce, (b) ORTModule
    under torch's DistributedDataParallel.  Both must follow the single-process full-batch run."""
    from onnxruntime_b200 import training
    from onnxruntime_b200.training import api
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    f = lambda *s: (rng.randn(*s) * 0.4).astype(np.float32)  # noqa: E731
    init = {"w1": f(8, 16), "b1": f(16), "w2": f(16, 5)}
    g = ol.make_graph([ol.make_node("MatMul", ["x", "w1"], ["h"]), ol.make_node("Add", ["h", "b1"], ["hb"]), ol.make_node("Tanh", ["hb"], ["t"]),
                       ol.make_node("MatMul", ["t", "w2"], ["logits"])], "mlp", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 8])],
                      [ol.make_tensor_value_info("logits", T.FLOAT, ["n", 5])], [ol.make_tensor(k, v) for k, v in init.items()])
    model = ol.make_model(g, opset=17)
    per = 8
    x_all, y_all = f(w * per, 8), rng.randint(0, 5, w * per).astype(np.int64)
    xs, ys = x_all[r * per:(r + 1) * per], y_all[r * per:(r + 1) * per]
    art = training.generate_artifacts(model, loss=training.LossType.CrossEntropyLoss, optimizer=training.OptimType.AdamW, target_name="labels",
                                      optimizer_options={"weight_decay": 0.0})
    state = api.CheckpointState.load_checkpoint(art["checkpoint"])
    module = api.Module(art["training_model.onnx"], state)
    optim = api.Optimizer(art["optimizer_model.onnx"], module)
    optim.set_learning_rate(0.05)
    for _ in range(5):
        module(xs, ys)
        module.all_reduce_gradients(bucket_bytes=300)      # small buckets: more than one collective per step
        optim.step()
        module.lazy_reset_grad()
    # single-process full batch in torch
    ref = {k: torch.tensor(v, requires_grad=True) for k, v in init.items()}
    topt = torch.optim.AdamW(list(ref.values()), lr=0.05, weight_decay=0.0)
    for _ in range(5):
        topt.zero_grad()
        logits = torch.tanh(torch.tensor(x_all) @ ref["w1"] + ref["b1"]) @ ref["w2"]
        torch.nn.functional.cross_entropy(logits, torch.tensor(y_all)).backward()
        topt.step()
    # (b) ORTModule under DDP: one backward pass, gradients averaged by DDP's own buckets
    ddp = torch.nn.parallel.DistributedDataParallel(training.ORTModule(model))
    torch.nn.functional.cross_entropy(ddp(torch.tensor(xs)), torch.tensor(ys)).backward()
    full = {k: torch.tensor(v, requires_grad=True) for k, v in init.items()}
    logits = torch.tanh(torch.tensor(x_all) @ full["w1"] + full["b1"]) @ full["w2"]
    torch.nn.functional.cross_entropy(logits, torch.tensor(y_all)).backward()
    torch.save({"api": {k: p.data.clone() for k, p in state.parameters.items()}, "ref": {k: v.detach() for k, v in ref.items()},
                "ddp_grad": {n: p.grad.clone() for n, p in ddp.module.named_onnx_parameters()},
                "full_grad": {k: v.grad for k, v in full.items()}}, os.path.join(out, f"rank{r}.pt"))


def case_megatron_training(info, device, out):
    """Column-parallel then row-parallel MLP with MegatronF / MegatronG: loss and gradients against the unsplit model."""
    from onnxruntime_b200 import training
    r, w = info.rank, info.world_size
    rng = np.random.RandomState(0)
    f = lambda *s: (rng.randn(*s) * 0.4).astype(np.float32)  # noqa: E731
    init = {"w0": f(8, 8), "w1": f(8, 16), "b1": f(16), "w2": f(16, 8)}
    g = ol.make_graph([ol.make_node("MatMul", ["x", "w0"], ["h0"]), ol.make_node("MatMul", ["h0", "w1"], ["h"]), ol.make_node("Add", ["h", "b1"], ["hb"]),
                       ol.make_node("Tanh", ["hb"], ["t"]), ol.make_node("MatMul", ["t", "w2"], ["y"])], "mlp",
                      [ol.make_tensor_value_info("x", T.FLOAT, ["n", 8])], [ol.make_tensor_value_info("y", T.FLOAT, ["n", 8])],
                      [ol.make_tensor(k, v) for k, v in init.items()])
    x, target = torch.tensor(f(6, 8)), torch.tensor(f(6, 8))
    sharded = training.megatron.shard_mlp(ol.make_model(g, opset=17), ["w1"], ["w2"], r, w, column_biases=["b1"])
    mod = training.ORTModule(sharded)
    loss = ((mod(x) - target) ** 2).mean()
    loss.backward()
    ref = {k: torch.tensor(v, requires_grad=True) for k, v in init.items()}
    ref_loss = (((torch.tanh(x @ ref["w0"] @ ref["w1"] + ref["b1"]) @ ref["w2"]) - target) ** 2).mean()
    ref_loss.backward()
    torch.save({"loss": loss.detach(), "ref_loss": ref_loss.detach(), "grads": {n: p.grad.clone() for n, p in mod.named_onnx_parameters()},
                "ref_grads": {k: v.grad for k, v in ref.items()}}, os.path.join(out, f"rank{r}.pt"))


def main():
    case, device, out = sys.argv[1], sys.argv[2], sys.argv[3]
    info = init_distributed("gloo" if device == "cpu" else "nccl", timeout_s=120)
    try:
        globals()[f"case_{case}"](info, device, out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
