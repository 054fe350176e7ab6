"""Training: gradient graph against autograd, the autograd-tape module, artifacts + the on-device training API.
Oracles are plain PyTorch fp32 restatements of the same models."""
import os

import numpy as np
import pytest
import torch

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol
from onnxruntime_b200 import training
from onnxruntime_b200.training import api

T = ol.TensorProto


def _block_model(rng):
    """x [n, 8] -> LayerNorm -> MatMul + bias -> Gelu(tanh) -> residual Gemm -> logits [n, 5]; a value used twice."""
    f = lambda *s: (rng.standard_normal(s) * 0.4).astype(np.float32)  # noqa: E731
    init = {"ln_w": 1 + f(8), "ln_b": f(8), "w1": f(8, 16), "b1": f(16), "w2": f(5, 16), "b2": f(5), "w3": f(8, 5)}
    nodes = [
        ol.make_node("LayerNormalization", ["x", "ln_w", "ln_b"], ["h0"], axis=-1, epsilon=1e-5),
        ol.make_node("MatMul", ["h0", "w1"], ["h1"]),
        ol.make_node("Add", ["h1", "b1"], ["h2"]),
        ol.make_node("FastGelu", ["h2"], ["h3"], domain="com.microsoft"),
        ol.make_node("Gemm", ["h3", "w2", "b2"], ["h4"], transB=1, alpha=0.5),
        ol.make_node("MatMul", ["h0", "w3"], ["skip"]),
        ol.make_node("Add", ["h4", "skip"], ["logits"]),
    ]
    g = ol.make_graph(nodes, "block", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 8])],
                      [ol.make_tensor_value_info("logits", T.FLOAT, ["n", 5])], [ol.make_tensor(k, v) for k, v in init.items()])
    return ol.make_model(g, opset=17), init


def _torch_block(p, x):
    h0 = torch.nn.functional.layer_norm(x, (8,), p["ln_w"], p["ln_b"], 1e-5)
    h3 = torch.nn.functional.gelu(h0 @ p["w1"] + p["b1"], approximate="tanh")
    return 0.5 * (h3 @ p["w2"].T) + p["b2"] + h0 @ p["w3"]


def test_gradient_graph_matches_autograd():
    rng = np.random.default_rng(0)
    model, init = _block_model(rng)
    model.graph.inputs.append(ol.make_tensor_value_info("labels", T.INT64, ["n"]))
    model.graph.nodes.append(ol.make_node("SoftmaxCrossEntropyLoss", ["logits", "labels"], ["loss"], reduction="mean"))
    model.graph.outputs[:] = [ol.make_tensor_value_info("loss", T.FLOAT, [])]
    grad_model = training.build_gradient_graph(model, list(init), "loss", input_grads=["x"])
    x = rng.standard_normal((6, 8)).astype(np.float32)
    y = rng.integers(0, 5, 6).astype(np.int64)
    sess = ort.InferenceSession(grad_model.serialize(), providers=["CPUExecutionProvider"])
    names = [o.name for o in sess.get_outputs()]
    got = dict(zip(names, sess.run(None, {"x": x, "labels": y})))
    p = {k: torch.tensor(v, requires_grad=True) for k, v in init.items()}
    xt = torch.tensor(x, requires_grad=True)
    loss = torch.nn.functional.cross_entropy(_torch_block(p, xt), torch.tensor(y))
    loss.backward()
    assert abs(float(got["loss"]) - float(loss.detach())) < 1e-5
    for k in init:
        np.testing.assert_allclose(got[k + "_grad"], p[k].grad.numpy(), rtol=2e-4, atol=2e-5, err_msg=k)
    np.testing.assert_allclose(got["x_grad"], xt.grad.numpy(), rtol=2e-4, atol=2e-5)


def test_gradient_rules_of_shape_and_movement_operators():
    """Transpose, Reshape, Softmax, Slice, Concat, Gather, ReduceMean, Mul / Div / Sub with broadcasting, Where, Sqrt."""
    rng = np.random.default_rng(1)
    w = rng.standard_normal((4, 6)).astype(np.float32)
    c = (rng.random((6,)) + 0.5).astype(np.float32)
    nodes = [
        ol.make_node("Transpose", ["w"], ["wt"], perm=[1, 0]),                      # [6, 4]
        ol.make_node("Softmax", ["wt"], ["sm"], axis=-1),
        ol.make_node("Slice", ["sm", "s_start", "s_end", "s_axes"], ["sl"]),        # [6, 2]
        ol.make_node("Concat", ["sl", "wt"], ["cat"], axis=1),                      # [6, 6]
        ol.make_node("Gather", ["cat", "idx"], ["gat"], axis=0),                    # [3, 6]
        ol.make_node("Div", ["gat", "c"], ["dv"]),
        ol.make_node("Mul", ["dv", "dv"], ["sq"]),
        ol.make_node("Sqrt", ["sq_eps"], ["rt"]),
        ol.make_node("Add", ["sq", "eps"], ["sq_eps"]),
        ol.make_node("Greater", ["gat", "zero"], ["pos"]),
        ol.make_node("Where", ["pos", "rt", "sq"], ["wh"]),
        ol.make_node("Reshape", ["wh", "flat"], ["rs"]),
        ol.make_node("ReduceMean", ["rs"], ["loss"], keepdims=0),
    ]
    nodes[7], nodes[8] = nodes[8], nodes[7]
    i64 = lambda *v: np.asarray(v, dtype=np.int64)  # noqa: E731
    inits = [ol.make_tensor("w", w), ol.make_tensor("c", c), ol.make_tensor("s_start", i64(1)), ol.make_tensor("s_end", i64(3)),
             ol.make_tensor("s_axes", i64(1)), ol.make_tensor("idx", i64(5, 0, 5)), ol.make_tensor("eps", np.float32(1e-3)),
             ol.make_tensor("zero", np.float32(0)), ol.make_tensor("flat", i64(-1))]
    g = ol.make_graph(nodes, "g", [], [ol.make_tensor_value_info("loss", T.FLOAT, [])], inits)
    gm = training.build_gradient_graph(ol.make_model(g, opset=17), ["w", "c"], "loss")
    sess = ort.InferenceSession(training.ortmodule.lift_initializers(gm, ["w", "c"]).serialize(), providers=["CPUExecutionProvider"])
    got = dict(zip([o.name for o in sess.get_outputs()], sess.run(None, {"w": w, "c": c})))
    wt_, ct_ = torch.tensor(w, requires_grad=True), torch.tensor(c, requires_grad=True)
    wt = wt_.T
    cat = torch.cat([torch.softmax(wt, -1)[:, 1:3], wt], 1)
    gat = cat[torch.tensor([5, 0, 5])]
    sq = (gat / ct_) ** 2
    loss = torch.where(gat > 0, torch.sqrt(sq + 1e-3), sq).reshape(-1).mean()
    loss.backward()
    assert abs(float(got["loss"]) - float(loss.detach())) < 1e-5
    np.testing.assert_allclose(got["w_grad"], wt_.grad.numpy(), rtol=2e-4, atol=2e-6)
    np.testing.assert_allclose(got["c_grad"], ct_.grad.numpy(), rtol=2e-4, atol=2e-6)


def test_unsupported_operator_is_named():
    g = ol.make_graph([ol.make_node("Erf", ["w"], ["y"]), ol.make_node("ReduceSum", ["y"], ["loss"], keepdims=0)], "g", [],
                      [ol.make_tensor_value_info("loss", T.FLOAT, [])], [ol.make_tensor("w", np.ones((2, 2), np.float32))])
    with pytest.raises(NotImplementedError, match="Erf"):
        training.build_gradient_graph(ol.make_model(g, opset=17), ["w"], "loss", recompute_fallback=False)


def test_operators_without_a_rule_are_differentiated_by_recomputation():
    """MaxPool, BatchNormalization (inference form), AveragePool and Erf have no rule: NodeGrad re-runs and differentiates them."""
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((4, 3, 3, 3)) * 0.3).astype(np.float32)
    bn = [(rng.random(4) + 0.5).astype(np.float32), _f(rng, 4) * 0.1, _f(rng, 4) * 0.1, (rng.random(4) + 0.5).astype(np.float32)]
    nodes = [ol.make_node("Conv", ["x", "w"], ["c"], pads=[1, 1, 1, 1]),
             ol.make_node("BatchNormalization", ["c", "bn_s", "bn_b", "bn_m", "bn_v"], ["n"], epsilon=1e-5),
             ol.make_node("MaxPool", ["n"], ["p"], kernel_shape=[2, 2], strides=[2, 2]),
             ol.make_node("AveragePool", ["p"], ["a"], kernel_shape=[2, 2], strides=[1, 1]),
             ol.make_node("Erf", ["a"], ["e"]), ol.make_node("ReduceSum", ["e"], ["loss"], keepdims=0)]
    inits = [ol.make_tensor("w", w)] + [ol.make_tensor(k, v) for k, v in zip(("bn_s", "bn_b", "bn_m", "bn_v"), bn)]
    g = ol.make_graph(nodes, "cnn", [ol.make_tensor_value_info("x", T.FLOAT, [2, 3, 8, 8])], [ol.make_tensor_value_info("loss", T.FLOAT, [])], inits)
    gm = training.build_gradient_graph(ol.make_model(g, opset=17), ["w", "bn_s", "bn_b"], "loss", input_grads=["x"])
    assert sum(n.op_type == "NodeGrad" for n in gm.graph.nodes) == 4
    x = _f(rng, 2, 3, 8, 8)
    sess = ort.InferenceSession(gm.serialize(), providers=["CPUExecutionProvider"])
    got = dict(zip([o.name for o in sess.get_outputs()], sess.run(None, {"x": x})))
    xt, wt = torch.tensor(x, requires_grad=True), torch.tensor(w, requires_grad=True)
    st, bt = torch.tensor(bn[0], requires_grad=True), torch.tensor(bn[1], requires_grad=True)
    c = torch.nn.functional.conv2d(xt, wt, padding=1)
    n = torch.nn.functional.batch_norm(c, torch.tensor(bn[2]), torch.tensor(bn[3]), st, bt, training=False, eps=1e-5)
    loss = torch.erf(torch.nn.functional.avg_pool2d(torch.nn.functional.max_pool2d(n, 2, 2), 2, 1)).sum()
    loss.backward()
    assert abs(float(got["loss"]) - loss.item()) < 1e-4
    for name, ref in (("w", wt), ("bn_s", st), ("bn_b", bt), ("x", xt)):
        np.testing.assert_allclose(got[name + "_grad"], ref.grad.numpy(), rtol=1e-3, atol=1e-5, err_msg=name)


def test_ortmodule_trains_with_a_torch_optimizer():
    rng = np.random.default_rng(2)
    model, init = _block_model(rng)
    mod = training.ORTModule(model)
    assert sorted(n for n, _ in mod.named_onnx_parameters()) == sorted(init)
    x = torch.tensor(rng.standard_normal((32, 8)).astype(np.float32))
    y = torch.tensor(rng.integers(0, 5, 32))
    ref = {k: torch.tensor(v, requires_grad=True) for k, v in init.items()}
    loss = torch.nn.functional.cross_entropy(mod(x), y)
    loss.backward()
    torch.nn.functional.cross_entropy(_torch_block(ref, x), y).backward()
    for name, p in mod.named_onnx_parameters():
        np.testing.assert_allclose(p.grad.numpy(), ref[name].grad.numpy(), rtol=2e-4, atol=2e-5, err_msg=name)
    opt = torch.optim.AdamW(mod.parameters(), lr=0.05)
    first = float(loss.detach())
    for _ in range(30):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(mod(x), y)
        loss.backward()
        opt.step()
    assert float(loss.detach()) < 0.5 * first


def test_artifacts_and_training_api(tmp_path):
    rng = np.random.default_rng(3)
    model, init = _block_model(rng)
    art = training.generate_artifacts(model, frozen_params=["w3"], loss=training.LossType.CrossEntropyLoss,
                                      optimizer=training.OptimType.AdamW, artifact_directory=str(tmp_path), target_name="labels",
                                      optimizer_options={"weight_decay": 0.0})
    assert set(os.listdir(tmp_path)) == {"training_model.onnx", "eval_model.onnx", "optimizer_model.onnx", "checkpoint"}
    state = api.CheckpointState.load_checkpoint(str(tmp_path / "checkpoint"))
    assert not state.parameters["w3"].requires_grad and state.parameters["w1"].requires_grad
    module = api.Module(str(tmp_path / "training_model.onnx"), state, str(tmp_path / "eval_model.onnx"))
    optim = api.Optimizer(art["optimizer_model.onnx"], module)
    optim.set_learning_rate(0.05)
    assert module.input_names() == ["x", "labels"]
    x = rng.standard_normal((32, 8)).astype(np.float32)
    y = rng.integers(0, 5, 32).astype(np.int64)
    # the same steps in torch: AdamW without decay, w3 frozen
    ref = {k: torch.tensor(v, requires_grad=(k != "w3")) for k, v in init.items()}
    topt = torch.optim.AdamW([v for k, v in ref.items() if k != "w3"], lr=0.05, weight_decay=0.0)
    losses = []
    for step in range(12):
        module.train()
        loss, _logits = module(x, y)           # the loss comes first, the forward model's own outputs follow
        losses.append(float(np.asarray(loss).reshape(-1)[0]))
        if step == 0:   # accumulation: a second pass without reset doubles the buffer
            g1 = state.parameters["w1"].grad.clone()
            module(x, y)
            np.testing.assert_allclose(state.parameters["w1"].grad.numpy(), 2 * g1.numpy(), rtol=1e-5)
            module.lazy_reset_grad()
            module(x, y)
            np.testing.assert_allclose(state.parameters["w1"].grad.numpy(), g1.numpy(), rtol=1e-5)
        optim.step()
        module.lazy_reset_grad()
        topt.zero_grad()
        tl = torch.nn.functional.cross_entropy(_torch_block(ref, torch.tensor(x)), torch.tensor(y))
        tl.backward()
        topt.step()
        assert abs(losses[-1] - tl.item()) < 2e-4 * max(1.0, abs(tl.item())), (step, losses[-1], tl.item())
    assert losses[-1] < 0.6 * losses[0]
    np.testing.assert_allclose(state.parameters["w1"].data.numpy(), ref["w1"].detach().numpy(), rtol=2e-3, atol=2e-4)
    np.testing.assert_array_equal(state.parameters["w3"].data.numpy(), init["w3"])
    # eval mode, checkpoint round trip (with optimizer state), export for inference
    module.eval()
    ev = module(x, y)
    ev_loss = float(np.asarray(ev[0] if isinstance(ev, tuple) else ev).reshape(-1)[0])
    api.CheckpointState.save_checkpoint(state, str(tmp_path / "ckpt2"))
    again = api.CheckpointState.load_checkpoint(str(tmp_path / "ckpt2"))
    assert again.optimizer_step == 12 and abs(again.learning_rate - 0.05) < 1e-9
    np.testing.assert_array_equal(again.parameters["w2"].data.numpy(), state.parameters["w2"].data.numpy())
    np.testing.assert_array_equal(again.optimizer["momentum1"]["w1"].numpy(), state.optimizer["momentum1"]["w1"].numpy())
    module.export_model_for_inferencing(str(tmp_path / "infer.onnx"), ["logits"])
    (logits,) = ort.InferenceSession(str(tmp_path / "infer.onnx"), providers=["CPUExecutionProvider"]).run(None, {"x": x})
    assert abs(float(torch.nn.functional.cross_entropy(torch.tensor(logits), torch.tensor(y))) - ev_loss) < 1e-5
    sched = api.LinearLRScheduler(optim, warmup_step_count=2, total_step_count=10, initial_lr=0.1)
    rates = []
    for _ in range(10):
        rates.append(optim.get_learning_rate())
        sched.step()
    assert rates[0] == 0.0 and abs(rates[2] - 0.1) < 1e-9 and rates[-1] < rates[3] and optim.get_learning_rate() == 0.0


# ---- single training operators against autograd -------------------------------------------------------------------
from helpers import run_node as _run_named  # noqa: E402

MS = "com.microsoft"


def run_node(op, inputs, **kw):
    return _run_named(op, {f"in{i}": (np.asarray(v) if not isinstance(v, (list, type(None))) else v) for i, v in enumerate(inputs)}, **kw)


def _f(rng, *s):
    return rng.standard_normal(s).astype(np.float32)


def test_activation_and_softmax_grad_ops():
    rng = np.random.default_rng(5)
    x, dy = _f(rng, 4, 7), _f(rng, 4, 7)
    cases = {
        "GeluGrad": (lambda t: torch.nn.functional.gelu(t), "x", {}),
        "FastGeluGrad": (lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "x", {}),
        "QuickGeluGrad": (lambda t: t * torch.sigmoid(1.702 * t), "x", {"alpha": 1.702}),
        "ReluGrad": (torch.relu, "x", {}),
        "SigmoidGrad": (torch.sigmoid, "y", {}),
        "TanhGrad": (torch.tanh, "y", {}),
        "LeakyReluGrad": (lambda t: torch.nn.functional.leaky_relu(t, 0.1), "y", {"alpha": 0.1}),
        "SoftmaxGrad_13": (lambda t: torch.softmax(t, 0), "y", {"axis": 0}),
        "LogSoftmaxGrad_13": (lambda t: torch.log_softmax(t, -1), "y", {"axis": -1}),
        "SoftmaxGrad": (lambda t: torch.softmax(t.reshape(-1), 0).reshape(t.shape), "y", {"axis": 0}),
    }
    for op, (fn, second, attrs) in cases.items():
        xt = torch.tensor(x, requires_grad=True)
        y = fn(xt)
        y.backward(torch.tensor(dy))
        (got,) = run_node(op, [dy, x if second == "x" else y.detach().numpy()], domain=MS, **attrs)
        np.testing.assert_allclose(got, xt.grad.numpy(), rtol=1e-4, atol=1e-5, err_msg=op)
    b = _f(rng, 7)
    for op, approx in (("BiasGeluGrad_dX", "none"), ("BiasFastGeluGrad_dX", "tanh")):
        xt = torch.tensor(x, requires_grad=True)
        torch.nn.functional.gelu(xt + torch.tensor(b), approximate=approx).backward(torch.tensor(dy))
        (got,) = run_node(op, [dy, x, b], domain=MS)
        np.testing.assert_allclose(got, xt.grad.numpy(), rtol=1e-4, atol=1e-5, err_msg=op)


def test_conv_batchnorm_and_simplified_layernorm_grad_ops():
    rng = np.random.default_rng(6)
    x, w, b = _f(rng, 2, 4, 9, 9), _f(rng, 6, 2, 3, 3), _f(rng, 6)
    xt, wt, bt = (torch.tensor(v, requires_grad=True) for v in (x, w, b))
    y = torch.nn.functional.conv2d(xt, wt, bt, stride=2, padding=1, groups=2)
    dy = _f(rng, *y.shape)
    y.backward(torch.tensor(dy))
    dx, dw, db = run_node("ConvGrad", [dy, x, w], domain=MS, n_outputs=3, strides=[2, 2], pads=[1, 1, 1, 1], group=2, kernel_shape=[3, 3])
    for got, ref in ((dx, xt), (dw, wt), (db, bt)):
        np.testing.assert_allclose(got, ref.grad.numpy(), rtol=1e-3, atol=1e-4)
    # batch normalisation in training form: saved mean / variance of the batch
    x, scale = _f(rng, 5, 3, 4), (rng.random(3) + 0.5).astype(np.float32)
    xt, st, bt = torch.tensor(x, requires_grad=True), torch.tensor(scale, requires_grad=True), torch.zeros(3, requires_grad=True)
    y = torch.nn.functional.batch_norm(xt, None, None, st, bt, training=True, eps=1e-5)
    dy = _f(rng, *y.shape)
    y.backward(torch.tensor(dy))
    mean, var = x.mean((0, 2)), x.var((0, 2))
    dx, ds, db = run_node("BatchNormalizationGrad", [dy, x, scale, mean, var], domain=MS, n_outputs=3, epsilon=1e-5)
    np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(ds, st.grad.numpy(), rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(db, bt.grad.numpy(), rtol=1e-3, atol=1e-5)
    # RMS norm
    x, scale = _f(rng, 3, 5, 8), (rng.random(8) + 0.5).astype(np.float32)
    xt, st = torch.tensor(x, requires_grad=True), torch.tensor(scale, requires_grad=True)
    inv = torch.rsqrt((xt * xt).mean(-1, keepdim=True) + 1e-6)
    y = xt * inv * st
    dy = _f(rng, *y.shape)
    y.backward(torch.tensor(dy))
    dx, ds = run_node("SimplifiedLayerNormalizationGrad", [dy, x, scale, inv.detach().numpy()], domain=MS, n_outputs=2, axis=-1)
    np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(ds, st.grad.numpy(), rtol=1e-3, atol=1e-5)


def test_movement_grad_ops_and_broadcast_helpers():
    rng = np.random.default_rng(7)
    i64 = lambda *v: np.asarray(v, dtype=np.int64)  # noqa: E731
    dy = _f(rng, 2, 3)
    (dx,) = run_node("SliceGrad", [dy, i64(4, 7), i64(3, 6), i64(0, 0), i64(0, 1), i64(-2, -2)], domain=MS)   # x[3:0:-2, 6:0:-2]
    ref = np.zeros((4, 7), np.float32)
    ref[3:0:-2, 6:0:-2] = dy
    np.testing.assert_array_equal(dx, ref)
    idx = i64(2, 0, 2).reshape(3, 1)
    upd = _f(rng, 3, 5)
    (dx,) = run_node("GatherNDGrad", [i64(4, 5), idx, upd], domain=MS, batch_dims=0)
    ref = np.zeros((4, 5), np.float32)
    np.add.at(ref, idx[:, 0], upd)
    np.testing.assert_allclose(dx, ref, rtol=1e-6)
    bidx = i64(1, 0, 2, 2).reshape(2, 2, 1)                     # batch_dims = 1 over data [2, 3, 4]
    upd = _f(rng, 2, 2, 4)
    (dx,) = run_node("GatherNDGrad", [i64(2, 3, 4), bidx, upd], domain=MS, batch_dims=1)
    ref = np.zeros((2, 3, 4), np.float32)
    for bi in range(2):
        for j in range(2):
            ref[bi, bidx[bi, j, 0]] += upd[bi, j]
    np.testing.assert_allclose(dx, ref, rtol=1e-6)
    eidx = rng.integers(0, 4, (2, 5)).astype(np.int64)
    upd = _f(rng, 2, 5)
    (dx,) = run_node("GatherElementsGrad", [upd, i64(4, 5), eidx], domain=MS, axis=0)
    np.testing.assert_allclose(dx, torch.zeros(4, 5).scatter_add_(0, torch.tensor(eidx), torch.tensor(upd)).numpy(), rtol=1e-6)
    gidx = i64(3, 1, 3, -1)
    upd = _f(rng, 2, 4, 3)
    (dx,) = run_node("GatherGrad", [i64(2, 5, 3), gidx, upd], domain=MS, axis=1)
    ref = np.zeros((2, 5, 3), np.float32)
    for j, k in enumerate([3, 1, 3, 4]):
        ref[:, k] += upd[:, j]
    np.testing.assert_allclose(dx, ref, rtol=1e-6)
    a_axes, b_axes = run_node("BroadcastGradientArgs", [i64(2, 1, 5), i64(4, 5)], domain=MS, n_outputs=2)
    assert a_axes.tolist() == [1] and b_axes.tolist() == [0]
    (s,) = run_node("ReduceSumTraining", [_f(rng, 2, 4, 5), i64(0, 2)], domain=MS, keepdims=0)
    assert s.shape == (4,)
    mask = rng.random((3, 4)) > 0.25
    (dx,) = run_node("DropoutGrad", [dy.repeat(2, 0)[:3, :3].repeat(2, 1)[:, :4].copy(), mask, np.float32(0.25), np.asarray(True)], domain=MS)
    assert dx.shape == (3, 4) and np.all(dx[~mask] == 0)
    a, bb, g = _f(rng, 3, 4), (rng.random((4,)) + 0.5).astype(np.float32), _f(rng, 3, 4)
    da, db = run_node("DivGrad", [g, a, bb], domain=MS, n_outputs=2)
    at_, bt_ = torch.tensor(a, requires_grad=True), torch.tensor(bb, requires_grad=True)
    (at_ / bt_).backward(torch.tensor(g))
    np.testing.assert_allclose(da, at_.grad.numpy(), rtol=1e-5)
    np.testing.assert_allclose(db, bt_.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_loss_ops_with_ignore_index_and_class_weights():
    rng = np.random.default_rng(8)
    logits, labels = _f(rng, 6, 5, 3), rng.integers(0, 5, (6, 3)).astype(np.int64)
    labels[0, 0] = labels[3, 2] = -100
    weight = (rng.random(5) + 0.5).astype(np.float32)
    lt = torch.tensor(logits, requires_grad=True)
    ref = torch.nn.functional.cross_entropy(lt, torch.tensor(labels), torch.tensor(weight), ignore_index=-100)
    ref.backward()
    loss, logp = run_node("SoftmaxCrossEntropyLossInternal", [logits, labels, weight, np.asarray(-100, dtype=np.int64)], domain=MS,
                          n_outputs=2, reduction="mean")
    assert abs(float(loss) - ref.item()) < 1e-5
    (dl,) = run_node("SoftmaxCrossEntropyLossInternalGrad", [np.float32(1.0), logp, labels, weight, np.asarray(-100, dtype=np.int64)],
                     domain=MS, reduction="mean")
    np.testing.assert_allclose(dl, lt.grad.numpy(), rtol=1e-4, atol=1e-6)
    (dl2,) = run_node("SoftmaxCrossEntropyLossGrad", [np.float32(1.0), logp, labels, weight], domain=MS, reduction="mean", ignore_index=-100)
    np.testing.assert_allclose(dl2, dl, rtol=1e-6)


def test_sgd_clip_and_scaling_ops():
    rng = np.random.default_rng(9)
    w, g = [_f(rng, 3, 2), _f(rng, 4)], [_f(rng, 3, 2), _f(rng, 4)]
    expect = [a - 0.1 * b for a, b in zip(w, g)]
    flag, new_w = run_node("SGDOptimizerV2", [np.float32(0.1), [a.copy() for a in w], g], domain=MS, n_outputs=2)
    assert bool(np.asarray(flag).reshape(-1)[0])
    for a, b in zip(new_w, expect):
        np.testing.assert_allclose(a, b, rtol=1e-6)
    (clipped,) = run_node("InplaceClipGradNorm", [[a.copy() for a in g]], domain=MS, max_norm=0.5)
    total = np.sqrt(sum((a ** 2).sum() for a in clipped))
    assert abs(total - 0.5) < 1e-3
    (norm,) = run_node("ReduceAllL2", g, domain=MS)
    assert abs(float(np.asarray(norm).reshape(-1)[0]) - np.sqrt(sum((a ** 2).sum() for a in g))) < 1e-4
    (scaled,) = run_node("MixedPrecisionScale", [np.float32(4.0), g[0]], domain=MS, to=10)
    assert scaled.dtype == np.float16 and np.allclose(scaled, g[0] * 4, rtol=2e-3, atol=1e-3)
    x = _f(rng, 8)
    out, mask = run_node("FakeQuant", [x, np.float32(0.02), np.float32(128)], domain=MS, n_outputs=2, quant_min=0, quant_max=255)
    q = np.round(x / 0.02 + 128)
    np.testing.assert_allclose(out, (np.clip(q, 0, 255) - 128) * 0.02, rtol=1e-5, atol=1e-6)
    assert mask.tolist() == ((q >= 0) & (q <= 255)).tolist()
    a, b = run_node("View", [x, np.asarray([2, 2], np.int64), np.asarray([4], np.int64)], domain=MS, n_outputs=2)
    assert a.shape == (2, 2) and b.tolist() == x[4:].tolist()


def test_bert_encoder_trains_and_the_two_gradient_paths_agree():
    """A two-layer BERT-shaped encoder from the model exporter: (a) ORTModule (autograd tape), with and without
    recomputation, (b) the gradient graph built from the same model; both against each other, then a few AdamW steps."""
    from onnxruntime_b200.models import bert
    cfg = bert.BertConfig(vocab_size=50, hidden_size=32, num_layers=2, num_heads=2, ffn_size=64, max_position=16)
    model = bert.build_bert(cfg)
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 50, (4, 12), generator=gen)
    mask = torch.ones(4, 12, dtype=torch.int64)
    mask[0, 8:] = 0
    mod, mod_rc = training.ORTModule(model), training.ORTModule(model, recompute=True)
    assert all(p.numel() > 1 for p in mod.parameters())          # one-element constants are not parameters
    target = torch.randn(4, 12, 32, generator=gen)
    for m in (mod, mod_rc):
        ((m(ids, mask) - target) ** 2).mean().backward()
    tape = {n: p.grad for n, p in mod.named_onnx_parameters()}
    for n, p in mod_rc.named_onnx_parameters():
        np.testing.assert_allclose(p.grad.numpy(), tape[n].numpy(), rtol=1e-5, atol=1e-7, err_msg=n)
    assert all(torch.isfinite(g).all() and g.abs().sum() > 0 for g in tape.values())
    # (b) gradient graph: append the same loss, differentiate with respect to a handful of parameters
    m = ol.load_model(model)
    out = m.graph.outputs[0].name
    m.graph.inputs.append(ol.make_tensor_value_info("target", T.FLOAT, [4, 12, 32]))
    m.graph.nodes += [ol.make_node("Sub", [out, "target"], ["t_diff"]), ol.make_node("Mul", ["t_diff", "t_diff"], ["t_sq"]),
                      ol.make_node("ReduceMean", ["t_sq"], ["loss"], keepdims=0)]
    m.graph.outputs[:] = [ol.make_tensor_value_info("loss", T.FLOAT, [])]
    picked = [n for n in tape if tape[n].dim() == 2][:4] + [n for n in tape if tape[n].dim() == 1][:4]
    gm = training.build_gradient_graph(m, picked, "loss")
    sess = ort.InferenceSession(gm.serialize(), providers=["CPUExecutionProvider"])
    got = dict(zip([o.name for o in sess.get_outputs()], sess.run(None, {"input_ids": ids.numpy(), "attention_mask": mask.numpy(), "target": target.numpy()})))
    for n in picked:
        np.testing.assert_allclose(got[n + "_grad"], tape[n].numpy(), rtol=2e-3, atol=2e-6, err_msg=n)
    opt = torch.optim.AdamW(mod.parameters(), lr=1e-2)
    losses = []
    for _ in range(15):
        opt.zero_grad()
        loss = ((mod(ids, mask) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.3 * losses[0]


def _llama_torch(cfg, w, ids):
    """Plain PyTorch restatement of the exported decoder (prompt pass, no past): RMSNorm, packed QKV, half-split rotary
    embedding, causal grouped-query attention, SwiGLU, tied to the exporter's weight names."""
    N, Nk, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    B, S = ids.shape

    def rms(x, g):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.rms_eps) * g

    def rope(x):                                  # [B, heads, S, H]
        cos, sin = w["cos_cache"][:S], w["sin_cache"][:S]
        a, b = x[..., : H // 2], x[..., H // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    h = w["model.embed_tokens.weight"][ids]
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        qkv = rms(h, w[p + "input_layernorm.weight"]) @ w[p + "attn.qkv_proj.weight"]
        q, k, v = qkv.split([N * H, Nk * H, Nk * H], -1)
        q = rope(q.reshape(B, S, N, H).transpose(1, 2))
        k = rope(k.reshape(B, S, Nk, H).transpose(1, 2)).repeat_interleave(N // Nk, 1)
        v = v.reshape(B, S, Nk, H).transpose(1, 2).repeat_interleave(N // Nk, 1)
        att = (q @ k.transpose(-1, -2)) / H ** 0.5 + torch.full((S, S), float("-inf")).triu(1)
        o = (torch.softmax(att, -1) @ v).transpose(1, 2).reshape(B, S, N * H)
        h = h + o @ w[p + "attn.o_proj.weight"]
        x = rms(h, w[p + "post_attention_layernorm.weight"])
        h = h + (torch.nn.functional.silu(x @ w[p + "mlp.gate_proj.weight"]) * (x @ w[p + "mlp.up_proj.weight"])) @ w[p + "mlp.down_proj.weight"]
    return rms(h, w["model.norm.weight"]) @ w["lm_head.weight"]


def test_llama_decoder_fine_tunes_through_the_fused_operators():
    """The Llama export (GroupQueryAttention with rotary embedding, SkipSimplifiedLayerNormalization, SwiGLU) as an
    ORTModule: gradients equal those of a plain PyTorch restatement; next-token loss falls under AdamW."""
    from onnxruntime_b200.models import llama
    cfg = llama.LlamaConfig.tiny(vocab_size=64, hidden_size=32, num_heads=4, num_kv_heads=2, head_dim=8, ffn_size=64,
                                 max_seq_len=32, dtype="fp32")
    model, _ = llama.build_llama(cfg, with_argmax=False, last_token_logits=False, weight_std=0.1)
    m = ol.load_model(model)
    mod = training.ORTModule(m, output_names=["logits"], trainable=[t.name for t in m.graph.initializers if "cache" not in t.name])
    B, S = 3, 10
    ids = torch.randint(0, 64, (B, S), generator=torch.Generator().manual_seed(0))
    feeds = dict(input_ids=ids, seqlens_k=torch.full((B,), S - 1, dtype=torch.int32), total_sequence_length=torch.tensor(S, dtype=torch.int32))
    for i in range(cfg.num_layers):
        feeds[f"past_key_values.{i}.key"] = torch.zeros(B, 2, 0, 8)
        feeds[f"past_key_values.{i}.value"] = torch.zeros(B, 2, 0, 8)

    def loss_of(logits):
        return torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 64), ids[:, 1:].reshape(-1))
    loss = loss_of(mod(**feeds))
    loss.backward()
    w = {t.name: torch.tensor(np.array(ol.to_array(t)), requires_grad=t.data_type == T.FLOAT) for t in m.graph.initializers}
    ref = loss_of(_llama_torch(cfg, w, ids))
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    for name, p in mod.named_onnx_parameters():
        np.testing.assert_allclose(p.grad.numpy(), w[name].grad.numpy(), rtol=2e-3, atol=2e-6, err_msg=name)
    opt = torch.optim.AdamW(mod.parameters(), lr=3e-3)
    for _ in range(25):
        opt.zero_grad()
        cur = loss_of(mod(**feeds))
        cur.backward()
        opt.step()
    assert cur.item() < 0.25 * loss.item()


@pytest.mark.parametrize("loss_type", ["MSELoss", "L1Loss", "BCEWithLogitsLoss"])
def test_artifact_losses_and_the_sgd_optimizer(loss_type):
    rng = np.random.default_rng(10)
    w, b = _f(rng, 6, 3) * 0.5, _f(rng, 3) * 0.1
    g = ol.make_graph([ol.make_node("Gemm", ["x", "w", "b"], ["y"])], "lin", [ol.make_tensor_value_info("x", T.FLOAT, ["n", 6])],
                      [ol.make_tensor_value_info("y", T.FLOAT, ["n", 3])], [ol.make_tensor("w", w), ol.make_tensor("b", b)])
    art = training.generate_artifacts(ol.make_model(g, opset=17), loss=training.LossType[loss_type], optimizer=training.OptimType.SGD)
    state = api.CheckpointState.load_checkpoint(art["checkpoint"])
    module = api.Module(art["training_model.onnx"], state, art["eval_model.onnx"])
    optim = api.Optimizer(art["optimizer_model.onnx"], module)
    optim.set_learning_rate(0.1)
    x = _f(rng, 16, 6)
    target = (rng.random((16, 3)) > 0.5).astype(np.float32) if loss_type == "BCEWithLogitsLoss" else _f(rng, 16, 3)
    wt, bt = torch.tensor(w, requires_grad=True), torch.tensor(b, requires_grad=True)
    fn = {"MSELoss": torch.nn.functional.mse_loss, "L1Loss": torch.nn.functional.l1_loss,
          "BCEWithLogitsLoss": torch.nn.functional.binary_cross_entropy_with_logits}[loss_type]
    for _ in range(4):
        loss, _y = module(x, target)
        ref = fn(torch.tensor(x) @ wt + bt, torch.tensor(target))
        assert abs(float(np.asarray(loss).reshape(-1)[0]) - ref.item()) < 1e-5
        optim.step()
        module.lazy_reset_grad()
        ref.backward()
        with torch.no_grad():
            wt -= 0.1 * wt.grad
            bt -= 0.1 * bt.grad
        wt.grad = bt.grad = None
    np.testing.assert_allclose(state.parameters["w"].data.numpy(), wt.detach().numpy(), rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(state.parameters["b"].data.numpy(), bt.detach().numpy(), rtol=1e-4, atol=1e-6)
