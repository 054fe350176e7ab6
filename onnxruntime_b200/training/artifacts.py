"""Training artifacts from a forward model: training model, eval model, optimizer model, checkpoint.

Layout as produced by the reference's ``onnxruntime.training.artifacts.generate_artifacts``
(``orttraining/orttraining/python/training/artifacts.py``, ``onnxblock/``):

* eval model: the forward graph plus the loss; parameters are graph inputs.
* training model: the eval model plus the gradient graph; each trainable parameter ``p`` has a gradient accumulation
  buffer input ``p_grad.accumulation.buffer`` and a boolean output ``p_grad.accumulation.out`` (``InPlaceAccumulatorV2``
  adds into the buffer in place, or overwrites it when the ``lazy_reset_grad`` input is true).
* optimizer model: ``AdamWOptimizer`` / ``SGDOptimizerV2`` over sequences of parameters, gradients and moments.
* checkpoint: parameter values, which of them are trainable, and (later) the optimizer state.
"""
from __future__ import annotations

import copy
import os
from enum import Enum
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

from .. import onnx_lite as ol
from .gradient_builder import MS, build_gradient_graph
from .ortmodule import lift_initializers

T = ol.TensorProto


class LossType(Enum):
    MSELoss = 1
    CrossEntropyLoss = 2
    BCEWithLogitsLoss = 3
    L1Loss = 4


class OptimType(Enum):
    AdamW = 1
    SGD = 2


def _append_loss(model: ol.Model, loss: LossType, output: str, target: str, reduction: str = "mean") -> str:
    g = model.graph
    out_info = next((o for o in g.outputs if o.name == output), None)
    elem = out_info.elem_type if out_info is not None and out_info.elem_type else T.FLOAT
    shape = out_info.shape if out_info is not None else None
    name = "loss"
    if loss == LossType.CrossEntropyLoss:
        label_shape = ([shape[0]] + list(shape[2:])) if shape else None
        g.inputs.append(ol.make_tensor_value_info(target, T.INT64, label_shape))
        g.nodes.append(ol.make_node("SoftmaxCrossEntropyLoss", [output, target], [name, name + "_log_prob"], name="loss_fn",
                                    reduction=reduction))
    else:
        g.inputs.append(ol.make_tensor_value_info(target, elem, shape))
        reduce = "ReduceMean" if reduction == "mean" else "ReduceSum"
        if loss == LossType.MSELoss:
            g.nodes.append(ol.make_node("Sub", [output, target], ["loss_diff"]))
            g.nodes.append(ol.make_node("Mul", ["loss_diff", "loss_diff"], ["loss_elem"]))
        elif loss == LossType.L1Loss:
            # |d| as sqrt(d^2 + eps): differentiable at 0 with the rules of the builder
            g.initializers.append(ol.make_tensor("loss_eps", np.asarray(1e-12, dtype=np.float32)))
            g.nodes.append(ol.make_node("Sub", [output, target], ["loss_diff"]))
            g.nodes.append(ol.make_node("Mul", ["loss_diff", "loss_diff"], ["loss_sq"]))
            g.nodes.append(ol.make_node("Add", ["loss_sq", "loss_eps"], ["loss_sq_eps"]))
            g.nodes.append(ol.make_node("Sqrt", ["loss_sq_eps"], ["loss_elem"]))
        else:  # BCE with logits: max(x, 0) - x t + log(1 + exp(-|x|)) = relu(x) - x t - log(sigmoid(|x|))
            g.nodes.append(ol.make_node("Relu", [output], ["loss_relu"]))
            g.nodes.append(ol.make_node("Mul", [output, target], ["loss_xt"]))
            g.nodes.append(ol.make_node("Neg", [output], ["loss_negx"]))
            g.nodes.append(ol.make_node("Relu", ["loss_negx"], ["loss_relu_neg"]))
            g.nodes.append(ol.make_node("Add", ["loss_relu", "loss_relu_neg"], ["loss_abs"]))        # |x|
            g.nodes.append(ol.make_node("Sigmoid", ["loss_abs"], ["loss_sig"]))
            g.nodes.append(ol.make_node("Log", ["loss_sig"], ["loss_logsig"]))
            g.nodes.append(ol.make_node("Sub", ["loss_relu", "loss_xt"], ["loss_a"]))
            g.nodes.append(ol.make_node("Sub", ["loss_a", "loss_logsig"], ["loss_elem"]))
        g.nodes.append(ol.make_node(reduce, ["loss_elem"], [name], keepdims=0))
    g.outputs.insert(0, ol.make_tensor_value_info(name, elem, []))
    return name


def _optimizer_model(kind: OptimType, n_params: int, **attrs) -> ol.Model:
    seq = lambda name: ol.ValueInfo(name, 0, None)   # noqa: E731  (sequence-typed: element type left open)
    ins = [ol.make_tensor_value_info("learning_rate", T.FLOAT, [1])]
    if kind == OptimType.AdamW:
        ins.append(ol.make_tensor_value_info("step", T.INT64, [1]))
        ins += [seq("params"), seq("gradients"), seq("first_order_moments"), seq("second_order_moments")]
        node = ol.make_node("AdamWOptimizer", [v.name for v in ins], ["updated_flag", "updated_params", "updated_m1", "updated_m2"],
                            name="optimizer", domain=MS, alpha=float(attrs.get("betas", (0.9, 0.999))[0]),
                            beta=float(attrs.get("betas", (0.9, 0.999))[1]), epsilon=float(attrs.get("eps", 1e-8)),
                            weight_decay=float(attrs.get("weight_decay", 0.01)), correct_bias=1, adam_mode=0)
    else:
        ins += [seq("params"), seq("gradients")]
        node = ol.make_node("SGDOptimizerV2", [v.name for v in ins], ["updated_flag", "updated_params"], name="optimizer", domain=MS)
    g = ol.make_graph([node], "optimizer", ins, [ol.make_tensor_value_info("updated_flag", T.BOOL, [1])])
    return ol.make_model(g, opset=17, metadata={"optimizer": kind.name, "param_count": str(n_params)})


def generate_artifacts(model: Union[str, bytes, ol.Model], requires_grad: Optional[Sequence[str]] = None,
                       frozen_params: Optional[Sequence[str]] = None, loss: Optional[LossType] = None,
                       optimizer: Optional[OptimType] = None, artifact_directory: Optional[str] = None, prefix: str = "",
                       loss_input: Optional[str] = None, target_name: str = "target", reduction: str = "mean",
                       optimizer_options: Optional[Dict[str, object]] = None) -> Dict[str, bytes]:
    """Builds the artifacts, writes them to ``artifact_directory`` when given (``training_model.onnx``,
    ``eval_model.onnx``, ``optimizer_model.onnx``, ``checkpoint``) and returns them as bytes by those names.
    ``loss`` is attached to the graph output ``loss_input`` (the first output by default); with ``loss=None`` the first
    output is taken to be the loss already."""
    from .api import CheckpointState
    base = copy.deepcopy(model) if isinstance(model, ol.Model) else ol.load_model(model)
    g = base.graph
    floats = (T.FLOAT, T.FLOAT16, T.BFLOAT16, T.DOUBLE)
    frozen = set(frozen_params or [])
    if requires_grad is None:
        requires_grad = [t.name for t in g.initializers if t.data_type in floats and t.name not in frozen and int(np.prod(t.dims)) > 1]
    requires_grad = [n for n in requires_grad if n not in frozen]
    known = {t.name for t in g.initializers}
    for n in list(requires_grad) + list(frozen):
        if n not in known:
            raise ValueError(f"'{n}' is not an initializer of the model")
    loss_name = g.outputs[0].name
    if loss is not None:
        loss_name = _append_loss(base, loss, loss_input or g.outputs[0].name, target_name, reduction)
    params = list(requires_grad) + [n for n in frozen]
    values = {t.name: np.array(ol.to_array(t)) for t in g.initializers if t.name in params}
    eval_model = lift_initializers(copy.deepcopy(base), params)
    train = build_gradient_graph(eval_model, requires_grad, loss_name)
    tg = train.graph
    tg.inputs.append(ol.make_tensor_value_info("lazy_reset_grad", T.BOOL, [1]))
    grad_outputs = {p + "_grad" for p in requires_grad}
    tg.outputs[:] = [o for o in tg.outputs if o.name not in grad_outputs]
    for p in requires_grad:
        buf = p + "_grad.accumulation.buffer"
        info = next(v for v in tg.inputs if v.name == p)
        tg.inputs.append(ol.make_tensor_value_info(buf, info.elem_type, info.shape))
        tg.nodes.append(ol.make_node("InPlaceAccumulatorV2", [buf, p + "_grad", "lazy_reset_grad"], [p + "_grad.accumulation.out"],
                                     name="acc_" + p, domain=MS))
        tg.outputs.append(ol.make_tensor_value_info(p + "_grad.accumulation.out", T.BOOL, [1]))
    out: Dict[str, bytes] = {prefix + "training_model.onnx": train.serialize(), prefix + "eval_model.onnx": eval_model.serialize()}
    if optimizer is not None:
        out[prefix + "optimizer_model.onnx"] = _optimizer_model(optimizer, len(requires_grad), **(optimizer_options or {})).serialize()
    state = CheckpointState.from_parameters(values, set(requires_grad))
    out[prefix + "checkpoint"] = state.to_bytes()
    if artifact_directory:
        os.makedirs(artifact_directory, exist_ok=True)
        for name, blob in out.items():
            with open(os.path.join(artifact_directory, name), "wb") as f:
                f.write(blob)
    return out
