"""Gradient graph builder: appends to a forward ONNX graph the nodes that compute d(loss)/d(parameter).

What the reference does in ``orttraining/orttraining/core/framework/gradient_graph_builder.cc`` with the per-operator
builders of ``orttraining/orttraining/core/graph/gradient_builder.cc``: walk the nodes that lie between the parameters
and the loss in reverse topological order, emit each node's backward nodes (operators of the ``com.microsoft`` training
set: ``ReluGrad``, ``SoftmaxGrad_13``, ``LayerNormalizationGrad``, ``SoftmaxCrossEntropyLossGrad``, ``ConvGrad`` ...),
and sum the contributions where a value feeds several consumers.  Broadcasting is undone by one node,
``com.ortb200.SumToShape(grad, like)``, in place of the reference's ``BroadcastGradientArgs`` + ``ReduceSum`` pair.
"""
from __future__ import annotations

import copy
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set

import numpy as np

from .. import onnx_lite as ol

MS = "com.microsoft"
OWN = "com.ortb200"


class _Builder:
    def __init__(self, graph: ol.Graph, opset: int):
        self.g = graph
        self.opset = opset
        self.new_nodes: List[ol.Node] = []
        self.new_inits: List[ol.Tensor] = []
        self.grads: Dict[str, List[str]] = {}
        self._n = 0
        self.consts = {t.name: t for t in graph.initializers}

    def name(self, hint: str) -> str:
        self._n += 1
        return f"{hint}_grad{self._n}"

    def emit(self, op: str, inputs: Sequence[str], n_out: int = 1, domain: str = "", hint: str = "", **attrs) -> List[str]:
        outs = [self.name(hint or op.lower()) for _ in range(n_out)]
        ready = {k: v for k, v in attrs.items() if isinstance(v, ol.Attribute)}        # copied from a forward node
        node = ol.make_node(op, list(inputs), outs, name=self.name(op), domain=domain,
                            **{k: v for k, v in attrs.items() if k not in ready})
        node.attributes.extend(copy.deepcopy(a) for a in ready.values())
        self.new_nodes.append(node)
        return outs

    def one(self, op: str, inputs: Sequence[str], domain: str = "", **attrs) -> str:
        return self.emit(op, inputs, 1, domain, **attrs)[0]

    def const(self, array, hint: str = "c") -> str:
        name = self.name(hint)
        self.new_inits.append(ol.make_tensor(name, np.asarray(array)))
        return name

    def add_grad(self, value: str, grad: str) -> None:
        self.grads.setdefault(value, []).append(grad)

    def grad_of(self, value: str) -> Optional[str]:
        parts = self.grads.get(value)
        if not parts:
            return None
        if len(parts) > 1:
            self.grads[value] = [self.one("Sum", parts)]
        return self.grads[value][0]

    def sum_to(self, grad: str, like: str) -> str:
        return self.one("SumToShape", [grad, like], OWN)

    def shape_of(self, value: str) -> str:
        return self.one("Shape", [value])


def _attr(node: ol.Node, name: str, default=None):
    return ol.attr_value(node, name, default)


def _copy_attrs(node: ol.Node, names: Iterable[str]) -> dict:
    return {a.name: a for a in node.attributes if a.name in names}


# ---- per-operator rules: rule(builder, node, output grads (None where absent), needs (per input)) --------------------
Rule = Callable[[_Builder, ol.Node, List[Optional[str]], List[bool]], None]
_RULES: Dict[str, Rule] = {}


def _rule(*ops: str):
    def deco(fn: Rule) -> Rule:
        for op in ops:
            _RULES[op] = fn
        return fn
    return deco


@_rule("Add", "Sub")
def _add(b, n, dy, needs):
    if needs[0]:
        b.add_grad(n.inputs[0], b.sum_to(dy[0], n.inputs[0]))
    if needs[1]:
        g = dy[0] if n.op_type == "Add" else b.one("Neg", [dy[0]])
        b.add_grad(n.inputs[1], b.sum_to(g, n.inputs[1]))


@_rule("Sum")
def _sum(b, n, dy, needs):
    for i, name in enumerate(n.inputs):
        if needs[i]:
            b.add_grad(name, b.sum_to(dy[0], name))


@_rule("Mul")
def _mul(b, n, dy, needs):
    for i in (0, 1):
        if needs[i]:
            b.add_grad(n.inputs[i], b.sum_to(b.one("Mul", [dy[0], n.inputs[1 - i]]), n.inputs[i]))


@_rule("Div")
def _div(b, n, dy, needs):
    da, db = b.emit("DivGrad", [dy[0], n.inputs[0], n.inputs[1]], 2, MS)
    if needs[0]:
        b.add_grad(n.inputs[0], da)
    if needs[1]:
        b.add_grad(n.inputs[1], db)


@_rule("Neg")
def _neg(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("Neg", [dy[0]]))


@_rule("Exp")
def _exp(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("Mul", [dy[0], n.outputs[0]]))


@_rule("Log")
def _log(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("Div", [dy[0], n.inputs[0]]))


@_rule("Sqrt")
def _sqrt(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("Div", [dy[0], b.one("Mul", [n.outputs[0], b.const(np.float32(2.0))])]))


@_rule("Pow")
def _pow(b, n, dy, needs):   # the exponent is treated as a constant
    if needs[0]:
        p = n.inputs[1]
        pm1 = b.one("Sub", [p, b.const(np.float32(1.0))])
        g = b.one("Mul", [dy[0], b.one("Mul", [p, b.one("Pow", [n.inputs[0], pm1])])])
        b.add_grad(n.inputs[0], b.sum_to(g, n.inputs[0]))


@_rule("MatMul")
def _matmul(b, n, dy, needs):
    a, w = n.inputs
    if needs[0]:
        b.add_grad(a, b.sum_to(b.one("FusedMatMul", [dy[0], w], MS, transB=1), a))
    if needs[1]:
        b.add_grad(w, b.sum_to(b.one("FusedMatMul", [a, dy[0]], MS, transA=1), w))


@_rule("Gemm")
def _gemm(b, n, dy, needs):
    ta, tb = int(_attr(n, "transA", 0)), int(_attr(n, "transB", 0))
    alpha, beta = float(_attr(n, "alpha", 1.0)), float(_attr(n, "beta", 1.0))
    a, w = n.inputs[0], n.inputs[1]
    if needs[0]:
        g = (b.one("Gemm", [dy[0], w], transA=0, transB=1 - tb, alpha=alpha) if not ta
             else b.one("Gemm", [w, dy[0]], transA=tb, transB=1, alpha=alpha))
        b.add_grad(a, g)
    if needs[1]:
        g = (b.one("Gemm", [a, dy[0]], transA=1 - ta, transB=0, alpha=alpha) if not tb
             else b.one("Gemm", [dy[0], a], transA=1, transB=ta, alpha=alpha))
        b.add_grad(w, g)
    if len(n.inputs) > 2 and n.inputs[2] and needs[2]:
        g = dy[0] if beta == 1.0 else b.one("Mul", [dy[0], b.const(np.float32(beta))])
        b.add_grad(n.inputs[2], b.sum_to(g, n.inputs[2]))


@_rule("Relu")
def _relu(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("ReluGrad", [dy[0], n.outputs[0]], MS))


@_rule("Sigmoid")
def _sigmoid(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("SigmoidGrad", [dy[0], n.outputs[0]], MS))


@_rule("Tanh")
def _tanh(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("TanhGrad", [dy[0], n.outputs[0]], MS))


@_rule("LeakyRelu")
def _leaky(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("LeakyReluGrad", [dy[0], n.outputs[0]], MS, alpha=float(_attr(n, "alpha", 0.01))))


@_rule("Gelu")
def _gelu(b, n, dy, needs):
    approx = _attr(n, "approximate", "none")
    approx = approx.decode() if isinstance(approx, bytes) else approx
    b.add_grad(n.inputs[0], b.one("FastGeluGrad" if approx == "tanh" else "GeluGrad", [dy[0], n.inputs[0]], MS))


@_rule("QuickGelu")
def _quick_gelu(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("QuickGeluGrad", [dy[0], n.inputs[0]], MS, alpha=float(_attr(n, "alpha", 1.702))))


@_rule("FastGelu", "BiasGelu")
def _bias_gelu(b, n, dy, needs):
    fast = n.op_type == "FastGelu"
    if len(n.inputs) > 1 and n.inputs[1]:
        g = b.one("BiasFastGeluGrad_dX" if fast else "BiasGeluGrad_dX", [dy[0], n.inputs[0], n.inputs[1]], MS)
        if needs[1]:
            b.add_grad(n.inputs[1], b.sum_to(g, n.inputs[1]))
    else:
        g = b.one("FastGeluGrad" if fast else "GeluGrad", [dy[0], n.inputs[0]], MS)
    if needs[0]:
        b.add_grad(n.inputs[0], g)


@_rule("Softmax", "LogSoftmax")
def _softmax(b, n, dy, needs):
    op = n.op_type + "Grad" + ("_13" if b.opset >= 13 else "")
    b.add_grad(n.inputs[0], b.one(op, [dy[0], n.outputs[0]], MS, axis=int(_attr(n, "axis", -1 if b.opset >= 13 else 1))))


@_rule("LayerNormalization", "SimplifiedLayerNormalization")
def _layer_norm(b, n, dy, needs):
    simplified = n.op_type.startswith("Simplified")
    want = 2 if simplified else 3
    while len(n.outputs) < want:                       # the backward half reads the saved statistics
        n.outputs.append("")
    for i in range(1, want):
        if not n.outputs[i]:
            n.outputs[i] = b.name("saved_stat")
    axis = int(_attr(n, "axis", -1))
    if simplified:
        dx, ds = b.emit("SimplifiedLayerNormalizationGrad", [dy[0], n.inputs[0], n.inputs[1], n.outputs[1]], 2, MS, axis=axis)
        db = None
    else:
        dx, ds, db = b.emit("LayerNormalizationGrad", [dy[0], n.inputs[0], n.inputs[1], n.outputs[1], n.outputs[2]], 3, MS, axis=axis)
    if needs[0]:
        b.add_grad(n.inputs[0], dx)
    if needs[1]:
        b.add_grad(n.inputs[1], ds)
    if db is not None and len(n.inputs) > 2 and n.inputs[2] and needs[2]:
        b.add_grad(n.inputs[2], db)


@_rule("Reshape", "Flatten", "Squeeze", "Unsqueeze")
def _reshape(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.one("Reshape", [dy[0], b.shape_of(n.inputs[0])]))


@_rule("Identity", "Dropout", "Cast")
def _identity(b, n, dy, needs):
    if n.op_type == "Dropout" and len(n.outputs) > 1 and n.outputs[1]:
        ins = [dy[0], n.outputs[1]] + [i for i in n.inputs[1:3]]
        b.add_grad(n.inputs[0], b.one("DropoutGrad", ins, MS))
    elif n.op_type == "Cast":
        b.add_grad(n.inputs[0], b.one("CastLike", [dy[0], n.inputs[0]]))
    else:
        b.add_grad(n.inputs[0], dy[0])


@_rule("Transpose")
def _transpose(b, n, dy, needs):
    perm = _attr(n, "perm", None)
    if perm is None:
        b.add_grad(n.inputs[0], b.one("Transpose", [dy[0]]))
    else:
        inv = [0] * len(perm)
        for i, p in enumerate(perm):
            inv[int(p)] = i
        b.add_grad(n.inputs[0], b.one("Transpose", [dy[0]], perm=inv))


@_rule("Expand")
def _expand(b, n, dy, needs):
    b.add_grad(n.inputs[0], b.sum_to(dy[0], n.inputs[0]))


@_rule("Where")
def _where(b, n, dy, needs):
    zero = b.one("Sub", [dy[0], dy[0]])
    if needs[1]:
        b.add_grad(n.inputs[1], b.sum_to(b.one("Where", [n.inputs[0], dy[0], zero]), n.inputs[1]))
    if needs[2]:
        b.add_grad(n.inputs[2], b.sum_to(b.one("Where", [n.inputs[0], zero, dy[0]]), n.inputs[2]))


@_rule("ReduceSum", "ReduceMean")
def _reduce(b, n, dy, needs):
    x = n.inputs[0]
    attrs = _copy_attrs(n, ("axes", "noop_with_empty_axes"))
    kept = b.one(n.op_type, list(n.inputs), keepdims=1, **attrs)          # only its shape is read
    g = b.one("Expand", [b.one("Reshape", [dy[0], b.shape_of(kept)]), b.shape_of(x)])
    if n.op_type == "ReduceMean":
        count = b.one("Div", [b.one("Size", [x]), b.one("Size", [kept])])
        g = b.one("Div", [g, b.one("CastLike", [count, g])])
    b.add_grad(x, g)


@_rule("Gather")
def _gather(b, n, dy, needs):
    if needs[0]:
        b.add_grad(n.inputs[0], b.one("GatherGrad", [b.shape_of(n.inputs[0]), n.inputs[1], dy[0]], MS, axis=int(_attr(n, "axis", 0))))


@_rule("GatherElements")
def _gather_elements(b, n, dy, needs):
    if needs[0]:
        b.add_grad(n.inputs[0], b.one("GatherElementsGrad", [dy[0], b.shape_of(n.inputs[0]), n.inputs[1]], MS, axis=int(_attr(n, "axis", 0))))


@_rule("GatherND")
def _gather_nd(b, n, dy, needs):
    if needs[0]:
        b.add_grad(n.inputs[0], b.one("GatherNDGrad", [b.shape_of(n.inputs[0]), n.inputs[1], dy[0]], MS, batch_dims=int(_attr(n, "batch_dims", 0))))


@_rule("Slice")
def _slice(b, n, dy, needs):
    if needs[0]:
        b.add_grad(n.inputs[0], b.one("SliceGrad", [dy[0], b.shape_of(n.inputs[0])] + list(n.inputs[1:]), MS))


@_rule("Concat")
def _concat(b, n, dy, needs):
    axis = int(_attr(n, "axis", 0))
    ax = b.const(np.asarray([axis], dtype=np.int64))
    lens = [b.one("Gather", [b.shape_of(i), ax]) for i in n.inputs]
    parts = b.emit("Split", [dy[0], b.one("Concat", lens, axis=0)], len(n.inputs), axis=axis)
    for i, name in enumerate(n.inputs):
        if needs[i]:
            b.add_grad(name, parts[i])


@_rule("Split")
def _split(b, n, dy, needs):
    axis = int(_attr(n, "axis", 0))
    parts = [d if d is not None else b.one("Sub", [o, o]) for d, o in zip(dy, n.outputs)]
    b.add_grad(n.inputs[0], b.one("Concat", parts, axis=axis))


@_rule("Conv")
def _conv(b, n, dy, needs):
    has_bias = len(n.inputs) > 2 and bool(n.inputs[2])
    outs = b.emit("ConvGrad", [dy[0], n.inputs[0], n.inputs[1]], 3 if has_bias else 2, MS,
                  **_copy_attrs(n, ("strides", "pads", "dilations", "group", "auto_pad", "kernel_shape")))
    for i in range(len(outs)):
        if needs[i]:
            b.add_grad(n.inputs[i], outs[i])


@_rule("SoftmaxCrossEntropyLoss")
def _sce(b, n, dy, needs):
    while len(n.outputs) < 2:
        n.outputs.append("")
    if not n.outputs[1]:
        n.outputs[1] = b.name("log_prob")
    ins = [dy[0], n.outputs[1], n.inputs[1]] + ([n.inputs[2]] if len(n.inputs) > 2 and n.inputs[2] else [])
    b.add_grad(n.inputs[0], b.one("SoftmaxCrossEntropyLossGrad", ins, MS, **_copy_attrs(n, ("reduction", "ignore_index"))))


# ---- fallback: differentiate the node itself -------------------------------------------------------------------
_NODE_SESSIONS: Dict[bytes, object] = {}


def _node_grad(*values, node: bytes = b"", n_inputs: int = 0, wrt=(), **_unused):
    """Kernel of ``com.ortb200.NodeGrad``: re-runs one forward node (held as a serialized single-node model in the
    ``node`` attribute) on the differentiable tensor-library kernels with autograd recording, and returns the gradients
    of its inputs ``wrt`` for the output gradients that follow the forward inputs in ``values``."""
    import torch

    from .. import capi
    key = bytes(node)
    sess = _NODE_SESSIONS.get(key)
    if sess is None:
        so = capi.SessionOptions()
        so.graph_optimization_level = capi.GraphOptimizationLevel.ORT_DISABLE_ALL
        so.add_session_config_entry("ortb200.generic_kernels_only", "1")
        on_gpu = any(isinstance(v, torch.Tensor) and v.is_cuda for v in values)
        sess = capi.InferenceSession(key, so, providers=(["CUDAExecutionProvider"] if on_gpu else []) + ["CPUExecutionProvider"])
        _NODE_SESSIONS[key] = sess
    n_inputs = int(n_inputs)
    fwd, dys = list(values[:n_inputs]), list(values[n_inputs:])
    names = [i.name for i in sess.get_inputs()]
    out_names = [o.name for o in sess.get_outputs()]
    wrt = [int(i) for i in wrt]
    with torch.enable_grad():
        leaves = {}
        feeds = []
        present = [v for v in fwd if v is not None]
        for slot, v in enumerate(fwd):
            if v is None:
                continue
            if slot in wrt and v.is_floating_point():
                v = v.detach().requires_grad_(True)
                leaves[slot] = v
            feeds.append(v)
        assert len(feeds) == len(names) == len(present)
        outs = sess._sess.run(capi.C.RunOptions(), names, feeds, out_names)
        pairs = [(o, d) for o, d in zip(outs, dys) if d is not None and isinstance(o, torch.Tensor) and o.requires_grad]
        if not pairs:
            raise RuntimeError("NodeGrad: the node's outputs do not depend differentiably on the requested inputs")
        order = [s for s in wrt if s in leaves]
        grads = torch.autograd.grad([o for o, _ in pairs], [leaves[s] for s in order], [d.to(o.dtype) for o, d in pairs], allow_unused=True)
    by_slot = dict(zip(order, grads))
    result = []
    for s in wrt:
        g = by_slot.get(s)
        result.append(g if g is not None else torch.zeros_like(fwd[s]))
    return result[0] if len(result) == 1 else tuple(result)


def _register_node_grad() -> None:
    from .. import capi
    try:
        capi.C.register_python_op(OWN, "NodeGrad", _node_grad)
    except Exception:  # pragma: no cover - a build without Python operators
        pass


_register_node_grad()


def _fallback_rule(b: _Builder, n: ol.Node, dy, needs, model: ol.Model) -> None:
    ins = [i for i in n.inputs]
    single = ol.make_graph([copy.deepcopy(n)], "node", [ol.make_tensor_value_info(i, 0, None) for i in ins if i],
                           [ol.make_tensor_value_info(o, 0, None) for o in n.outputs if o])
    blob = ol.Model(single, dict(model.opset_imports), model.ir_version).serialize()
    wrt = [i for i, need in enumerate(needs) if need]
    dys = [d if d is not None else "" for d, o in zip(dy, n.outputs) if o]
    outs = b.emit("NodeGrad", ins + dys, len(wrt), OWN, node=blob, n_inputs=len(ins), wrt=wrt)
    for slot, g in zip(wrt, outs):
        b.add_grad(n.inputs[slot], g)


def supported_ops() -> List[str]:
    """Operators a gradient can be taken through."""
    return sorted(_RULES)


def build_gradient_graph(model: ol.Model, requires_grad: Sequence[str], loss: str,
                         input_grads: Sequence[str] = (), recompute_fallback: bool = True) -> ol.Model:
    """Returns a copy of ``model`` whose graph also computes, for every name in ``requires_grad`` (initializers or graph
    inputs) and ``input_grads``, the output ``<name>_grad`` = d ``loss`` / d name.  The loss may have any shape; its own
    gradient is a tensor of ones.  An operator without a rule of its own gets a ``com.ortb200.NodeGrad`` node, which re-runs
    that one node with autograd recording and differentiates it (so every operator whose tensor-library kernel is
    differentiable is covered, at the price of computing it twice); with ``recompute_fallback=False`` such an operator
    raises ``NotImplementedError`` naming it instead."""
    model = copy.deepcopy(model)
    g = model.graph
    opset = int(model.opset_imports.get("", 17))
    b = _Builder(g, opset)
    wanted = list(requires_grad) + [n for n in input_grads if n not in requires_grad]
    # forward reachability from the differentiated values, backward reachability from the loss
    reach: Set[str] = set(wanted)
    for n in g.nodes:
        if any(i in reach for i in n.inputs):
            reach.update(o for o in n.outputs if o)
    if loss not in reach:
        raise ValueError(f"the loss '{loss}' does not depend on any of {wanted}")
    feeds_loss: Set[str] = {loss}
    for n in reversed(g.nodes):
        if any(o in feeds_loss for o in n.outputs):
            feeds_loss.update(i for i in n.inputs if i)
    one = np.ones((), dtype=np.float32)
    b.add_grad(loss, b.one("ConstantOfShape", [b.shape_of(loss)], value=ol.make_tensor("one", one.reshape(1))))
    for n in reversed(g.nodes):
        if not any(o in feeds_loss and o in reach for o in n.outputs):
            continue
        dy = [b.grad_of(o) if o else None for o in n.outputs]
        if all(d is None for d in dy):
            continue
        needs = [bool(i) and i in reach for i in n.inputs]
        if not any(needs):
            continue
        rule = _RULES.get(n.op_type)
        if rule is None:
            if not recompute_fallback:
                raise NotImplementedError(f"no gradient rule for operator '{n.op_type}' (node '{n.name}')")
            _fallback_rule(b, n, dy, needs, model)
            continue
        if dy[0] is None and n.op_type not in ("Split",):
            continue
        rule(b, n, dy, needs)
    known = {v.name: v for v in g.inputs}
    inits = {t.name: t for t in g.initializers}
    for name in wanted:
        grad = b.grad_of(name)
        if grad is None:
            raise ValueError(f"'{name}' does not influence the loss")
        out = name + "_grad"
        b.new_nodes.append(ol.make_node("Identity", [grad], [out], name=b.name("GradOut")))
        if name in inits:
            t = inits[name]
            g.outputs.append(ol.make_tensor_value_info(out, t.data_type, list(t.dims)))
        else:
            v = known.get(name)
            g.outputs.append(ol.make_tensor_value_info(out, v.elem_type if v else ol.TensorProto.FLOAT, v.shape if v else None))
    g.nodes.extend(b.new_nodes)
    g.initializers.extend(b.new_inits)
    model.opset_imports.setdefault(MS, 1)
    model.opset_imports.setdefault(OWN, 1)
    return model
