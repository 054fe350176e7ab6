"""Shared test helpers: a one-node-model harness in the spirit of the reference's OpTester
(onnxruntime/test/unittest_util/op_tester.h): declare an op with attributes, feed inputs, compare the
session's outputs with expected values computed independently (numpy / torch fp32)."""
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

import onnxruntime_b200 as ort
from onnxruntime_b200 import onnx_lite as ol

T = ol.TensorProto


def run_node(op_type: str, inputs: Dict[str, Optional[np.ndarray]], n_outputs: int = 1, domain: str = "", opset: int = 17,
             initializers: Sequence[str] = (), providers=("CPUExecutionProvider",), optimize: bool = False,
             **attrs) -> List[np.ndarray]:
    """Build a single-node model and run it.  Inputs named in `initializers` become constant initializers;
    a None value marks an omitted optional input."""
    names = list(inputs.keys())
    node_inputs = [n if inputs[n] is not None else "" for n in names]
    out_names = [f"out{i}" for i in range(n_outputs)]
    node = ol.make_node(op_type, node_inputs, out_names, domain=domain, **attrs)
    graph_inputs, inits = [], []
    for n in names:
        v = inputs[n]
        if v is None:
            continue
        if n in initializers:
            inits.append(ol.make_tensor(n, v))
        elif isinstance(v, (dict, list)):     # a map- or sequence-typed input: no tensor type to declare
            graph_inputs.append(ol.make_tensor_value_info(n, 0, None))
        else:
            graph_inputs.append(ol.make_tensor_value_info(n, ol.np_dtype_to_onnx(v.dtype), list(v.shape)))
    graph = ol.make_graph([node], "test", graph_inputs, [ol.make_tensor_value_info(o, 0, None) for o in out_names], inits)
    model = ol.make_model(graph, opset=opset).serialize()
    so = ort.SessionOptions()
    if not optimize:
        so.graph_optimization_level = ort.GraphOptimizationLevel.ORT_DISABLE_ALL
    sess = ort.InferenceSession(model, so, providers=list(providers))
    feeds = {n: inputs[n] for n in names if inputs[n] is not None and n not in initializers}
    return sess.run(None, feeds)


def graph_model(nodes, inputs, outputs, inits=(), opset: int = 17) -> bytes:
    return ol.make_model(ol.make_graph(list(nodes), "g", list(inputs), list(outputs), list(inits)), opset=opset).serialize()


def op_counts(sess) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for n in sess.graph_nodes():
        out[n["op_type"]] = out.get(n["op_type"], 0) + 1
    return out
