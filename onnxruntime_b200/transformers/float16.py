"""float32 -> float16 model conversion (the counterpart of onnxruntime/python/tools/transformers/float16.py).

Initializers, value infos and ``Cast(to=FLOAT)`` / ``Constant`` / ``ConstantOfShape`` payloads become float16; ops on
the block list keep float32 and get Cast nodes around them; with ``keep_io_types`` the graph inputs / outputs stay
float32 behind Cast nodes.  Values outside the float16 range are clamped to +-max_finite_val, tiny ones to
+-min_positive_val (as in the reference's ``convert_np_to_float16``)."""
from __future__ import annotations

from typing import Iterable, Optional, Union

import numpy as np

from .. import onnx_lite as ol

T = ol.TensorProto
DEFAULT_OP_BLOCK_LIST = ["ArrayFeatureExtractor", "Binarizer", "CastMap", "CategoryMapper", "DictVectorizer", "FeatureVectorizer",
                         "Imputer", "LabelEncoder", "LinearClassifier", "LinearRegressor", "Normalizer", "OneHotEncoder",
                         "RandomUniformLike", "SVMClassifier", "SVMRegressor", "Scaler", "TreeEnsembleClassifier",
                         "TreeEnsembleRegressor", "ZipMap", "NonMaxSuppression", "TopK", "RoiAlign", "Resize", "Range", "CumSum",
                         "Min", "Max", "Upsample"]


def _to_half(arr: np.ndarray, min_positive_val: float, max_finite_val: float) -> np.ndarray:
    a = arr.astype(np.float32).copy()
    small = (a != 0) & (np.abs(a) < min_positive_val)
    a[small] = np.sign(a[small]) * min_positive_val
    a = np.clip(a, -max_finite_val, max_finite_val)
    return a.astype(np.float16)


def convert_float_to_float16(model: Union[str, bytes, ol.Model], min_positive_val: float = 5.96e-08, max_finite_val: float = 65504.0,
                             keep_io_types: bool = False, op_block_list: Optional[Iterable[str]] = None,
                             node_block_list: Iterable[str] = ()) -> ol.Model:
    m = model if isinstance(model, ol.Model) else ol.load_model(model)
    g = m.graph
    block_ops = set(DEFAULT_OP_BLOCK_LIST if op_block_list is None else op_block_list)
    block_nodes = set(node_block_list)

    def blocked(n: ol.Node) -> bool:
        return n.op_type in block_ops or n.name in block_nodes

    # values that must stay float32: everything touching a blocked node
    keep32 = set()
    for n in g.nodes:
        if blocked(n):
            keep32.update(i for i in n.inputs if i)
            keep32.update(n.outputs)

    for t in g.initializers:
        if t.data_type == T.FLOAT and t.external is None and t.name not in keep32:
            half = _to_half(ol.to_array(t), min_positive_val, max_finite_val)
            t.data_type, t.raw = T.FLOAT16, half.tobytes()
    for vi in g.value_info:
        if vi.elem_type == T.FLOAT and vi.name not in keep32:
            vi.elem_type = T.FLOAT16

    new_nodes = []
    counter = [0]

    def cast(src: str, dst: str, to: int) -> ol.Node:
        counter[0] += 1
        return ol.make_node("Cast", [src], [dst], name=f"fp16_cast_{counter[0]}", to=to)

    # element types known from value_info (before conversion everything listed as FLOAT16 was FLOAT)
    value_types = {v.name: (T.FLOAT if v.elem_type == T.FLOAT16 else v.elem_type) for v in g.value_info}
    rename = {}
    # graph inputs
    for vi in g.inputs:
        if vi.elem_type != T.FLOAT or vi.name in keep32:
            continue
        if keep_io_types:
            new_nodes.append(cast(vi.name, vi.name + "_fp16", T.FLOAT16))
            rename[vi.name] = vi.name + "_fp16"
        else:
            vi.elem_type = T.FLOAT16
    out_names = {}
    for vi in g.outputs:
        if vi.elem_type != T.FLOAT or vi.name in keep32:
            continue
        if keep_io_types:
            out_names[vi.name] = vi.name + "_fp16"
        else:
            vi.elem_type = T.FLOAT16

    for n in g.nodes:
        n.inputs = [rename.get(i, i) for i in n.inputs]
        if blocked(n):
            # the node keeps float32: values computed in float16 upstream are cast up on the way in, and its float
            # outputs are cast down for the float16 consumers
            init_names = {t.name for t in g.initializers}
            graph_in = {v.name for v in g.inputs}
            for k, i in enumerate(n.inputs):
                if i and i not in init_names and i not in graph_in and value_types.get(i, T.FLOAT) == T.FLOAT:
                    new_nodes.append(cast(i, i + "_to_fp32", T.FLOAT))
                    n.inputs[k] = i + "_to_fp32"
            outs = list(n.outputs)
            n.outputs = [o + "_fp32" if o and value_types.get(o, T.FLOAT) == T.FLOAT else o for o in outs]
            new_nodes.append(n)
            for o, o32 in zip(outs, n.outputs):
                if o != o32:
                    new_nodes.append(cast(o32, out_names.get(o, o), T.FLOAT16))
            continue
        for a in n.attributes:
            if a.type == ol.ATTR_TENSOR and a.value is not None and a.value.data_type == T.FLOAT:
                half = _to_half(ol.to_array(a.value), min_positive_val, max_finite_val)
                a.value.data_type, a.value.raw = T.FLOAT16, half.tobytes()
            if n.op_type == "Cast" and a.name == "to" and a.value == T.FLOAT:
                a.value = T.FLOAT16
            if a.name == "dtype" and a.value == T.FLOAT and n.op_type in ("RandomNormal", "RandomUniform", "EyeLike", "RandomNormalLike"):
                a.value = T.FLOAT16
        n.outputs = [out_names.get(o, o) for o in n.outputs]
        new_nodes.append(n)
    for orig, tmp in out_names.items():
        new_nodes.append(cast(tmp, orig, T.FLOAT))
    g.nodes = new_nodes
    return m
