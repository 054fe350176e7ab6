"""ORT-format models (``.ort``): the reference's FlatBuffers serialisation of a model (file identifier ``ORTM``).

Schema: onnxruntime/core/flatbuffers/schema/ort.fbs of the reference (root table ``InferenceSession`` holding
``ort_version``, ``model`` and a kernel type-string resolver).  ``ort_to_onnx`` turns such a file into the ONNX
model this runtime loads; ``onnx_to_ort`` writes one (used by ``session.save_model_format = ORT``, by
``tools/convert_onnx_models_to_ort.py`` and by the tests).  Field indices below follow the schema's declaration
order; a union occupies two consecutive indices (type tag, then value).

Not carried over: sparse initializers, runtime-optimization records and the kernel type-string resolver (this
runtime resolves kernels from its own registry), and node edges (they are recomputed from the value names).
"""
from __future__ import annotations

from typing import Dict, List, Optional

from . import flatbuf_lite as fb
from . import onnx_lite as ol

IDENTIFIER = b"ORTM"
ORT_VERSION = "1.23.0-ortb200"   # written into files; any value is accepted on load

# field indices --------------------------------------------------------------------------------------------------
_IS_ORT_VERSION, _IS_MODEL, _IS_RESOLVER = 0, 1, 3
_M_IR, _M_OPSETS, _M_PRODUCER, _M_PRODUCER_VER, _M_DOMAIN, _M_VERSION, _M_DOC, _M_GRAPH, _M_GRAPH_DOC, _M_META = range(10)
_G_INITS, _G_NODE_ARGS, _G_NODES, _G_MAX_NODE, _G_EDGES, _G_INPUTS, _G_OUTPUTS = range(7)
_N_NAME, _N_DOC, _N_DOMAIN, _N_SINCE, _N_INDEX, _N_OP, _N_TYPE, _N_EP, _N_INPUTS, _N_OUTPUTS, _N_ATTRS, _N_ARG_COUNTS, _N_IMPLICIT = range(13)
_A_NAME, _A_DOC, _A_TYPE, _A_F, _A_I, _A_S, _A_T, _A_G, _A_FLOATS, _A_INTS, _A_STRINGS, _A_TENSORS, _A_GRAPHS = range(13)
_T_NAME, _T_DOC, _T_DIMS, _T_TYPE, _T_RAW, _T_STRINGS, _T_EXT_OFFSET = range(7)
_VI_NAME, _VI_DOC, _VI_TYPE = range(3)
_TI_DENOTATION, _TI_VALUE_TYPE, _TI_VALUE = range(3)
_TS_ELEM, _TS_SHAPE = range(2)
_DIM_VALUE, _DIM_DENOTATION = range(2)
_DV_TYPE, _DV_VALUE, _DV_PARAM = range(3)


def is_ort_format(buf) -> bool:
    return len(buf) >= 8 and bytes(buf[4:8]) == IDENTIFIER


# ------------------------------------------------------------------------------------------------------- reading
def _tensor(t: fb.Table) -> ol.Tensor:
    strings = t.strings(_T_STRINGS)
    if strings:
        return ol.Tensor(t.string(_T_NAME), ol.TensorProto.STRING, tuple(t.scalars(_T_DIMS, "q")), b"", None,
                         [s.encode("utf-8") if isinstance(s, str) else bytes(s) for s in strings])
    if t.scalar(_T_EXT_OFFSET, "q", -1) != -1:
        raise ValueError(f"initializer '{t.string(_T_NAME)}' lives in an external file, which is not supported for ORT-format models")
    return ol.Tensor(t.string(_T_NAME), t.scalar(_T_TYPE, "i"), tuple(t.scalars(_T_DIMS, "q")), t.bytes_(_T_RAW))


def _value_info(v: fb.Table) -> ol.ValueInfo:
    name = v.string(_VI_NAME)
    ti = v.table(_VI_TYPE)
    if ti is None or ti.scalar(_TI_VALUE_TYPE, "B") != 1:        # 1 = tensor_type; sequences / maps keep the name only
        return ol.ValueInfo(name)
    ts = ti.table(_TI_VALUE)
    shape_t = ts.table(_TS_SHAPE)
    shape = None
    if shape_t is not None:
        shape = []
        for d in shape_t.tables(0):
            dv = d.table(_DIM_VALUE)
            kind = dv.scalar(_DV_TYPE, "b") if dv is not None else 0
            shape.append(int(dv.scalar(_DV_VALUE, "q")) if kind == 1 else (dv.string(_DV_PARAM) if kind == 2 else None))
    return ol.ValueInfo(name, ts.scalar(_TS_ELEM, "i"), shape)


def _attribute(a: fb.Table) -> ol.Attribute:
    name, t = a.string(_A_NAME), a.scalar(_A_TYPE, "i")
    if t == ol.ATTR_FLOAT:
        return ol.Attribute(name, t, a.scalar(_A_F, "f"))
    if t == ol.ATTR_INT:
        return ol.Attribute(name, t, a.scalar(_A_I, "q"))
    if t == ol.ATTR_STRING:
        return ol.Attribute(name, t, a.string(_A_S))
    if t == ol.ATTR_TENSOR:
        return ol.Attribute(name, t, _tensor(a.table(_A_T)))
    if t == ol.ATTR_GRAPH:
        return ol.Attribute(name, t, _graph(a.table(_A_G), name))
    if t == ol.ATTR_FLOATS:
        return ol.Attribute(name, t, a.scalars(_A_FLOATS, "f"))
    if t == ol.ATTR_INTS:
        return ol.Attribute(name, t, a.scalars(_A_INTS, "q"))
    if t == ol.ATTR_STRINGS:
        return ol.Attribute(name, t, a.strings(_A_STRINGS))
    raise ValueError(f"attribute '{name}' has type {t}, which is not supported")


def _graph(g: fb.Table, name: str) -> ol.Graph:
    inits = [_tensor(t) for t in g.tables(_G_INITS)]
    infos: Dict[str, ol.ValueInfo] = {}
    for v in g.tables(_G_NODE_ARGS):
        vi = _value_info(v)
        infos[vi.name] = vi
    nodes = []
    for n in sorted(g.tables(_G_NODES), key=lambda n: n.scalar(_N_INDEX, "I")):
        nodes.append(ol.Node(n.string(_N_OP), n.strings(_N_INPUTS), n.strings(_N_OUTPUTS), n.string(_N_NAME), n.string(_N_DOMAIN),
                             [_attribute(a) for a in n.tables(_N_ATTRS)]))
    in_names, out_names = g.strings(_G_INPUTS), g.strings(_G_OUTPUTS)
    take = lambda names: [infos.get(n, ol.ValueInfo(n)) for n in names]
    inner = set(in_names) | set(out_names)
    return ol.Graph(nodes, name, take(in_names), take(out_names), inits, [v for k, v in infos.items() if k not in inner and v.elem_type])


def ort_to_onnx(buf) -> ol.Model:
    """Parse an ORT-format buffer into an ONNX model description (``onnx_lite.Model``)."""
    buf = bytes(buf)
    root = fb.root_table(buf, IDENTIFIER)
    m = root.table(_IS_MODEL)
    if m is None:
        raise ValueError("ORT-format file without a model")
    opsets = {("" if o.string(0) == "ai.onnx" else o.string(0)): int(o.scalar(1, "q")) for o in m.tables(_M_OPSETS)}
    g = m.table(_M_GRAPH)
    if g is None:
        raise ValueError("ORT-format model without a graph")
    meta = {e.string(0): e.string(1) for e in m.tables(_M_META)}
    model = ol.Model(_graph(g, "main_graph"), opsets, int(m.scalar(_M_IR, "q")) or 8, m.string(_M_PRODUCER) or "onnxruntime", meta,
                     m.string(_M_DOC))
    return model


# ------------------------------------------------------------------------------------------------------- writing
def _w_tensor(t: ol.Tensor):
    if t.external is not None:
        raise ValueError(f"initializer '{t.name}' uses external data; load it before converting")
    if t.strings is not None:
        return [("str", t.name), None, ("vec_i64", [int(d) for d in t.dims]), ("i32", int(t.data_type)), None,
                ("vec_str", [s.decode("utf-8") if isinstance(s, (bytes, bytearray)) else str(s) for s in t.strings])]
    return [("str", t.name), None, ("vec_i64", [int(d) for d in t.dims]), ("i32", int(t.data_type)), ("vec_u8", bytes(t.raw))]


def _w_value_info(v: ol.ValueInfo):
    if not v.elem_type:
        return [("str", v.name)]
    ts = [("i32", int(v.elem_type))]
    if v.shape is not None:
        dims = []
        for d in v.shape:
            if isinstance(d, str):
                dv = [("i8", 2), None, ("str", d)]
            elif d is None:
                dv = [("i8", 0)]
            else:
                dv = [("i8", 1), ("i64", int(d))]
            dims.append([("table", dv)])
        ts.append(("table", [("vec_table", dims)]))
    return [("str", v.name), None, ("table", [None, ("u8", 1), ("table", ts)])]


def _w_attribute(a: ol.Attribute):
    f: List[Optional[tuple]] = [("str", a.name), None, ("i32", int(a.type))] + [None] * 10
    t, v = a.type, a.value
    if t == ol.ATTR_FLOAT:
        f[_A_F] = ("f32", float(v))
    elif t == ol.ATTR_INT:
        f[_A_I] = ("i64", int(v))
    elif t == ol.ATTR_STRING:
        f[_A_S] = ("str", v.decode() if isinstance(v, (bytes, bytearray)) else str(v))
    elif t == ol.ATTR_TENSOR:
        f[_A_T] = ("table", _w_tensor(v))
    elif t == ol.ATTR_GRAPH:
        f[_A_G] = ("table", _w_graph(v))
    elif t == ol.ATTR_FLOATS:
        f[_A_FLOATS] = ("vec_f32", [float(x) for x in v])
    elif t == ol.ATTR_INTS:
        f[_A_INTS] = ("vec_i64", [int(x) for x in v])
    elif t == ol.ATTR_STRINGS:
        f[_A_STRINGS] = ("vec_str", [s.decode() if isinstance(s, (bytes, bytearray)) else str(s) for s in v])
    else:
        raise ValueError(f"attribute '{a.name}' has type {t}, which is not supported")
    return f


def _w_graph(g: ol.Graph, opsets: Optional[Dict[str, int]] = None):
    infos = {v.name: v for v in list(g.value_info) + list(g.inputs) + list(g.outputs)}
    nodes = []
    for i, n in enumerate(g.nodes):
        since = (opsets or {}).get(n.domain if n.domain != "ai.onnx" else "", 0)
        nodes.append([("str", n.name), None, ("str", n.domain), ("i32", int(since)), ("u32", i), ("str", n.op_type), ("i32", 0), None,
                      ("vec_str", list(n.inputs)), ("vec_str", list(n.outputs)), ("vec_table", [_w_attribute(a) for a in n.attributes])])
    return [("vec_table", [_w_tensor(t) for t in g.initializers]), ("vec_table", [_w_value_info(v) for v in infos.values()]),
            ("vec_table", nodes), ("u32", max(len(g.nodes) - 1, 0)), None,
            ("vec_str", [v.name for v in g.inputs]), ("vec_str", [v.name for v in g.outputs])]


def onnx_to_ort(model: ol.Model) -> bytes:
    """Serialise an ONNX model description as an ORT-format buffer."""
    m = [("i64", int(model.ir_version)),
         ("vec_table", [[("str", d), ("i64", int(v))] for d, v in model.opset_imports.items()]),
         ("str", model.producer_name), None, None, None, ("str", model.doc_string or ""),
         ("table", _w_graph(model.graph, model.opset_imports)), None,
         ("vec_table", [[("str", k), ("str", v)] for k, v in model.metadata.items()])]
    root = [("str", ORT_VERSION), ("table", m), None, ("table", [("vec_table", [])])]
    return fb.Builder(IDENTIFIER).finish(root)
