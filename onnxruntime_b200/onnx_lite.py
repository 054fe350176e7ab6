"""A small stand-alone ONNX protobuf writer/reader in pure Python.

The ``onnx`` package is not required anywhere in this project: model builders,
exporters and tests author graphs with the helpers below (``make_node``,
``make_tensor``, ``make_graph``, ``make_model`` mirror ``onnx.helper``) and get
``ModelProto`` bytes back.  The encoder is independent from the C++ parser in
``csrc/core/onnx_pb.cc``, so round-trip tests check one against the other.

Field numbers follow onnx.proto (ModelProto, GraphProto, NodeProto,
AttributeProto, TensorProto, ValueInfoProto, TypeProto).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np


class TensorProto:
    UNDEFINED, FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL = range(10)
    FLOAT16, DOUBLE, UINT32, UINT64, COMPLEX64, COMPLEX128, BFLOAT16 = range(10, 17)
    FLOAT8E4M3FN, FLOAT8E4M3FNUZ, FLOAT8E5M2, FLOAT8E5M2FNUZ, UINT4, INT4, FLOAT4E2M1 = range(17, 24)


_NP_TO_ONNX = {
    np.dtype("float32"): TensorProto.FLOAT, np.dtype("uint8"): TensorProto.UINT8, np.dtype("int8"): TensorProto.INT8,
    np.dtype("uint16"): TensorProto.UINT16, np.dtype("int16"): TensorProto.INT16, np.dtype("int32"): TensorProto.INT32,
    np.dtype("int64"): TensorProto.INT64, np.dtype("bool"): TensorProto.BOOL, np.dtype("float16"): TensorProto.FLOAT16,
    np.dtype("float64"): TensorProto.DOUBLE, np.dtype("uint32"): TensorProto.UINT32,
    np.dtype("uint64"): TensorProto.UINT64,
}
_ONNX_TO_NP = {v: k for k, v in _NP_TO_ONNX.items()}

ATTR_FLOAT, ATTR_INT, ATTR_STRING, ATTR_TENSOR, ATTR_GRAPH, ATTR_FLOATS, ATTR_INTS, ATTR_STRINGS = 1, 2, 3, 4, 5, 6, 7, 8


# ------------------------------------------------------------------ wire writer
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _key(field_no: int, wire: int) -> bytes:
    return _varint((field_no << 3) | wire)


def _f_varint(field_no: int, v: int) -> bytes:
    return _key(field_no, 0) + _varint(int(v))


def _f_bytes(field_no: int, b: Union[bytes, bytearray, memoryview]) -> bytes:
    return _key(field_no, 2) + _varint(len(b)) + bytes(b)


def _f_str(field_no: int, s: Union[str, bytes]) -> bytes:
    return _f_bytes(field_no, s.encode("utf-8") if isinstance(s, str) else s)


def _f_float(field_no: int, v: float) -> bytes:
    return _key(field_no, 5) + struct.pack("<f", v)


def _packed_varints(field_no: int, vals: Iterable[int]) -> bytes:
    body = b"".join(_varint(int(v)) for v in vals)
    return _f_bytes(field_no, body) if body else b""


# ------------------------------------------------------------------ messages
@dataclass
class Tensor:
    name: str
    data_type: int
    dims: Tuple[int, ...]
    raw: bytes = b""
    external: Optional[Dict[str, str]] = None  # location / offset / length
    strings: Optional[List[bytes]] = None      # string tensors (data_type STRING): one entry per element

    def serialize(self) -> bytes:
        out = _packed_varints(1, self.dims)
        out += _f_varint(2, self.data_type)
        if self.name:
            out += _f_str(8, self.name)
        if self.strings is not None:
            for s in self.strings:
                out += _f_bytes(6, s)
        elif self.external is not None:
            for k, v in self.external.items():
                out += _f_bytes(13, _f_str(1, k) + _f_str(2, str(v)))
            out += _f_varint(14, 1)
        else:
            out += _f_bytes(9, self.raw)
        return out


@dataclass
class SparseTensor:
    """COO sparse initializer: `indices` are linear positions [nnz] or coordinates [nnz, rank]; the name is the values tensor's."""
    values: Tensor
    indices: Tensor
    dims: Tuple[int, ...]

    def serialize(self) -> bytes:
        return _f_bytes(1, self.values.serialize()) + _f_bytes(2, self.indices.serialize()) + _packed_varints(3, self.dims)


def make_sparse_tensor(name: str, dense) -> SparseTensor:
    """Sparse initializer holding the non-zeros of a dense numpy array (coordinates form)."""
    dense = np.asarray(dense)
    coords = np.argwhere(dense != 0).astype(np.int64)
    return SparseTensor(make_tensor(name, dense[dense != 0]), make_tensor("", coords.reshape(-1, dense.ndim)), tuple(dense.shape))


@dataclass
class ValueInfo:
    name: str
    elem_type: int = 0
    shape: Optional[Sequence[Union[int, str, None]]] = None

    def serialize(self) -> bytes:
        out = _f_str(1, self.name)
        if self.elem_type:
            tt = _f_varint(1, self.elem_type)
            if self.shape is not None:
                dims = b""
                for d in self.shape:
                    if isinstance(d, (int, np.integer)):
                        dims += _f_bytes(1, _f_varint(1, int(d)))
                    elif isinstance(d, str):
                        dims += _f_bytes(1, _f_str(2, d))
                    else:
                        dims += _f_bytes(1, b"")
                tt += _f_bytes(2, dims)
            out += _f_bytes(2, _f_bytes(1, tt))
        return out


@dataclass
class Attribute:
    name: str
    type: int
    value: Any

    def serialize(self) -> bytes:
        out = _f_str(1, self.name)
        t, v = self.type, self.value
        if t == ATTR_FLOAT:
            out += _f_float(2, float(v))
        elif t == ATTR_INT:
            out += _f_varint(3, int(v))
        elif t == ATTR_STRING:
            out += _f_str(4, v)
        elif t == ATTR_TENSOR:
            out += _f_bytes(5, v.serialize())
        elif t == ATTR_GRAPH:
            out += _f_bytes(6, v.serialize())
        elif t == ATTR_FLOATS:
            if len(v):
                out += _f_bytes(7, struct.pack(f"<{len(v)}f", *[float(x) for x in v]))
        elif t == ATTR_INTS:
            out += _packed_varints(8, v)
        elif t == ATTR_STRINGS:
            for s in v:
                out += _f_str(9, s)
        else:
            raise ValueError(f"unsupported attribute type {t}")
        out += _f_varint(20, t)
        return out


@dataclass
class Node:
    op_type: str
    inputs: List[str]
    outputs: List[str]
    name: str = ""
    domain: str = ""
    attributes: List[Attribute] = field(default_factory=list)

    def serialize(self) -> bytes:
        out = b"".join(_f_str(1, i) for i in self.inputs)
        out += b"".join(_f_str(2, o) for o in self.outputs)
        if self.name:
            out += _f_str(3, self.name)
        out += _f_str(4, self.op_type)
        out += b"".join(_f_bytes(5, a.serialize()) for a in self.attributes)
        if self.domain:
            out += _f_str(7, self.domain)
        return out


@dataclass
class Graph:
    nodes: List[Node]
    name: str
    inputs: List[ValueInfo]
    outputs: List[ValueInfo]
    initializers: List[Tensor] = field(default_factory=list)
    value_info: List[ValueInfo] = field(default_factory=list)
    sparse_initializers: List["SparseTensor"] = field(default_factory=list)

    def serialize(self) -> bytes:
        out = b"".join(_f_bytes(1, n.serialize()) for n in self.nodes)
        out += _f_str(2, self.name)
        out += b"".join(_f_bytes(5, t.serialize()) for t in self.initializers)
        out += b"".join(_f_bytes(15, t.serialize()) for t in self.sparse_initializers)
        out += b"".join(_f_bytes(11, v.serialize()) for v in self.inputs)
        out += b"".join(_f_bytes(12, v.serialize()) for v in self.outputs)
        out += b"".join(_f_bytes(13, v.serialize()) for v in self.value_info)
        return out


@dataclass
class Model:
    graph: Graph
    opset_imports: Dict[str, int]
    ir_version: int = 8
    producer_name: str = "onnxruntime_b200"
    metadata: Dict[str, str] = field(default_factory=dict)
    doc_string: str = ""

    def serialize(self) -> bytes:
        out = _f_varint(1, self.ir_version)
        out += _f_str(2, self.producer_name)
        if self.doc_string:
            out += _f_str(6, self.doc_string)
        out += _f_bytes(7, self.graph.serialize())
        for domain, version in self.opset_imports.items():
            body = (_f_str(1, domain) if domain else b"") + _f_varint(2, version)
            out += _f_bytes(8, body)
        for k, v in self.metadata.items():
            out += _f_bytes(14, _f_str(1, k) + _f_str(2, v))
        return out

    SerializeToString = serialize


# ------------------------------------------------------------------ helpers
def np_dtype_to_onnx(dt) -> int:
    dt = np.dtype(dt)
    if dt.kind in "OUS":   # object / unicode / bytes arrays hold strings
        return TensorProto.STRING
    return _NP_TO_ONNX[dt]


def onnx_to_np_dtype(t: int):
    return _ONNX_TO_NP[t]


def make_tensor(name: str, array, data_type: Optional[int] = None) -> Tensor:
    """Initializer from a numpy array or a torch tensor (bf16 / fp8 torch tensors keep their bits)."""
    try:
        import torch
    except ImportError:  # pragma: no cover
        torch = None
    if torch is not None and isinstance(array, torch.Tensor):
        t = array.detach().cpu().contiguous()
        tmap = {torch.float32: TensorProto.FLOAT, torch.float16: TensorProto.FLOAT16, torch.bfloat16: TensorProto.BFLOAT16,
                torch.int64: TensorProto.INT64, torch.int32: TensorProto.INT32, torch.int8: TensorProto.INT8,
                torch.uint8: TensorProto.UINT8, torch.bool: TensorProto.BOOL, torch.float64: TensorProto.DOUBLE,
                torch.int16: TensorProto.INT16, torch.float8_e4m3fn: TensorProto.FLOAT8E4M3FN,
                torch.float8_e5m2: TensorProto.FLOAT8E5M2}
        dt = data_type if data_type is not None else tmap[t.dtype]
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        return Tensor(name, dt, tuple(t.shape), raw)
    arr = np.asarray(array)
    if arr.dtype.kind in "USO":   # strings
        flat = [s if isinstance(s, bytes) else str(s).encode("utf-8") for s in arr.reshape(-1)]
        return Tensor(name, TensorProto.STRING, tuple(arr.shape), b"", None, flat)
    arr = np.ascontiguousarray(arr).reshape(arr.shape)  # ascontiguousarray promotes 0-d arrays to 1-d
    dt = data_type if data_type is not None else np_dtype_to_onnx(arr.dtype)
    return Tensor(name, dt, tuple(arr.shape), arr.tobytes())


def make_external_tensor(name: str, data_type: int, dims: Sequence[int], location: str = "*session*",
                         offset: Optional[int] = None, length: Optional[int] = None) -> Tensor:
    """Initializer whose bytes live outside the model.

    ``location="*session*"`` marks a tensor the caller hands to the session with
    ``SessionOptions.add_external_initializers``; any other value is a file name
    relative to the model's directory."""
    ext = {"location": location}
    if offset is not None:
        ext["offset"] = str(offset)
    if length is not None:
        ext["length"] = str(length)
    return Tensor(name, data_type, tuple(dims), b"", ext)


def make_tensor_value_info(name: str, elem_type: int, shape: Optional[Sequence[Union[int, str, None]]]) -> ValueInfo:
    return ValueInfo(name, elem_type, shape)


def make_attribute(name: str, value: Any) -> Attribute:
    if isinstance(value, bool):
        return Attribute(name, ATTR_INT, int(value))
    if isinstance(value, (int, np.integer)):
        return Attribute(name, ATTR_INT, int(value))
    if isinstance(value, (float, np.floating)):
        return Attribute(name, ATTR_FLOAT, float(value))
    if isinstance(value, (str, bytes)):
        return Attribute(name, ATTR_STRING, value)
    if isinstance(value, Tensor):
        return Attribute(name, ATTR_TENSOR, value)
    if isinstance(value, Graph):
        return Attribute(name, ATTR_GRAPH, value)
    if isinstance(value, np.ndarray):
        return Attribute(name, ATTR_TENSOR, make_tensor("", value))
    if isinstance(value, (list, tuple)):
        if len(value) == 0:
            return Attribute(name, ATTR_INTS, [])
        if all(isinstance(v, (int, np.integer)) and not isinstance(v, bool) for v in value):
            return Attribute(name, ATTR_INTS, list(value))
        if all(isinstance(v, (int, float, np.floating, np.integer)) for v in value):
            return Attribute(name, ATTR_FLOATS, list(value))
        if all(isinstance(v, (str, bytes)) for v in value):
            return Attribute(name, ATTR_STRINGS, list(value))
    raise TypeError(f"cannot infer the attribute type of {name}={value!r}")


def make_node(op_type: str, inputs: Sequence[str], outputs: Sequence[str], name: str = "", domain: str = "",
              **attrs: Any) -> Node:
    return Node(op_type, list(inputs), list(outputs), name, domain,
                [make_attribute(k, v) for k, v in attrs.items() if v is not None])


def make_graph(nodes: Sequence[Node], name: str, inputs: Sequence[ValueInfo], outputs: Sequence[ValueInfo],
               initializer: Sequence[Tensor] = (), value_info: Sequence[ValueInfo] = ()) -> Graph:
    return Graph(list(nodes), name, list(inputs), list(outputs), list(initializer), list(value_info))


def make_model(graph: Graph, opset: int = 17, ms_opset: Optional[int] = 1, ir_version: int = 8,
               producer_name: str = "onnxruntime_b200", metadata: Optional[Dict[str, str]] = None,
               extra_opsets: Optional[Dict[str, int]] = None) -> Model:
    opsets = {"": opset}
    if ms_opset is not None:
        opsets["com.microsoft"] = ms_opset
    if extra_opsets:
        opsets.update(extra_opsets)
    return Model(graph, opsets, ir_version, producer_name, dict(metadata or {}))


# ------------------------------------------------------------------ wire reader (for tests / tools)
def parse_message(buf: bytes) -> List[Tuple[int, int, Any]]:
    """Decode one protobuf message into (field, wire_type, value) triples; nested messages stay bytes."""
    out = []
    i, n = 0, len(buf)
    while i < n:
        key = 0
        shift = 0
        while True:
            b = buf[i]
            i += 1
            key |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        field_no, wire = key >> 3, key & 7
        if wire == 0:
            v = 0
            shift = 0
            while True:
                b = buf[i]
                i += 1
                v |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            out.append((field_no, wire, v))
        elif wire == 1:
            out.append((field_no, wire, buf[i:i + 8]))
            i += 8
        elif wire == 2:
            ln = 0
            shift = 0
            while True:
                b = buf[i]
                i += 1
                ln |= (b & 0x7F) << shift
                shift += 7
                if not b & 0x80:
                    break
            out.append((field_no, wire, buf[i:i + ln]))
            i += ln
        elif wire == 5:
            out.append((field_no, wire, buf[i:i + 4]))
            i += 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
    return out


# ------------------------------------------------------------------ model reader (tools edit models through it)
def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _unpack_varints(buf: bytes) -> List[int]:
    out, i, n = [], 0, len(buf)
    while i < n:
        v = shift = 0
        while True:
            b = buf[i]
            i += 1
            v |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                break
        out.append(_signed(v))
    return out


_TYPED_FIELD_DTYPES = {
    # storage of the non-raw TensorProto fields: field number -> numpy dtype of the stored values
    4: np.float32, 7: np.int64, 10: np.float64, 11: np.uint64,
}


def _tensor_from_fields(fields) -> Tensor:
    name, dt, dims, raw, ext = "", 0, [], None, None
    typed: Dict[int, List] = {}
    strings: List[bytes] = []
    for f, w, v in fields:
        if f == 6:
            strings.append(bytes(v))
        elif f == 1:
            dims += _unpack_varints(v) if w == 2 else [_signed(v)]
        elif f == 2:
            dt = v
        elif f == 8:
            name = bytes(v).decode()
        elif f == 9:
            raw = bytes(v)
        elif f == 13:
            kv = {ff: bytes(vv).decode() for ff, _, vv in parse_message(v)}
            ext = ext or {}
            ext[kv.get(1, "")] = kv.get(2, "")
        elif f in (4, 10):  # float_data / double_data: packed fixed-width or single values
            typed.setdefault(f, []).append(bytes(v))
        elif f in (5, 7, 11):  # int32_data / int64_data / uint64_data: packed varints or single values
            typed.setdefault(f, []).extend(_unpack_varints(v) if w == 2 else [_signed(v)])
    if raw is None and ext is None:
        if 4 in typed:
            raw = b"".join(typed[4])
        elif 10 in typed:
            raw = b"".join(typed[10])
        elif 7 in typed:
            raw = np.asarray(typed[7], dtype=np.int64).tobytes()
        elif 11 in typed:
            raw = np.asarray(typed[11], dtype=np.uint64).tobytes()
        elif 5 in typed:
            vals = np.asarray(typed[5], dtype=np.int64)
            if dt in (TensorProto.FLOAT16, TensorProto.BFLOAT16, TensorProto.UINT16):
                raw = vals.astype(np.uint16).tobytes()
            elif dt == TensorProto.INT16:
                raw = vals.astype(np.int16).tobytes()
            elif dt in (TensorProto.INT8,):
                raw = vals.astype(np.int8).tobytes()
            elif dt in (TensorProto.UINT8, TensorProto.BOOL, TensorProto.FLOAT8E4M3FN, TensorProto.FLOAT8E4M3FNUZ,
                        TensorProto.FLOAT8E5M2, TensorProto.FLOAT8E5M2FNUZ, TensorProto.UINT4, TensorProto.INT4):
                raw = vals.astype(np.uint8).tobytes()
            else:
                raw = vals.astype(np.int32).tobytes()
        else:
            raw = b""
    return Tensor(name, dt, tuple(dims), raw or b"", ext, strings if dt == TensorProto.STRING else None)


def _value_info_from_bytes(buf: bytes) -> ValueInfo:
    name, elem, shape = "", 0, None
    for f, _, v in parse_message(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            for f2, _, v2 in parse_message(v):
                if f2 != 1:
                    continue  # only tensor types carry a shape here
                for f3, _, v3 in parse_message(v2):
                    if f3 == 1:
                        elem = v3
                    elif f3 == 2:
                        shape = []
                        for f4, _, v4 in parse_message(v3):
                            if f4 != 1:
                                continue
                            d: Union[int, str, None] = None
                            for f5, _, v5 in parse_message(v4):
                                if f5 == 1:
                                    d = _signed(v5)
                                elif f5 == 2:
                                    d = bytes(v5).decode()
                            shape.append(d)
    return ValueInfo(name, elem, shape)


def _attribute_from_bytes(buf: bytes) -> Attribute:
    name, atype = "", 0
    f_val = i_val = s_val = t_val = g_val = None
    floats: List[float] = []
    ints: List[int] = []
    strings: List[bytes] = []
    for f, w, v in parse_message(buf):
        if f == 1:
            name = bytes(v).decode()
        elif f == 2:
            f_val = struct.unpack("<f", v)[0]
        elif f == 3:
            i_val = _signed(v)
        elif f == 4:
            s_val = bytes(v)
        elif f == 5:
            t_val = _tensor_from_fields(parse_message(v))
        elif f == 6:
            g_val = _graph_from_bytes(v)
        elif f == 7:
            floats += list(struct.unpack(f"<{len(v) // 4}f", v)) if w == 2 else [struct.unpack("<f", v)[0]]
        elif f == 8:
            ints += _unpack_varints(v) if w == 2 else [_signed(v)]
        elif f == 9:
            strings.append(bytes(v))
        elif f == 20:
            atype = v
    if not atype:  # writers before IR 4 did not set the type
        atype = (ATTR_FLOAT if f_val is not None else ATTR_INT if i_val is not None else ATTR_STRING if s_val is not None else
                 ATTR_TENSOR if t_val is not None else ATTR_GRAPH if g_val is not None else ATTR_FLOATS if floats else
                 ATTR_INTS if ints else ATTR_STRINGS)
    value = {ATTR_FLOAT: f_val if f_val is not None else 0.0, ATTR_INT: i_val if i_val is not None else 0,
             ATTR_STRING: s_val if s_val is not None else b"", ATTR_TENSOR: t_val, ATTR_GRAPH: g_val, ATTR_FLOATS: floats,
             ATTR_INTS: ints, ATTR_STRINGS: strings}.get(atype)
    return Attribute(name, atype, value)


def _node_from_bytes(buf: bytes) -> Node:
    n = Node("", [], [])
    for f, _, v in parse_message(buf):
        if f == 1:
            n.inputs.append(bytes(v).decode())
        elif f == 2:
            n.outputs.append(bytes(v).decode())
        elif f == 3:
            n.name = bytes(v).decode()
        elif f == 4:
            n.op_type = bytes(v).decode()
        elif f == 5:
            n.attributes.append(_attribute_from_bytes(v))
        elif f == 7:
            n.domain = bytes(v).decode()
    return n


def _graph_from_bytes(buf: bytes) -> Graph:
    g = Graph([], "", [], [])
    for f, _, v in parse_message(buf):
        if f == 1:
            g.nodes.append(_node_from_bytes(v))
        elif f == 2:
            g.name = bytes(v).decode()
        elif f == 5:
            g.initializers.append(_tensor_from_fields(parse_message(v)))
        elif f == 11:
            g.inputs.append(_value_info_from_bytes(v))
        elif f == 12:
            g.outputs.append(_value_info_from_bytes(v))
        elif f == 13:
            g.value_info.append(_value_info_from_bytes(v))
    return g


def load_model(source: Union[str, bytes, bytearray, memoryview]) -> Model:
    """ModelProto bytes (or a file path) -> editable ``Model``.  Functions, training info and sparse
    initializers are not carried over; tools that need them should work on the bytes."""
    if isinstance(source, str):
        with open(source, "rb") as f:
            source = f.read()
    m = Model(Graph([], "", [], []), {})
    for f, _, v in parse_message(bytes(source)):
        if f == 1:
            m.ir_version = v
        elif f == 2:
            m.producer_name = bytes(v).decode()
        elif f == 6:
            m.doc_string = bytes(v).decode()
        elif f == 7:
            m.graph = _graph_from_bytes(v)
        elif f == 8:
            domain, version = "", 0
            for f2, _, v2 in parse_message(v):
                if f2 == 1:
                    domain = bytes(v2).decode()
                elif f2 == 2:
                    version = v2
            m.opset_imports[domain] = version
        elif f == 14:
            kv = {ff: bytes(vv).decode() for ff, _, vv in parse_message(v)}
            m.metadata[kv.get(1, "")] = kv.get(2, "")
    return m


def load_tensor(source: Union[str, bytes]) -> Tensor:
    """A serialized TensorProto (the ``input_0.pb`` files of ONNX test data sets) -> ``Tensor``."""
    if isinstance(source, str):
        with open(source, "rb") as f:
            source = f.read()
    return _tensor_from_fields(parse_message(bytes(source)))


def to_array(t: Tensor):
    """Initializer -> numpy array; bf16 and fp8 tensors come back as torch tensors (numpy has no such types)."""
    if t.external is not None:
        raise ValueError(f"tensor {t.name!r} keeps its data outside the model")
    shape = tuple(int(d) for d in t.dims)
    if t.data_type in _ONNX_TO_NP:
        return np.frombuffer(t.raw, dtype=_ONNX_TO_NP[t.data_type]).reshape(shape).copy()
    import torch
    tmap = {TensorProto.BFLOAT16: torch.bfloat16, TensorProto.FLOAT8E4M3FN: torch.float8_e4m3fn, TensorProto.FLOAT8E5M2: torch.float8_e5m2}
    if t.data_type in tmap:
        return torch.frombuffer(bytearray(t.raw), dtype=torch.uint8).view(tmap[t.data_type]).reshape(shape)
    raise TypeError(f"no array type for ONNX data type {t.data_type}")


def attr_value(node: Node, name: str, default: Any = None) -> Any:
    for a in node.attributes:
        if a.name == name:
            return a.value
    return default
