"""Reader and writer for the reference's LoRA adapter files (FlatBuffers, file identifier ``TORT``).

Schema (onnxruntime/lora/adapter_format/adapter_schema.fbs of the reference)::

    table Parameter { name:string; dims:[int64]; data_type:TensorDataType; raw_data:[uint8] (force_align: 8); }
    table Adapter   { format_version:int; adapter_version:int; model_version:int; parameters:[Parameter]; }
    root_type Adapter;  file_identifier "TORT";

Only what this schema needs of the FlatBuffers wire format is implemented: a table starts with a signed 32-bit
offset back to its vtable (``vtable = table - soffset``); the vtable holds its own size, the table's inline size and
one 16-bit in-table offset per field (0 = absent, the default applies); scalars are stored inline, strings / vectors
/ tables through unsigned 32-bit offsets relative to the referring slot; a vector is a 32-bit count followed by its
elements; a string additionally ends with a zero byte.  ``TensorDataType`` uses the ONNX TensorProto numbering.
"""
from __future__ import annotations

import struct
from typing import List, Tuple

FILE_IDENTIFIER = b"TORT"
ADAPTER_FORMAT_VERSION = 1

Parameter = Tuple[str, List[int], int, bytes]   # name, dims, ONNX element type, raw little-endian data


class _Table:
    def __init__(self, buf: bytes, pos: int):
        if pos < 0 or pos + 4 > len(buf):
            raise ValueError("table offset outside the buffer")
        self.buf, self.pos = buf, pos
        (so,) = struct.unpack_from("<i", buf, pos)
        self.vt = pos - so
        if self.vt < 0 or self.vt + 4 > len(buf):
            raise ValueError("vtable offset outside the buffer")
        self.vt_size, self.inline_size = struct.unpack_from("<HH", buf, self.vt)
        if self.vt + self.vt_size > len(buf) or pos + self.inline_size > len(buf):
            raise ValueError("table does not fit the buffer")

    def _slot(self, field: int) -> int:
        off = 4 + 2 * field
        if off + 2 > self.vt_size:
            return 0
        (rel,) = struct.unpack_from("<H", self.buf, self.vt + off)
        return self.pos + rel if rel else 0

    def scalar(self, field: int, fmt: str, default=0):
        slot = self._slot(field)
        if not slot:
            return default
        return struct.unpack_from("<" + fmt, self.buf, slot)[0]

    def _indirect(self, field: int) -> int:
        slot = self._slot(field)
        if not slot:
            return 0
        (rel,) = struct.unpack_from("<I", self.buf, slot)
        target = slot + rel
        if target + 4 > len(self.buf):
            raise ValueError("offset outside the buffer")
        return target

    def string(self, field: int) -> str:
        p = self._indirect(field)
        if not p:
            return ""
        (n,) = struct.unpack_from("<I", self.buf, p)
        if p + 4 + n > len(self.buf):
            raise ValueError("string outside the buffer")
        return bytes(self.buf[p + 4:p + 4 + n]).decode("utf-8")

    def vector(self, field: int, elem_size: int) -> Tuple[int, int]:
        """(position of the first element, count)"""
        p = self._indirect(field)
        if not p:
            return 0, 0
        (n,) = struct.unpack_from("<I", self.buf, p)
        if p + 4 + n * elem_size > len(self.buf):
            raise ValueError("vector outside the buffer")
        return p + 4, n


def is_adapter_flatbuffer(buf: bytes) -> bool:
    return len(buf) >= 8 and bytes(buf[4:8]) == FILE_IDENTIFIER


def read_adapter(buf: bytes):
    """-> (format_version, adapter_version, model_version, [Parameter])"""
    if not is_adapter_flatbuffer(buf):
        raise ValueError("not an adapter flatbuffer (file identifier TORT missing)")
    (root,) = struct.unpack_from("<I", buf, 0)
    t = _Table(buf, root)
    fmt, av, mv = t.scalar(0, "i"), t.scalar(1, "i"), t.scalar(2, "i")
    first, n = t.vector(3, 4)
    params: List[Parameter] = []
    for i in range(n):
        slot = first + 4 * i
        (rel,) = struct.unpack_from("<I", buf, slot)
        p = _Table(buf, slot + rel)
        name = p.string(0)
        dpos, dn = p.vector(1, 8)
        dims = list(struct.unpack_from("<%dq" % dn, buf, dpos)) if dn else []
        dtype = p.scalar(2, "i")
        rpos, rn = p.vector(3, 1)
        params.append((name, dims, dtype, bytes(buf[rpos:rpos + rn])))
    return fmt, av, mv, params


def write_adapter(adapter_version: int, model_version: int, params: List[Parameter],
                  format_version: int = ADAPTER_FORMAT_VERSION) -> bytes:
    buf = bytearray()

    def align(n: int, bias: int = 0) -> None:
        while (len(buf) + bias) % n:
            buf.append(0)

    def patch(slot: int, target: int) -> None:
        struct.pack_into("<I", buf, slot, target - slot)

    buf += b"\0\0\0\0" + FILE_IDENTIFIER
    # Adapter: vtable (12 bytes: sizes + 4 fields), then the table (vtable offset + 3 ints + 1 offset = 20 bytes)
    vt = len(buf)
    buf += struct.pack("<HHHHHH", 12, 20, 4, 8, 12, 16)
    align(4)
    tab = len(buf)
    buf += struct.pack("<iiii", tab - vt, int(format_version), int(adapter_version), int(model_version)) + b"\0\0\0\0"
    struct.pack_into("<I", buf, 0, tab)
    align(4)
    vec = len(buf)
    patch(tab + 16, vec)
    buf += struct.pack("<I", len(params)) + b"\0" * (4 * len(params))
    # one vtable shared by all Parameter tables: name, dims, data_type, raw_data at 4, 8, 12, 16
    pvt = len(buf)
    buf += struct.pack("<HHHHHH", 12, 20, 4, 8, 12, 16)
    tables = []
    for i, (name, dims, dtype, raw) in enumerate(params):
        align(4)
        pt = len(buf)
        buf += struct.pack("<i", pt - pvt) + b"\0\0\0\0" + b"\0\0\0\0" + struct.pack("<i", int(dtype)) + b"\0\0\0\0"
        patch(vec + 4 + 4 * i, pt)
        tables.append(pt)
    for pt, (name, dims, dtype, raw) in zip(tables, params):
        align(4)
        patch(pt + 4, len(buf))
        nb = name.encode("utf-8")
        buf += struct.pack("<I", len(nb)) + nb + b"\0"
        align(8, bias=4)          # the int64 elements (behind the 32-bit count) sit on an 8-byte boundary
        patch(pt + 8, len(buf))
        buf += struct.pack("<I", len(dims)) + struct.pack("<%dq" % len(dims), *[int(d) for d in dims])
        align(8, bias=4)          # force_align: 8 for the data
        patch(pt + 16, len(buf))
        buf += struct.pack("<I", len(raw)) + bytes(raw)
    align(8)
    return bytes(buf)


# ------------------------------------------------------------------------------------------------------------------
# Generic helpers used by the ORT-format reader / writer (ort_format.py)
class Table(_Table):
    """Read access to one FlatBuffers table by field index."""

    def table(self, field: int):
        p = self._indirect(field)
        return Table(self.buf, p) if p else None

    def tables(self, field: int) -> List["Table"]:
        first, n = self.vector(field, 4)
        out = []
        for i in range(n):
            slot = first + 4 * i
            (rel,) = struct.unpack_from("<I", self.buf, slot)
            out.append(Table(self.buf, slot + rel))
        return out

    def strings(self, field: int) -> List[str]:
        first, n = self.vector(field, 4)
        out = []
        for i in range(n):
            slot = first + 4 * i
            (rel,) = struct.unpack_from("<I", self.buf, slot)
            p = slot + rel
            (ln,) = struct.unpack_from("<I", self.buf, p)
            if p + 4 + ln > len(self.buf):
                raise ValueError("string outside the buffer")
            out.append(bytes(self.buf[p + 4:p + 4 + ln]).decode("utf-8"))
        return out

    def scalars(self, field: int, fmt: str) -> list:
        size = struct.calcsize("<" + fmt)
        first, n = self.vector(field, size)
        return list(struct.unpack_from("<%d%s" % (n, fmt), self.buf, first)) if n else []

    def bytes_(self, field: int) -> bytes:
        first, n = self.vector(field, 1)
        return bytes(self.buf[first:first + n])


def root_table(buf: bytes, identifier: bytes) -> Table:
    if len(buf) < 8 or bytes(buf[4:8]) != identifier:
        raise ValueError("file identifier %r missing" % identifier)
    (root,) = struct.unpack_from("<I", buf, 0)
    return Table(buf, root)


_SCALAR = {"i8": "b", "u8": "B", "bool": "?", "i32": "i", "u32": "I", "i64": "q", "u64": "Q", "f32": "f"}


class Builder:
    """Forward-writing FlatBuffers builder: a table is described as a list ``[(kind, value) or None, ...]`` indexed by
    field id.  Kinds: the scalar names of ``_SCALAR``; ``str``; ``table`` (a nested description); ``vec_table``;
    ``vec_str``; ``vec_<scalar>`` (``vec_u8`` takes bytes).  Every referenced object is written behind the table that
    refers to it, so all offsets point forward as the format requires."""

    def __init__(self, identifier: bytes):
        self.buf = bytearray(b"\0\0\0\0" + identifier)

    def _align(self, n: int, bias: int = 0) -> None:
        while (len(self.buf) + bias) % n:
            self.buf.append(0)

    def _patch(self, slot: int, target: int) -> None:
        struct.pack_into("<I", self.buf, slot, target - slot)

    def finish(self, root_fields) -> bytes:
        pos = self._table(root_fields)
        struct.pack_into("<I", self.buf, 0, pos)
        self._align(8)
        return bytes(self.buf)

    def _table(self, fields) -> int:
        # inline layout: 4-byte vtable offset, then the present fields in order with natural alignment
        layout, off, big = [], 4, 4
        for f in fields:
            if f is None:
                layout.append(0)
                continue
            kind = f[0]
            size = struct.calcsize("<" + _SCALAR[kind]) if kind in _SCALAR else 4
            off = (off + size - 1) // size * size
            layout.append(off)
            off += size
            big = max(big, size)
        inline = (off + 3) // 4 * 4
        self._align(2)
        vt_size = 4 + 2 * len(fields)
        # the table must start on a `big` boundary: pad in front of the vtable
        self._align(big, bias=vt_size + (-vt_size % 4))
        vt = len(self.buf)
        self.buf += struct.pack("<HH", vt_size, inline) + b"".join(struct.pack("<H", o) for o in layout)
        self._align(4)
        tab = len(self.buf)
        assert tab % big == 0
        self.buf += struct.pack("<i", tab - vt) + b"\0" * (inline - 4)
        pending = []
        for f, o in zip(fields, layout):
            if f is None:
                continue
            kind, value = f
            if kind in _SCALAR:
                struct.pack_into("<" + _SCALAR[kind], self.buf, tab + o, value)
            else:
                pending.append((tab + o, kind, value))
        for slot, kind, value in pending:
            self._patch(slot, self._object(kind, value))
        return tab

    def _string(self, s: str) -> int:
        self._align(4)
        pos = len(self.buf)
        b = s.encode("utf-8")
        self.buf += struct.pack("<I", len(b)) + b + b"\0"
        return pos

    def _object(self, kind: str, value) -> int:
        if kind == "str":
            return self._string(value)
        if kind == "table":
            return self._table(value)
        if kind in ("vec_table", "vec_str"):
            self._align(4)
            pos = len(self.buf)
            self.buf += struct.pack("<I", len(value)) + b"\0" * (4 * len(value))
            for i, v in enumerate(value):
                target = self._table(v) if kind == "vec_table" else self._string(v)
                self._patch(pos + 4 + 4 * i, target)
            return pos
        if kind.startswith("vec_"):
            fmt = _SCALAR[kind[4:]]
            size = struct.calcsize("<" + fmt)
            self._align(max(size, 8) if kind == "vec_u8" else max(size, 4), bias=4)
            pos = len(self.buf)
            if kind == "vec_u8":
                self.buf += struct.pack("<I", len(value)) + bytes(value)
            else:
                self.buf += struct.pack("<I", len(value)) + struct.pack("<%d%s" % (len(value), fmt), *value)
            return pos
        raise ValueError("unknown kind " + kind)
