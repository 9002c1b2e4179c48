"""Read and write `.dab` model files without the FlatBuffers library.

A `.dab` file is a little-endian FlatBuffers buffer whose root is `flatbnn.Model`
(reference common/dab.fbs:146-153).  Field slots (vtable byte offsets) are those of the reference's
generated accessors, common/dab_generated.h: Model :1799-1802, Layer :1555-1570, Tensor :145-150,
Input :261-262, conv params :389-395, pool params :663-667, FC :1009-1012, Add :1101-1103,
Concat :1179-1181, Affine :1385-1388, PRelu :1477-1479, two-string layers (Relu, Softmax,
Binarize, Shuffle) :325-326.

FlatBuffers wire format used here: the file starts with a uint32 offset to the root table; a table
starts with an int32 (table position minus vtable position) followed by its inline fields; a vtable
is {uint16 vtable bytes, uint16 table bytes, uint16 field offset per slot (0 = absent)}; strings,
vectors and sub-tables are referenced by uint32 offsets relative to the referring field; a vector
is {uint32 count, elements}; a string is {uint32 length, bytes, NUL}.  The writer lays children out
after their parent, which keeps every such offset positive.

The C++ runtime has its own reader (csrc/dab_reader.h); this module is what produces model files
(synthetic networks, converted weights) and is cross-checked against that reader in the tests.
"""
from __future__ import annotations

import struct

import numpy as np

from .model_spec import LAYER_TYPES, LayerSpec, ModelSpec, TensorSpec

# (field name, slot id, kind) per parameter table; slot byte offset in the vtable = 4 + 2*id
_CONV = [("input", 0, "str"), ("weight", 1, "str"), ("bias", 2, "str"), ("pads", 3, "vi32"),
         ("strides", 4, "vi32"), ("dilations", 5, "vi32"), ("output", 6, "str")]
_POOL = [("input", 0, "str"), ("kernel_shape", 1, "vi32"), ("pads", 2, "vi32"), ("strides", 3, "vi32"),
         ("output", 4, "str")]
_IO = [("input", 0, "str"), ("output", 1, "str")]
PARAM_TABLES = {
    "FpConv2D": (1, _CONV), "BinConv2D": (2, _CONV), "AvePool": (3, _POOL), "MaxPool": (4, _POOL),
    "Relu": (5, _IO), "Softmax": (6, _IO),
    "FC": (7, [("input", 0, "str"), ("weight", 1, "str"), ("bias", 2, "str"), ("output", 3, "str")]),
    "Add": (8, [("input1", 0, "str"), ("input2", 1, "str"), ("output", 2, "str")]),
    "Concat": (9, [("inputs", 0, "vstr"), ("axis", 1, "i32"), ("output", 2, "str")]),
    "Affine": (10, [("input", 0, "str"), ("a", 1, "str"), ("b", 2, "str"), ("output", 3, "str")]),
    "Binarize": (11, _IO),
    "Split": (12, [("input", 0, "str"), ("outputs", 1, "vstr")]),
    "Shuffle": (13, _IO),
    "PRelu": (15, [("input", 0, "str"), ("slope", 1, "str"), ("output", 2, "str")]),
}
_LAYER_NAME_SLOT = 14

_SCALAR = {"u8": "<B", "i8": "<b", "bool": "<B", "u32": "<I", "i32": "<i"}
_VEC_DTYPE = {"vu64": np.uint64, "vf32": np.float32, "vu32": np.uint32, "vi32": np.int32}


# ------------------------------------------------------------------------------------ writer
class _Writer:
    def __init__(self):
        self.b = bytearray()

    def _align(self, n, bias=0):
        while (len(self.b) + bias) % n:
            self.b.append(0)

    def _patch_offset(self, field_pos, target):
        struct.pack_into("<I", self.b, field_pos, target - field_pos)

    def table(self, fields):
        """fields: list of (slot id, kind, value); returns the table position."""
        fields = [f for f in fields if f[2] is not None]
        nslots = max((f[0] for f in fields), default=-1) + 1
        # inline layout: int32 vtable offset, then 4-byte fields, then 1-byte fields
        order = sorted(fields, key=lambda f: 0 if f[1] not in ("u8", "i8", "bool") else 1)
        off, layout = 4, {}
        for slot, kind, _ in order:
            layout[slot] = off
            off += 1 if kind in ("u8", "i8", "bool") else 4
        tsize = (off + 3) // 4 * 4
        vsize = 4 + 2 * nslots
        self._align(4, bias=vsize)          # so that the table itself is 4-aligned
        vpos = len(self.b)
        self.b += struct.pack("<HH", vsize, tsize)
        for s in range(nslots):
            self.b += struct.pack("<H", layout.get(s, 0))
        tpos = len(self.b)
        self.b += struct.pack("<i", tpos - vpos) + bytes(tsize - 4)
        children = []
        for slot, kind, val in order:
            fpos = tpos + layout[slot]
            if kind in _SCALAR:
                struct.pack_into(_SCALAR[kind], self.b, fpos, int(val))
            else:
                children.append((fpos, kind, val))
        for fpos, kind, val in children:
            self._patch_offset(fpos, self._child(kind, val))
        return tpos

    def _child(self, kind, val):
        if kind == "str":
            return self.string(val)
        if kind in _VEC_DTYPE:
            arr = np.ascontiguousarray(val, dtype=_VEC_DTYPE[kind]).ravel()
            self._align(4)
            if arr.itemsize == 8:
                self._align(8, bias=4)      # elements 8-aligned, the count sits just before them
            pos = len(self.b)
            self.b += struct.pack("<I", arr.size) + arr.astype(arr.dtype.newbyteorder("<")).tobytes()
            return pos
        if kind in ("vstr", "vtable"):
            self._align(4)
            pos = len(self.b)
            self.b += struct.pack("<I", len(val)) + bytes(4 * len(val))
            for i, v in enumerate(val):
                target = self.string(v) if kind == "vstr" else self.table(v)
                self._patch_offset(pos + 4 + 4 * i, target)
            return pos
        if kind == "table":
            return self.table(val)
        raise ValueError(kind)

    def string(self, s):
        raw = s.encode("utf-8")
        self._align(4)
        pos = len(self.b)
        self.b += struct.pack("<I", len(raw)) + raw + b"\0"
        return pos


def _tensor_fields(t: TensorSpec):
    is_bit = t.kind == "bit"
    return [(0, "i8", 1 if is_bit else 0),
            (1, "vu64", t.data if is_bit else None),
            (2, "vf32", None if is_bit else t.data),
            (3, "vu32", list(t.shape)),
            (4, "str", t.name),
            (5, "bool", 1 if t.align_hwc_to_128 else None)]


def _layer_fields(l: LayerSpec):
    slot, schema = PARAM_TABLES[l.type]
    params = []
    for fname, fid, kind in schema:
        v = l.fields.get(fname)
        if v is None or (kind == "str" and v == ""):
            continue
        params.append((fid, kind, v))
    return [(0, "i8", LAYER_TYPES.index(l.type)), (slot, "table", params),
            (_LAYER_NAME_SLOT, "str", l.name)]


def write_dab(spec: ModelSpec) -> bytes:
    """Serialise a ModelSpec as `.dab` bytes."""
    w = _Writer()
    w.b += bytes(4)
    _, h, wd, c = spec.input_shape
    root = w.table([
        (0, "vtable", [_layer_fields(l) for l in spec.layers]),
        (1, "vtable", [_tensor_fields(t) for t in spec.tensors]),
        (2, "vtable", [[(0, "vu32", [1, h, wd, c]), (1, "str", spec.input_name)]]),
        (3, "u32", spec.version),
    ])
    struct.pack_into("<I", w.b, 0, root)
    return bytes(w.b)


# ------------------------------------------------------------------------------------ reader
class _Table:
    def __init__(self, buf, pos):
        self.buf, self.pos = buf, pos
        if pos < 0 or pos + 4 > len(buf):
            raise ValueError("dab: table out of bounds")
        self.vt = pos - struct.unpack_from("<i", buf, pos)[0]
        if self.vt < 0 or self.vt + 4 > len(buf):
            raise ValueError("dab: vtable out of bounds")
        self.vsize = struct.unpack_from("<H", buf, self.vt)[0]

    def _field(self, slot):
        o = 4 + 2 * slot
        if o + 2 > self.vsize:
            return None
        rel = struct.unpack_from("<H", self.buf, self.vt + o)[0]
        return self.pos + rel if rel else None

    def scalar(self, slot, fmt, default=0):
        p = self._field(slot)
        return default if p is None else struct.unpack_from(fmt, self.buf, p)[0]

    def _indirect(self, slot):
        p = self._field(slot)
        if p is None:
            return None
        t = p + struct.unpack_from("<I", self.buf, p)[0]
        if t + 4 > len(self.buf):
            raise ValueError("dab: offset out of bounds")
        return t

    def string(self, slot):
        t = self._indirect(slot)
        return None if t is None else _read_string(self.buf, t)

    def vector(self, slot, dtype):
        t = self._indirect(slot)
        if t is None:
            return None
        n = struct.unpack_from("<I", self.buf, t)[0]
        return np.frombuffer(self.buf, dtype=np.dtype(dtype).newbyteorder("<"), count=n, offset=t + 4)

    def table(self, slot):
        t = self._indirect(slot)
        return None if t is None else _Table(self.buf, t)

    def vector_of(self, slot, what):
        t = self._indirect(slot)
        if t is None:
            return []
        n = struct.unpack_from("<I", self.buf, t)[0]
        out = []
        for i in range(n):
            p = t + 4 + 4 * i
            tgt = p + struct.unpack_from("<I", self.buf, p)[0]
            out.append(_read_string(self.buf, tgt) if what == "str" else _Table(self.buf, tgt))
        return out


def _read_string(buf, t):
    n = struct.unpack_from("<I", buf, t)[0]
    return bytes(buf[t + 4:t + 4 + n]).decode("utf-8")


def read_dab(buf: bytes) -> ModelSpec:
    """Parse `.dab` bytes into a ModelSpec (inverse of write_dab)."""
    if len(buf) < 8:
        raise ValueError("dab: buffer too small")
    root = _Table(buf, struct.unpack_from("<I", buf, 0)[0])
    version = root.scalar(3, "<I")
    inputs = root.vector_of(2, "table")
    if not inputs:
        raise ValueError("dab: model has no input")
    shape = tuple(int(v) for v in inputs[0].vector(0, np.uint32))
    tensors = []
    for t in root.vector_of(1, "table"):
        is_bit = t.scalar(0, "<b") == 1
        data = t.vector(1, np.uint64) if is_bit else t.vector(2, np.float32)
        tensors.append(TensorSpec(t.string(4), "bit" if is_bit else "f32",
                                  tuple(int(v) for v in t.vector(3, np.uint32)),
                                  np.array(data), bool(t.scalar(5, "<B"))))
    layers = []
    for l in root.vector_of(0, "table"):
        ltype = LAYER_TYPES[l.scalar(0, "<b")]
        slot, schema = PARAM_TABLES[ltype]
        p = l.table(slot)
        fields = {}
        for fname, fid, kind in schema:
            if kind == "str":
                v = p.string(fid)
            elif kind == "vi32":
                v = p.vector(fid, np.int32)
                v = None if v is None else [int(x) for x in v]
            elif kind == "vstr":
                v = p.vector_of(fid, "str")
            else:
                v = p.scalar(fid, "<i")
            if v is not None:
                fields[fname] = v
        layers.append(LayerSpec(ltype, l.string(_LAYER_NAME_SLOT) or "", fields))
    return ModelSpec(inputs[0].string(1), shape, tensors, layers, version)
