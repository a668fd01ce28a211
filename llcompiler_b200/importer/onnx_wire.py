"""Reader (and a small writer) for the ONNX protobuf wire format, without the `onnx` package.

Only the fields the importer needs are decoded (field numbers from onnx/onnx.proto, IR version 3+):
ModelProto.graph = 7; GraphProto.node = 1, initializer = 5, input = 11, output = 12; NodeProto.input = 1, output = 2,
name = 3, op_type = 4, attribute = 5; AttributeProto.name = 1, f = 2, i = 3, s = 4, t = 5, floats = 7, ints = 8;
TensorProto.dims = 1, data_type = 2, float_data = 4, int64_data = 7, name = 8, raw_data = 9; ValueInfoProto.name = 1,
type = 2; TypeProto.tensor_type = 1; TypeProto.Tensor.elem_type = 1, shape = 2; TensorShapeProto.dim = 1;
Dimension.dim_value = 1, dim_param = 2.  The writer exists so that tests (and users without `onnx`) can build models.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Tuple, Union

import numpy as np

FLOAT, INT64 = 1, 7
_NP = {FLOAT: np.float32, INT64: np.int64, 6: np.int32, 11: np.float64}


# ---- wire primitives ------------------------------------------------------------------------
def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    out = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if not b & 0x80:
            return out, pos
        shift += 7


def _fields(buf: bytes):
    """Yields (field number, wire type, value) for one message; length-delimited values are bytes."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        yield num, wt, val


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def _packed_ints(val, wt) -> List[int]:
    if wt == 0:
        return [_signed(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed(v))
    return out


# ---- decoded model --------------------------------------------------------------------------
@dataclass
class OnnxNode:
    op_type: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, object] = field(default_factory=dict)
    name: str = ""


@dataclass
class OnnxValue:
    name: str
    elem_type: int
    dims: List[Union[int, str]]


@dataclass
class OnnxGraph:
    nodes: List[OnnxNode]
    initializers: Dict[str, np.ndarray]
    inputs: List[OnnxValue]
    outputs: List[OnnxValue]


def _tensor(buf: bytes) -> Tuple[str, np.ndarray]:
    dims, dtype, name, raw, floats, ints = [], FLOAT, "", None, [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_ints(val, wt)
        elif num == 2:
            dtype = val
        elif num == 4:
            floats += list(struct.unpack(f"<{len(val) // 4}f", val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 7:
            ints += _packed_ints(val, wt)
        elif num == 8:
            name = val.decode()
        elif num == 9:
            raw = val
    if dtype not in _NP:
        raise NotImplementedError(f"ONNX tensor element type {dtype}")
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(_NP[dtype]).newbyteorder("<")).astype(_NP[dtype])
    else:
        arr = np.array(floats if dtype == FLOAT else ints, dtype=_NP[dtype])
    return name, arr.reshape(dims)


def _attribute(buf: bytes) -> Tuple[str, object]:
    name, value, ints, floats = "", None, [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            value = struct.unpack("<f", val)[0]
        elif num == 3:
            value = _signed(val)
        elif num == 4:
            value = val.decode(errors="replace")
        elif num == 5:
            value = _tensor(val)[1]
        elif num == 7:
            floats += list(struct.unpack(f"<{len(val) // 4}f", val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 8:
            ints += _packed_ints(val, wt)
    if ints:
        value = ints
    elif floats:
        value = floats
    return name, value


def _value_info(buf: bytes) -> OnnxValue:
    name, elem, dims = "", FLOAT, []
    for num, _, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            for n2, _, v2 in _fields(val):
                if n2 != 1:
                    continue
                for n3, _, v3 in _fields(v2):
                    if n3 == 1:
                        elem = v3
                    elif n3 == 2:
                        for n4, _, v4 in _fields(v3):
                            if n4 != 1:
                                continue
                            d: Union[int, str] = "?"
                            for n5, _, v5 in _fields(v4):
                                d = _signed(v5) if n5 == 1 else (v5.decode() if n5 == 2 else d)
                            dims.append(d)
    return OnnxValue(name, elem, dims)


def parse_model(data: bytes) -> OnnxGraph:
    """Decodes a serialized ModelProto (the bytes of a .onnx file)."""
    graph = None
    for num, _, val in _fields(data):
        if num == 7:
            graph = val
    if graph is None:
        raise ValueError("not an ONNX model: no graph")
    nodes, inits, inputs, outputs = [], {}, [], []
    for num, _, val in _fields(graph):
        if num == 1:
            n = OnnxNode("", [], [])
            for n2, _, v2 in _fields(val):
                if n2 == 1:
                    n.inputs.append(v2.decode())
                elif n2 == 2:
                    n.outputs.append(v2.decode())
                elif n2 == 3:
                    n.name = v2.decode()
                elif n2 == 4:
                    n.op_type = v2.decode()
                elif n2 == 5:
                    k, v = _attribute(v2)
                    n.attrs[k] = v
            nodes.append(n)
        elif num == 5:
            k, arr = _tensor(val)
            inits[k] = arr
        elif num == 11:
            inputs.append(_value_info(val))
        elif num == 12:
            outputs.append(_value_info(val))
    return OnnxGraph(nodes, inits, [i for i in inputs if i.name not in inits], outputs)


# ---- writer ---------------------------------------------------------------------------------
def _enc_varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _ld(num: int, payload: bytes) -> bytes:
    return _enc_varint(num << 3 | 2) + _enc_varint(len(payload)) + payload


def _vi(num: int, v: int) -> bytes:
    return _enc_varint(num << 3) + _enc_varint(v)


def _enc_tensor(name: str, arr: np.ndarray) -> bytes:
    dtype = FLOAT if arr.dtype == np.float32 else INT64
    arr = np.ascontiguousarray(arr.astype(np.float32 if dtype == FLOAT else np.int64))
    out = b"".join(_vi(1, d) for d in arr.shape) + _vi(2, dtype) + _ld(8, name.encode()) + _ld(9, arr.tobytes())
    return out


def _enc_value(name: str, dims, elem: int = FLOAT) -> bytes:
    shape = b"".join(_ld(1, _vi(1, d) if isinstance(d, int) else _ld(2, str(d).encode())) for d in dims)
    return _ld(1, name.encode()) + _ld(2, _ld(1, _vi(1, elem) + _ld(2, shape)))


def _enc_attr(name: str, v) -> bytes:
    out = _ld(1, name.encode())
    if isinstance(v, float):
        return out + _enc_varint(2 << 3 | 5) + struct.pack("<f", v) + _vi(20, 1)
    if isinstance(v, int):
        return out + _vi(3, v) + _vi(20, 2)
    if isinstance(v, str):
        return out + _ld(4, v.encode()) + _vi(20, 3)
    if isinstance(v, np.ndarray):
        return out + _ld(5, _enc_tensor("", v)) + _vi(20, 4)
    return out + b"".join(_vi(8, int(i)) for i in v) + _vi(20, 7)


def build_model(nodes, initializers: Dict[str, np.ndarray], inputs, outputs) -> bytes:
    """nodes: (op_type, [inputs], [outputs], {attrs}); inputs / outputs: (name, [dims]) or (name, [dims], element type code).
    Returns ModelProto bytes."""
    g = b""
    for op, ins, outs, attrs in nodes:
        n = b"".join(_ld(1, i.encode()) for i in ins) + b"".join(_ld(2, o.encode()) for o in outs) + _ld(4, op.encode())
        n += b"".join(_ld(5, _enc_attr(k, v)) for k, v in (attrs or {}).items())
        g += _ld(1, n)
    g += _ld(2, b"graph")
    g += b"".join(_ld(5, _enc_tensor(k, v)) for k, v in initializers.items())
    g += b"".join(_ld(11, _enc_value(*v)) for v in inputs)
    g += b"".join(_ld(12, _enc_value(*v)) for v in outputs)
    opset = _ld(1, b"") + _vi(2, 17)
    return _vi(1, 8) + _ld(8, opset) + _ld(7, g)
