"""Minimal protobuf wire-format reader for ONNX ``TensorProto`` / ``ModelProto`` files.

The reference stores its single-op golden vectors as serialized ONNX TensorProto
messages (``input_N.pb`` / ``output_N.pb`` next to a ``model.onnx``), compared by
``tests/single_op.rs:16-47`` of the reference.  Neither ``onnx`` nor ``protoc`` is
available to this project, so the handful of fields that matter are decoded by hand:

TensorProto: 1=dims (varint, packed or not), 2=data_type, 4=float_data, 7=int64_data,
             8=name, 9=raw_data.
data_type:   1=f32, 3=i8, 6=i32, 7=i64, 16=bf16 (stored as uint16 bit patterns).
"""
import struct

import numpy as np


def _varint(buf, pos):
    val = 0
    shift = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7


def fields(buf):
    """Yield (field_number, wire_type, value) for one message."""
    pos = 0
    n = len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        fno, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 1:
            v = buf[pos:pos + 8]
            pos += 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            v = buf[pos:pos + ln]
            pos += ln
        elif wt == 5:
            v = buf[pos:pos + 4]
            pos += 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        yield fno, wt, v


_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 6: np.int32, 7: np.int64, 11: np.float64, 16: np.uint16}


def parse_tensor(buf):
    """Return (name, data_type, ndarray).  bf16 comes back as uint16 bit patterns."""
    dims, dtype, raw, name = [], None, None, ""
    floats, int64s, int32s = [], [], []
    for fno, wt, v in fields(buf):
        if fno == 1:
            if wt == 0:
                dims.append(v)
            else:
                p = 0
                while p < len(v):
                    d, p = _varint(v, p)
                    dims.append(d)
        elif fno == 2:
            dtype = v
        elif fno == 4:
            if wt == 2:
                floats.extend(struct.unpack(f"<{len(v) // 4}f", v))
            else:
                floats.append(struct.unpack("<f", v)[0])
        elif fno == 5:
            if wt == 2:
                p = 0
                while p < len(v):
                    d, p = _varint(v, p)
                    int32s.append(d)
            else:
                int32s.append(v)
        elif fno == 7:
            if wt == 2:
                p = 0
                while p < len(v):
                    d, p = _varint(v, p)
                    int64s.append(d - (1 << 64) if d >> 63 else d)
            else:
                int64s.append(v - (1 << 64) if v >> 63 else v)
        elif fno == 8:
            name = bytes(v).decode()
        elif fno == 9:
            raw = bytes(v)
    np_dt = _DTYPES[dtype]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np_dt).copy()
    elif floats:
        arr = np.asarray(floats, dtype=np_dt)
    elif int64s:
        arr = np.asarray(int64s, dtype=np_dt)
    elif int32s:
        arr = np.asarray(int32s).astype(np_dt)
    else:
        arr = np.zeros(0, dtype=np_dt)
    return name, dtype, arr.reshape(dims)


def load_tensor(path):
    with open(path, "rb") as f:
        return parse_tensor(f.read())


def model_nodes(path):
    """Return a list of (op_type, {attr_name: value}) plus graph initializers of a model.onnx.

    ModelProto.graph = 7; GraphProto.node = 1, .initializer = 5;
    NodeProto.op_type = 4, .attribute = 5; AttributeProto name=1, f=2, i=3.
    """
    with open(path, "rb") as f:
        buf = f.read()
    nodes, inits = [], []
    for fno, _, v in fields(buf):
        if fno != 7:
            continue
        for gno, _, gv in fields(v):
            if gno == 1:
                op, attrs = None, {}
                for nno, _, nv in fields(gv):
                    if nno == 4:
                        op = bytes(nv).decode()
                    elif nno == 5:
                        an, av = None, None
                        for ano, awt, aval in fields(nv):
                            if ano == 1:
                                an = bytes(aval).decode()
                            elif ano == 2:
                                av = struct.unpack("<f", aval)[0]
                            elif ano == 3:
                                av = aval - (1 << 64) if aval >> 63 else aval
                        attrs[an] = av
                nodes.append((op, attrs))
            elif gno == 5:
                inits.append(parse_tensor(gv))
    return nodes, inits
