"""Writes small ONNX files for the tests: a protobuf encoder for the handful of onnx.proto messages
an importer has to read (field numbers from onnx.proto).  Test infrastructure only."""
import struct

import numpy as np


def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _key(num, wt):
    return _varint((num << 3) | wt)


def _ld(num, payload: bytes) -> bytes:
    return _key(num, 2) + _varint(len(payload)) + payload


def _vi(num, v: int) -> bytes:
    return _key(num, 0) + _varint(v)


def tensor(name, arr, raw=True) -> bytes:
    arr = np.asarray(arr)
    dt = {np.dtype(np.float32): 1, np.dtype(np.int64): 7, np.dtype(np.float64): 11}[arr.dtype]
    out = b"".join(_vi(1, d) for d in arr.shape) + _vi(2, dt)
    if raw:
        out += _ld(9, arr.astype(arr.dtype.newbyteorder("<")).tobytes())
    elif dt == 1:
        out += _ld(4, arr.astype("<f4").tobytes())          # packed float_data
    elif dt == 7:
        out += _ld(7, b"".join(_varint(int(x)) for x in arr.ravel()))
    else:
        out += _ld(10, arr.astype("<f8").tobytes())
    return out + _ld(8, name.encode())


def attribute(name, value) -> bytes:
    out = _ld(1, name.encode())
    if isinstance(value, float):
        return out + _key(2, 5) + struct.pack("<f", value) + _vi(20, 1)
    if isinstance(value, int):
        return out + _vi(3, value) + _vi(20, 2)
    if isinstance(value, str):
        return out + _ld(4, value.encode()) + _vi(20, 3)
    if isinstance(value, np.ndarray):
        return out + _ld(5, tensor("", value)) + _vi(20, 4)
    if isinstance(value, (list, tuple)) and all(isinstance(x, int) for x in value):
        return out + b"".join(_vi(8, x) for x in value) + _vi(20, 7)
    raise TypeError(value)


def node(op_type, inputs, outputs, name="", **attrs) -> bytes:
    out = b"".join(_ld(1, i.encode()) for i in inputs) + b"".join(_ld(2, o.encode()) for o in outputs)
    out += _ld(3, name.encode()) + _ld(4, op_type.encode())
    return out + b"".join(_ld(5, attribute(k, v)) for k, v in attrs.items())


def value_info(name, dims) -> bytes:
    shape = b""
    for d in dims:
        dim = _ld(2, d.encode()) if isinstance(d, str) else _vi(1, d)
        shape += _ld(1, dim)
    tensor_type = _vi(1, 1) + _ld(2, shape)
    return _ld(1, name.encode()) + _ld(2, _ld(1, tensor_type))


def model(nodes, initializers, inputs, outputs, initializers_as_inputs=False) -> bytes:
    """nodes: encoded NodeProtos; initializers: {name: array} or encoded tensors; inputs: [(name, dims)]."""
    g = b"".join(_ld(1, n) for n in nodes) + _ld(2, b"g")
    enc = [tensor(k, v) if not isinstance(v, bytes) else v for k, v in initializers.items()]
    g += b"".join(_ld(5, t) for t in enc)
    ins = list(inputs)
    if initializers_as_inputs:
        ins += [(k, list(np.asarray(v).shape)) for k, v in initializers.items() if not isinstance(v, bytes)]
    g += b"".join(_ld(11, value_info(n, d)) for n, d in ins)
    g += b"".join(_ld(12, value_info(n, [])) for n in outputs)
    opset = _ld(1, b"") + _vi(2, 17)
    return _vi(1, 8) + _ld(2, b"tests") + _ld(7, g) + _ld(8, opset)
