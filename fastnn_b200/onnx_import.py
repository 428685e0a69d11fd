"""ONNX file -> the arguments of `AotExecutor` (node dicts, parameter arrays, names, shapes).

fastnn's Python front end reads a model with the `onnx` package, renames operators through its
ONNX_TO_IR_OP table, flattens attributes into the node dict and hands `nodes, params, input_names,
output_names, input_shapes` to the Rust `AotExecutor` (fastnn/io/onnx.py:22-66, 182-238, 276-466;
src/python/nn.rs:1221-1364).  This module produces the same five arguments for the operators on the
CUDA path.  The `onnx` package is not a dependency: an ONNX file is a protobuf message, and the
handful of fields needed (onnx.proto: ModelProto.graph, GraphProto.{node, initializer, input,
output}, NodeProto, AttributeProto, TensorProto, ValueInfoProto) are read straight from the wire
format.

Two import-time rewrites make exporter output land on the quantized MatMul, both on constants
only:
  * `Gemm` with transB=1 (what PyTorch emits for nn.Linear) whose B is an initializer used by that
    node alone: the initializer is transposed here, so the graph holds the `[K, N]` constant the
    quantization pass selects (src/compiler/passes/quantization.rs:144-156); alpha and beta other
    than 1 are folded into B and C the same way.  With a non-constant B the node is passed on as
    it is and `AotExecutor` refuses it.
  * `Sigmoid(x)` followed by `Mul(x, sigmoid)` (PyTorch's export of SiLU) becomes one `Silu` node.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from .backend import BackendError

# onnx.proto TensorProto.DataType -> numpy
_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64,
           9: np.bool_, 10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}

# Operators the CUDA path serves, ONNX name -> the op_type `AotExecutor` takes (the reference's
# table keeps these names unchanged, fastnn/io/onnx.py:22-66; Dropout becomes Identity there).
ONNX_TO_IR_OP = {
    "MatMul": "MatMul", "Gemm": "Gemm", "Add": "Add", "Relu": "Relu", "Gelu": "Gelu",
    "Swish": "Swish", "Softmax": "Softmax", "LayerNormalization": "LayerNormalization",
    "RMSNormalization": "RMSNorm", "SimplifiedLayerNormalization": "SimplifiedLayerNormalization",
    "Sigmoid": "Sigmoid", "Mul": "Mul", "Identity": "Identity", "Dropout": "Identity",
}


# ---- protobuf wire format ---------------------------------------------------------------------

def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = shift = 0
    while True:
        if pos >= len(buf):
            raise BackendError("Compilation", "onnx: truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise BackendError("Compilation", "onnx: varint longer than 10 bytes")


def _fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
    """(field number, wire type, value) of one message; value is an int (varint, fixed) or bytes."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            if pos + 8 > end:
                raise BackendError("Compilation", "onnx: truncated 64-bit field")
            val, pos = struct.unpack_from("<Q", buf, pos)[0], pos + 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            if pos + n > end:
                raise BackendError("Compilation", "onnx: length-delimited field runs past its message")
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            if pos + 4 > end:
                raise BackendError("Compilation", "onnx: truncated 32-bit field")
            val, pos = struct.unpack_from("<I", buf, pos)[0], pos + 4
        else:
            raise BackendError("Compilation", f"onnx: wire type {wt} is not used by onnx.proto")
        yield num, wt, val


def _signed64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(wt: int, val) -> List[int]:
    if wt == 0:
        return [_signed64(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed64(v))
    return out


def _packed_floats(wt: int, val) -> List[float]:
    if wt == 5:
        return [struct.unpack("<f", struct.pack("<I", val))[0]]
    return list(np.frombuffer(val, dtype="<f4"))


# ---- messages -----------------------------------------------------------------------------------

@dataclass
class OnnxNode:
    op_type: str = ""
    name: str = ""
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    attrs: Dict[str, object] = field(default_factory=dict)


@dataclass
class OnnxModel:
    nodes: List[OnnxNode]
    initializers: Dict[str, np.ndarray]
    inputs: List[Tuple[str, List[object]]]    # (name, dims: int or symbol string) without initializers
    outputs: List[str]


def _tensor(buf: bytes) -> Tuple[str, np.ndarray]:
    dims: List[int] = []
    dtype, name, raw = 1, "", None
    floats: List[float] = []
    ints: List[int] = []
    doubles: List[float] = []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_varints(wt, val)
        elif num == 2:
            dtype = int(val)
        elif num == 4:
            floats += _packed_floats(wt, val)
        elif num in (5, 7):
            ints += _packed_varints(wt, val)
        elif num == 8:
            name = val.decode()
        elif num == 9:
            raw = val
        elif num == 10:
            doubles += list(np.frombuffer(val, dtype="<f8")) if wt == 2 else [struct.unpack("<d", struct.pack("<Q", val))[0]]
        elif num == 13 and val:
            raise BackendError("UnsupportedOp", f"onnx: initializer '{name}' keeps its data in an external file")
    if dtype not in _DTYPES:
        raise BackendError("UnsupportedOp", f"onnx: tensor '{name}' has data type {dtype}")
    np_dtype = _DTYPES[dtype]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(np_dtype).newbyteorder("<")).astype(np_dtype)
    elif floats:
        arr = np.asarray(floats, dtype=np_dtype)
    elif doubles:
        arr = np.asarray(doubles, dtype=np_dtype)
    else:
        arr = np.asarray(ints, dtype=np_dtype)
    count = int(np.prod(dims)) if dims else arr.size
    if arr.size != count:
        raise BackendError("Compilation", f"onnx: tensor '{name}' holds {arr.size} elements for dims {dims}")
    return name, arr.reshape(dims) if dims else arr.reshape(())


def _attribute(buf: bytes) -> Tuple[str, object]:
    name, value = "", None
    floats: List[float] = []
    ints: List[int] = []
    strings: List[str] = []
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            value = struct.unpack("<f", struct.pack("<I", val))[0]
        elif num == 3:
            value = _signed64(val)
        elif num == 4:
            value = val.decode(errors="replace")
        elif num == 5:
            value = _tensor(val)[1]
        elif num == 7:
            floats += _packed_floats(wt, val)
        elif num == 8:
            ints += _packed_varints(wt, val)
        elif num == 9:
            strings.append(val.decode(errors="replace"))
    if value is None:
        value = floats or ints or strings or None
    return name, value


def _node(buf: bytes) -> OnnxNode:
    n = OnnxNode()
    for num, wt, val in _fields(buf):
        if num == 1:
            n.inputs.append(val.decode())
        elif num == 2:
            n.outputs.append(val.decode())
        elif num == 3:
            n.name = val.decode()
        elif num == 4:
            n.op_type = val.decode()
        elif num == 5:
            k, v = _attribute(val)
            if v is not None:
                n.attrs[k] = v
    return n


def _value_info(buf: bytes) -> Tuple[str, List[object]]:
    name, dims = "", []
    for num, _, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:                                   # TypeProto
            for n2, _, v2 in _fields(val):
                if n2 != 1:                              # tensor_type
                    continue
                for n3, _, v3 in _fields(v2):
                    if n3 != 2:                          # shape
                        continue
                    for n4, _, v4 in _fields(v3):
                        if n4 != 1:                      # dim
                            continue
                        d: object = "?"
                        for n5, _, v5 in _fields(v4):
                            if n5 == 1:
                                d = _signed64(v5)
                            elif n5 == 2:
                                d = v5.decode()
                        dims.append(d)
    return name, dims


def read_onnx(source) -> OnnxModel:
    """Parse an ONNX file (a path, or the bytes of one)."""
    data = source if isinstance(source, (bytes, bytearray)) else open(source, "rb").read()
    graph = None
    for num, wt, val in _fields(bytes(data)):
        if num == 7 and wt == 2:
            graph = val
    if graph is None:
        raise BackendError("Compilation", "onnx: the file holds no graph")
    nodes, inits, inputs, outputs = [], {}, [], []
    for num, wt, val in _fields(graph):
        if wt != 2:
            continue
        if num == 1:
            nodes.append(_node(val))
        elif num == 5:
            name, arr = _tensor(val)
            inits[name] = arr
        elif num == 11:
            inputs.append(_value_info(val))
        elif num == 12:
            outputs.append(_value_info(val)[0])
    inputs = [(n, d) for n, d in inputs if n not in inits]   # old exporters list initializers as inputs
    return OnnxModel(nodes, inits, inputs, outputs)


# ---- to AotExecutor arguments ---------------------------------------------------------------------

def _uses(nodes: Sequence[OnnxNode], outputs: Sequence[str]) -> Dict[str, int]:
    count: Dict[str, int] = {}
    for n in nodes:
        for i in n.inputs:
            count[i] = count.get(i, 0) + 1
    for o in outputs:
        count[o] = count.get(o, 0) + 1
    return count


def to_aot_arguments(model: OnnxModel, input_shapes: Optional[Dict[str, Sequence[int]]] = None):
    """`(nodes, params, input_names, output_names, input_shapes)` for `AotExecutor`.  A symbolic or
    unknown dimension becomes a negative number (-1, -2, ... per distinct symbol), which
    `AotExecutor` reads as a runtime dimension; `input_shapes` overrides what the file declares."""
    params = {k: v for k, v in model.initializers.items()}
    nodes = [OnnxNode(n.op_type, n.name, list(n.inputs), list(n.outputs), dict(n.attrs)) for n in model.nodes]
    uses = _uses(nodes, model.outputs)

    # Constant nodes are parameters too (src/onnx/converter.rs:114-133)
    kept = []
    for n in nodes:
        if n.op_type == "Constant" and isinstance(n.attrs.get("value"), np.ndarray):
            params[n.outputs[0]] = n.attrs["value"]
        else:
            kept.append(n)
    nodes = kept

    # Gemm: fold transB / alpha / beta into constant operands
    for n in nodes:
        if n.op_type != "Gemm":
            continue
        if int(n.attrs.get("transA", 0)):
            raise BackendError("UnsupportedOp", f"onnx: Gemm '{n.name}' with transA=1 is not on the CUDA path")
        alpha, beta = float(n.attrs.get("alpha", 1.0)), float(n.attrs.get("beta", 1.0))
        b = n.inputs[1]
        if b in params and uses.get(b, 0) == 1 and params[b].ndim == 2:
            w = params[b].astype(np.float32)
            if int(n.attrs.get("transB", 0)):
                w = np.ascontiguousarray(w.T)
                n.attrs["transB"] = 0
            if alpha != 1.0:
                w = (w * np.float32(alpha)).astype(np.float32)
                n.attrs["alpha"] = 1.0
            params[b] = w
        elif alpha != 1.0:
            raise BackendError("UnsupportedOp", f"onnx: Gemm '{n.name}' scales a non-constant product (alpha={alpha})")
        if len(n.inputs) > 2 and beta != 1.0:
            c = n.inputs[2]
            if c in params and uses.get(c, 0) == 1:
                params[c] = (params[c].astype(np.float32) * np.float32(beta)).astype(np.float32)
                n.attrs["beta"] = 1.0
            else:
                raise BackendError("UnsupportedOp", f"onnx: Gemm '{n.name}' scales a non-constant C (beta={beta})")

    # Sigmoid(x) * x -> Silu(x); Identity / Dropout -> renamed away
    by_output = {o: n for n in nodes for o in n.outputs}
    drop, rename = set(), {}
    for n in nodes:
        if n.op_type == "Mul" and len(n.inputs) == 2:
            for a, s in ((n.inputs[0], n.inputs[1]), (n.inputs[1], n.inputs[0])):
                sg = by_output.get(s)
                if sg is not None and sg.op_type == "Sigmoid" and sg.inputs == [a] and uses.get(s, 0) == 1:
                    n.op_type, n.inputs = "Silu", [a]
                    drop.add(id(sg))
                    break
        elif n.op_type in ("Identity", "Dropout"):
            rename[n.outputs[0]] = n.inputs[0]
            drop.add(id(n))

    def resolve(name: str) -> str:
        while name in rename:
            name = rename[name]
        return name

    out_nodes: List[Dict[str, str]] = []
    for n in nodes:
        if id(n) in drop:
            continue
        op = n.op_type if n.op_type == "Silu" else ONNX_TO_IR_OP.get(n.op_type)
        if op is None:
            raise BackendError("UnsupportedOp", f"onnx: operator '{n.op_type}' ({n.name}) is not on the CUDA path")
        d = {"name": n.name, "op_type": op,
             "inputs": "[" + ", ".join(resolve(i) for i in n.inputs if i) + "]",
             "outputs": "[" + ", ".join(n.outputs) + "]"}
        for k, v in n.attrs.items():                      # flattened like the reference's _extract_attrs
            if isinstance(v, (int, float, str)):
                d[k] = str(v)
            elif isinstance(v, list):
                d[k] = str(v)
        out_nodes.append(d)

    symbols: Dict[str, int] = {}
    shapes: Dict[str, List[int]] = {}
    for name, dims in model.inputs:
        if input_shapes and name in input_shapes:
            shapes[name] = [int(x) for x in input_shapes[name]]
            continue
        out = []
        for dd in dims:
            if isinstance(dd, int) and dd > 0:
                out.append(dd)
            else:
                key = dd if isinstance(dd, str) and dd != "?" else f"?{len(symbols)}"
                out.append(-symbols.setdefault(key, len(symbols) + 1))
        shapes[name] = out
    used = set()
    for d in out_nodes:
        used.update(x.strip() for x in d["inputs"].strip("[]").split(",") if x.strip())
    params = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in params.items() if k in used}
    return (out_nodes, params, [n for n, _ in model.inputs], [resolve(o) for o in model.outputs], shapes)
