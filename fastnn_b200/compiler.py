"""Host-side graph pipeline in front of ``CudaBackend``: the slice of fastnn's IR, builder,
compiler passes and executor that the quantized-weight MatMul path runs through.

It mirrors, by name and behaviour, the reference call stack
``GraphBuilder::compile_and_execute_with_quantize`` (src/ir/builder.rs:2383-2424) ->
``GraphExecutor::compile_with_weight_dtype`` (src/backend/executor.rs:205-321: shape inference,
fusion, weight quantization, memory planning, ``backend.compile``) ->
``GraphExecutor::execute`` (src/backend/executor.rs:599-858), and the Python entry
``AotExecutor`` (src/python/nn.rs:1219-1431).  Only the opcodes on the path exist here:
Input, Constant, MatMul, Add/Sub/Mul, Relu/Gelu/Silu, RMSNorm, LayerNorm, Softmax.

The heavy lifting is not here: quantization calls the library's host pass
(``fnn_quantize_weights``) and every plan instruction runs as a CUDA kernel.
"""
from __future__ import annotations

import ctypes
import enum
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from . import _lib as L
from .backend import (BackendError, BufferSlice, CallKernel, CudaBackend, DimExpr, ExecutablePlan,
                      Fill, MemCopy, QuantizedWeightMeta, ShapeEnv, SYMBOL_DIM_MAX, WriteConst)

# ------------------------------------------------------------------------------ IR


class Opcode(enum.Enum):
    Input = "Input"
    Constant = "Constant"
    MatMul = "MatMul"
    Add = "Add"
    Sub = "Sub"
    Mul = "Mul"
    Relu = "Relu"
    Gelu = "Gelu"
    Silu = "Silu"
    RMSNorm = "RMSNorm"
    LayerNorm = "LayerNorm"
    Softmax = "Softmax"


@dataclass
class IrDType:
    """src/ir/node.rs:535-592: packed variants carry their scales on the dtype."""
    kind: str = "F32"  # F32 | I4 | I8Scaled | F8 | F4
    scales: Optional[np.ndarray] = None
    zero_points: Optional[np.ndarray] = None
    codebooks: List[np.ndarray] = field(default_factory=list)

    @property
    def is_quantized(self) -> bool:
        return self.kind != "F32"


F32 = IrDType("F32")


@dataclass
class TensorType:
    shape: List[DimExpr]
    dtype: IrDType = field(default_factory=lambda: IrDType("F32"))

    @staticmethod
    def new(shape: Sequence[DimExpr], dtype: IrDType = F32) -> "TensorType":
        return TensorType(list(shape), dtype)

    def numel_max(self) -> int:
        n = 1
        for d in self.shape:
            n *= SYMBOL_DIM_MAX if isinstance(d, str) else int(d)
        return n

    def byte_size(self) -> int:
        """src/ir/node.rs:717-850: packed weights are rows*ceil(inner/ITEMS)+16 words."""
        if not self.dtype.is_quantized:
            return self.numel_max() * 4
        items = 4 if self.dtype.kind in ("I8Scaled", "F8") else 8
        if len(self.shape) == 2:
            k, n = int(self.shape[0]), int(self.shape[1])  # logical [K,N]; packed as [N,K]
            return (n * (-(-k // items)) + 16) * 4
        return ((-(-self.numel_max() // items)) + 16) * 4


@dataclass
class IRNode:
    id: int
    opcode: Opcode
    inputs: List[int]
    output_type: TensorType
    attrs: Dict[str, str] = field(default_factory=dict)
    value: Union[None, bytes, float] = None  # Constant payload: Data bytes or scalar
    name: str = ""


class ComputeGraph:
    def __init__(self):
        self.nodes: List[IRNode] = []
        self.inputs: List[int] = []
        self.outputs: List[int] = []
        self.next_id = 0

    def add(self, opcode, inputs, output_type, value=None, attrs=None, name="") -> IRNode:
        node = IRNode(self.next_id, opcode, list(inputs), output_type, dict(attrs or {}), value,
                      name or f"{opcode.value.lower()}_{self.next_id}")
        self.next_id += 1
        self.nodes.append(node)
        return node

    def get_node(self, node_id: int) -> Optional[IRNode]:
        for n in self.nodes:
            if n.id == node_id:
                return n
        return None

    def consumers(self, node_id: int) -> List[int]:
        return [n.id for n in self.nodes if node_id in n.inputs]

    def remove_node(self, node_id: int) -> None:
        self.nodes = [n for n in self.nodes if n.id != node_id]

    def topological(self) -> List[IRNode]:
        by_id = {n.id: n for n in self.nodes}
        seen, order = set(), []

        def visit(nid):
            if nid in seen:
                return
            seen.add(nid)
            for i in by_id[nid].inputs:
                visit(i)
            order.append(by_id[nid])

        for n in self.nodes:
            visit(n.id)
        return order

    def clone(self) -> "ComputeGraph":
        g = ComputeGraph()
        g.nodes = [IRNode(n.id, n.opcode, list(n.inputs),
                          TensorType(list(n.output_type.shape), n.output_type.dtype),
                          dict(n.attrs), n.value, n.name) for n in self.nodes]
        g.inputs, g.outputs, g.next_id = list(self.inputs), list(self.outputs), self.next_id
        return g

    def has_static_shapes(self) -> bool:
        return all(not isinstance(d, str) for n in self.nodes for d in n.output_type.shape)


class GraphTensor:
    def __init__(self, builder: "GraphBuilder", node_id: int):
        self._builder = builder
        self._id = node_id

    def node_id(self) -> int:
        return self._id

    def shape(self) -> List[DimExpr]:
        return list(self._builder.graph.get_node(self._id).output_type.shape)


class WeightDtype(enum.Enum):
    """src/backend/executor.rs `WeightDtype` (the variants on this path)."""
    F32 = "f32"
    I4 = "i4"
    I8 = "i8"
    F8x4 = "f8"
    F4x8 = "f4"
    I4Codebook = "i4cb"

    @staticmethod
    def from_quantize(quantize) -> "WeightDtype":
        """src/python/nn.rs:1320-1358."""
        if quantize is None:
            return WeightDtype.F32
        if isinstance(quantize, (int, np.integer)) and not isinstance(quantize, bool):
            if int(quantize) == 4:
                return WeightDtype.I4
            if int(quantize) == 8:
                return WeightDtype.I8
            raise ValueError(
                f"unsupported quantize value for integer: {quantize} (expected 4 or 8)")
        if isinstance(quantize, str):
            try:
                return WeightDtype(quantize)
            except ValueError:
                raise ValueError(f"unsupported quantize string: '{quantize}' "
                                 "(expected f32, i4, i8, f8, f4, i4cb, 4, or 8)")
        raise TypeError("quantize must be int (4, 8) or str (f32, i4, i8, f8, f4, i4cb) or None")


_WD_FMT = {WeightDtype.I8: L.FMT_I8, WeightDtype.I4: L.FMT_I4, WeightDtype.F8x4: L.FMT_F8,
           WeightDtype.F4x8: L.FMT_F4, WeightDtype.I4Codebook: L.FMT_I4CB}
_FMT_KIND = {L.FMT_I8: "I8Scaled", L.FMT_I4: "I4", L.FMT_F8: "F8", L.FMT_F4: "F4",
             L.FMT_I4CB: "I4"}


# ------------------------------------------------------------------------------ builder


class GraphBuilder:
    """The builder calls the path uses (src/ir/builder.rs:303-362, 2332-2424)."""

    def __init__(self):
        self.graph = ComputeGraph()
        self._inputs: List[int] = []

    def input(self, shape: Sequence[int]) -> GraphTensor:
        return self.input_with_dims(list(shape), F32)

    def input_with_dims(self, dims: Sequence[DimExpr], dtype: IrDType = F32) -> GraphTensor:
        node = self.graph.add(Opcode.Input, [], TensorType.new(dims, dtype))
        self._inputs.append(node.id)
        return GraphTensor(self, node.id)

    def constant(self, data: Union[bytes, np.ndarray], tensor_type: TensorType) -> GraphTensor:
        raw = data.tobytes() if isinstance(data, np.ndarray) else bytes(data)
        node = self.graph.add(Opcode.Constant, [], tensor_type, value=raw)
        return GraphTensor(self, node.id)

    def _binary(self, op: Opcode, a: GraphTensor, b: GraphTensor) -> GraphTensor:
        sa, sb = a.shape(), b.shape()
        out_shape = sa if len(sa) >= len(sb) else sb
        node = self.graph.add(op, [a.node_id(), b.node_id()], TensorType.new(out_shape))
        return GraphTensor(self, node.id)

    def matmul(self, a: GraphTensor, b: GraphTensor) -> GraphTensor:
        sa, sb = a.shape(), b.shape()
        if len(sa) < 2 or len(sb) != 2 or sa[-1] != sb[0]:
            raise ValueError(f"matmul shape mismatch: {sa} @ {sb}")
        node = self.graph.add(Opcode.MatMul, [a.node_id(), b.node_id()],
                              TensorType.new(list(sa[:-1]) + [sb[1]]))
        return GraphTensor(self, node.id)

    def add(self, a, b):
        return self._binary(Opcode.Add, a, b)

    def sub(self, a, b):
        return self._binary(Opcode.Sub, a, b)

    def mul(self, a, b):
        return self._binary(Opcode.Mul, a, b)

    def _unary(self, op: Opcode, x: GraphTensor) -> GraphTensor:
        node = self.graph.add(op, [x.node_id()], TensorType.new(x.shape()))
        return GraphTensor(self, node.id)

    def relu(self, x):
        return self._unary(Opcode.Relu, x)

    def gelu(self, x):
        return self._unary(Opcode.Gelu, x)

    def silu(self, x):
        return self._unary(Opcode.Silu, x)

    def rms_norm(self, x: GraphTensor, weight: GraphTensor, eps: float = 1e-5) -> GraphTensor:
        """src/ir/builder.rs:1624: RMSNorm(input, weight) with attribute `eps`."""
        node = self.graph.add(Opcode.RMSNorm, [x.node_id(), weight.node_id()], TensorType.new(x.shape()))
        node.attrs["eps"] = repr(float(eps))
        return GraphTensor(self, node.id)

    def layer_norm(self, x: GraphTensor, weight: GraphTensor, bias: GraphTensor,
                   eps: float = 1e-5) -> GraphTensor:
        """src/ir/builder.rs:1095-1117: LayerNorm(input, weight, bias), attributes `eps` and
        `normalized_ndims` (rank of the weight)."""
        node = self.graph.add(Opcode.LayerNorm, [x.node_id(), weight.node_id(), bias.node_id()],
                              TensorType.new(x.shape()))
        node.attrs["eps"] = repr(float(eps))
        node.attrs["normalized_ndims"] = str(len(weight.shape()))
        return GraphTensor(self, node.id)

    def softmax(self, x: GraphTensor, dim: int = -1) -> GraphTensor:
        """src/ir/builder.rs:816-828: Softmax with attribute `axis`."""
        node = self.graph.add(Opcode.Softmax, [x.node_id()], TensorType.new(x.shape()))
        node.attrs["axis"] = str(int(dim))
        return GraphTensor(self, node.id)

    def recorded_input_ids(self) -> List[int]:
        return list(self._inputs)

    def to_graph(self) -> ComputeGraph:
        return self.graph.clone()

    def compile_and_execute_with_quantize(self, outputs: Sequence[GraphTensor], backend,
                                          inputs: Sequence[bytes],
                                          quantize: Optional[int]) -> List[bytes]:
        """Argument order as in src/ir/builder.rs:2383: outputs, backend, inputs, quantize;
        `quantize` accepts only 4 or 8 (or None)."""
        if quantize not in (None, 4, 8):
            raise BackendError("Compilation", f"unsupported quantize bit width {quantize}")
        graph = self.to_graph()
        graph.inputs = self.recorded_input_ids()
        graph.outputs = [t.node_id() for t in outputs]
        executor = GraphExecutor(backend)
        plan, memory_plan, compiled = executor.compile_with_plan_and_quantize(graph, quantize)
        return executor.execute(compiled, plan, memory_plan, inputs)

    def compile_and_execute(self, outputs, backend, inputs) -> List[bytes]:
        return self.compile_and_execute_with_quantize(outputs, backend, inputs, None)


# ------------------------------------------------------------------------------ passes


def fuse_operators(graph: ComputeGraph) -> None:
    """MatMulAdd{Relu,Gelu,Silu} then Op{Relu,Gelu,Silu}
    (src/compiler/passes/fusion/matmul_add_relu.rs:22-142, fusion/op_relu.rs:22-99)."""
    act_names = {Opcode.Relu: "Relu", Opcode.Gelu: "Gelu", Opcode.Silu: "Silu"}
    for act_op, suffix in act_names.items():
        changed = True
        while changed:
            changed = False
            for mm in list(graph.nodes):
                if mm.opcode != Opcode.MatMul or graph.get_node(mm.id) is None:
                    continue
                cons = graph.consumers(mm.id)
                if len(cons) != 1:
                    continue
                add = graph.get_node(cons[0])
                if add is None or add.opcode != Opcode.Add:
                    continue
                add_cons = graph.consumers(add.id)
                if len(add_cons) != 1:
                    continue
                act = graph.get_node(add_cons[0])
                if act is None or act.opcode != act_op:
                    continue
                bias_in = [i for i in add.inputs if i != mm.id]
                if len(bias_in) == 1 and len(graph.get_node(bias_in[0]).output_type.shape) >= 2:
                    continue  # not a bias: rank >= 2
                fused = graph.add(Opcode.MatMul, list(mm.inputs) + bias_in, act.output_type,
                                  attrs={"fused_op": "MatMulAdd" + suffix},
                                  name="fused_" + mm.name)
                for n in graph.nodes:
                    n.inputs = [fused.id if i == act.id else i for i in n.inputs]
                graph.outputs = [fused.id if o == act.id else o for o in graph.outputs]
                for dead in (mm.id, add.id, act.id):
                    graph.remove_node(dead)
                changed = True
    for act_op, suffix in act_names.items():
        changed = True
        while changed:
            changed = False
            for op in list(graph.nodes):
                if graph.get_node(op.id) is None:
                    continue
                if op.opcode in (Opcode.Relu, Opcode.Gelu, Opcode.Silu, Opcode.Input,
                                 Opcode.Constant) or "fused_op" in op.attrs:
                    continue
                cons = graph.consumers(op.id)
                if len(cons) != 1:
                    continue
                act = graph.get_node(cons[0])
                if act is None or act.opcode != act_op:
                    continue
                op.attrs["fused_op"] = "Op" + suffix
                op.output_type = act.output_type
                for n in graph.nodes:
                    n.inputs = [op.id if i == act.id else i for i in n.inputs]
                graph.outputs = [op.id if o == act.id else o for o in graph.outputs]
                graph.remove_node(act.id)
                changed = True


def eliminate_dead_code(graph: ComputeGraph) -> None:
    live, stack = set(), list(graph.outputs)
    by_id = {n.id: n for n in graph.nodes}
    while stack:
        nid = stack.pop()
        if nid in live or nid not in by_id:
            continue
        live.add(nid)
        stack.extend(by_id[nid].inputs)
    graph.nodes = [n for n in graph.nodes if n.id in live or n.id in graph.inputs]


def quantize_weight_constant(w_kn: np.ndarray, fmt: int):
    """One weight through the library's host pass: [K,N] f32 -> (payload bytes incl. margin,
    scales, zeros, codebook).  Same transposition and quantizers as
    src/compiler/passes/quantization.rs:140-189, 361-447."""
    lib = L.load()
    w_kn = np.ascontiguousarray(w_kn, dtype=np.float32)
    k, n = w_kn.shape
    nbytes = lib.fnn_quant_packed_bytes(fmt, n, k)
    packed = np.zeros(nbytes, dtype=np.uint8)
    scales = np.zeros(lib.fnn_quant_num_scales(fmt, n, k), dtype=np.float32)
    zeros = np.zeros(n, dtype=np.float32)
    codebook = np.zeros(16, dtype=np.float32)
    rc = lib.fnn_quantize_weights(fmt, w_kn.ctypes.data, k, n, packed.ctypes.data,
                                  scales.ctypes.data, zeros.ctypes.data, codebook.ctypes.data)
    if rc != L.FNN_OK:
        raise BackendError("Compilation", f"fnn_quantize_weights failed with status {rc}")
    return packed, scales, zeros, codebook


def quantize_weights(graph: ComputeGraph, weight_dtype: WeightDtype) -> None:
    """`quantize_weights` / `quantize_weights_fp` (src/compiler/passes/quantization.rs:36-273,
    281-495): only f32 `Constant` data of rank >= 2 feeding input[1] of a MatMul is quantized;
    the node keeps its logical [K,N] shape, the payload is [N,K] packed rows + margin."""
    if weight_dtype == WeightDtype.F32:
        return
    fmt = _WD_FMT[weight_dtype]
    targets = []
    for node in graph.topological():
        if node.opcode != Opcode.MatMul or len(node.inputs) < 2:
            continue
        w = graph.get_node(node.inputs[1])
        if (w is not None and w.opcode == Opcode.Constant and isinstance(w.value, bytes)
                and not w.output_type.dtype.is_quantized and w.id not in targets):
            targets.append(w.id)
    for wid in targets:
        w = graph.get_node(wid)
        shape = w.output_type.shape
        if len(shape) < 2 or any(isinstance(d, str) for d in shape):
            continue  # 1-D constants and symbolic shapes are skipped (:134-138)
        if len(shape) != 2:
            raise BackendError("UnsupportedOp", "only 2-D MatMul weights are on the CUDA path")
        k, n = int(shape[0]), int(shape[1])
        if len(w.value) != k * n * 4 or k * n == 0:
            continue
        w_kn = np.frombuffer(w.value, dtype=np.float32).reshape(k, n)
        packed, scales, zeros, codebook = quantize_weight_constant(w_kn, fmt)
        if fmt == L.FMT_F8:
            dtype = IrDType("F8", scales, None, [])
        elif fmt == L.FMT_I4CB:
            dtype = IrDType("I4", scales, np.zeros(0, np.float32), [codebook])
            w.attrs["quant_block_size"] = "32"  # :486-490
        else:
            dtype = IrDType(_FMT_KIND[fmt], scales, zeros, [])
        w.attrs["packed_fmt"] = str(fmt)
        w.value = packed.tobytes()
        w.output_type = TensorType(list(shape), dtype)


@dataclass
class Slot:
    offset: int
    size: int


@dataclass
class MemoryPlan:
    """src/compiler/passes/memory_planning.rs:17-29."""
    slots: Dict[int, Slot]
    total_size: int
    inputs: List[Tuple[int, Slot]]
    outputs: List[Tuple[int, Slot]]


_ALIGN = 64  # memory_planning.rs:652-663


def _byte_size_with_env(t: "TensorType", env: ShapeEnv) -> int:
    """`TensorType::byte_size_with_env` (src/ir/node.rs:717-850) for f32 tensors: symbols take
    their runtime value; quantized constants have no symbolic dimension."""
    if t.dtype.is_quantized or not any(isinstance(d, str) for d in t.shape):
        return t.byte_size()
    n = 1
    for d in t.shape:
        n *= env.resolve(d)
    return n * 4


def tighten(memory_plan: "MemoryPlan", graph: "ComputeGraph", env: ShapeEnv) -> "MemoryPlan":
    """`MemoryPlan::tighten` (src/compiler/passes/memory_planning.rs:44-236): shrink every slot
    whose symbolic dimensions resolved to less than the planning maximum; offsets stay, the
    total becomes the highest end of any slot.  A batch of 3 then needs 3 rows of every
    activation slot instead of SYMBOL_DIM_MAX."""
    slots, top = {}, 0
    for nid, slot in memory_plan.slots.items():
        node = graph.get_node(nid)
        size = min(slot.size, max(_byte_size_with_env(node.output_type, env), 4)) if node is not None else slot.size
        slots[nid] = Slot(slot.offset, size)
        top = max(top, slot.offset + size)
    return MemoryPlan(slots, max(top, _ALIGN), [(i, slots[i]) for i, _ in memory_plan.inputs],
                      [(o, slots[o]) for o, _ in memory_plan.outputs])


def tighten_slices(plan: ExecutablePlan, memory_plan: "MemoryPlan", tight: "MemoryPlan",
                   env: ShapeEnv) -> ExecutablePlan:
    """`tighten_slices` (src/backend/executor.rs:1194-1284): the instructions of `plan` with
    every slice cut to its tightened slot and symbolic kernel params resolved."""
    by_offset = {}
    for nid, slot in memory_plan.slots.items():
        by_offset[(slot.offset, slot.size)] = tight.slots[nid].size

    def cut(s: BufferSlice) -> BufferSlice:
        return BufferSlice(s.offset, by_offset.get((s.offset, s.size), s.size))

    out = []
    for ins in plan.instructions:
        if isinstance(ins, CallKernel):
            params = list(ins.params)
            if ins.param_dims is not None and ins.kernel_name.startswith("matmul_"):
                params[:3] = [env.resolve(d) for d in ins.param_dims[:3]]
            out.append(CallKernel(ins.kernel_name, [cut(s) for s in ins.input_slices], cut(ins.output_slice),
                                  params, ins.node_id, ins.param_dims, ins.weight_meta,
                                  ins.secondary_output_slice))
        elif isinstance(ins, MemCopy):
            out.append(MemCopy(cut(ins.dst), cut(ins.src)))
        elif isinstance(ins, Fill):
            out.append(Fill(cut(ins.dst), ins.value))
        else:
            out.append(ins)
    return ExecutablePlan(out, tight.total_size, list(plan.levels))


def plan_memory(graph: ComputeGraph) -> MemoryPlan:
    """One slot per node at 64-byte aligned offsets; constants, inputs and outputs live for
    the whole execution (so weights persist across calls); an elementwise node reuses the slot
    of an input that dies at it (src/compiler/passes/memory_planning.rs:343-728)."""
    order = graph.topological()
    last_use: Dict[int, int] = {}
    for step, n in enumerate(order):
        for i in n.inputs:
            last_use[i] = step
        # a norm may absorb the Add in front of it at lowering time and then reads the Add's operands
        # itself: they stay alive until the norm
        if n.opcode in (Opcode.RMSNorm, Opcode.LayerNorm):
            src = graph.get_node(n.inputs[0])
            if src.opcode == Opcode.Add:
                for i in src.inputs:
                    last_use[i] = step
    persistent = set(graph.outputs) | set(graph.inputs)
    persistent |= {n.id for n in order if n.opcode == Opcode.Constant}
    slots: Dict[int, Slot] = {}
    free: List[Slot] = []
    top = 0
    elementwise = (Opcode.Add, Opcode.Sub, Opcode.Mul, Opcode.Relu, Opcode.Gelu, Opcode.Silu,
                   Opcode.RMSNorm, Opcode.LayerNorm, Opcode.Softmax)   # the row kernels work in place
    for step, n in enumerate(order):
        size = max(n.output_type.byte_size(), 4)
        padded = -(-size // _ALIGN) * _ALIGN
        placed = None
        if n.opcode in elementwise:
            for i in n.inputs:
                src = graph.get_node(i)
                if (i not in persistent and last_use.get(i) == step and i in slots
                        and slots[i].size >= size and n.inputs.count(i) == 1
                        and src.output_type.byte_size() == size):
                    placed = Slot(slots[i].offset, size)
                    break
        if placed is None:
            for f in free:
                if f.size >= padded:
                    free.remove(f)
                    placed = Slot(f.offset, size)
                    if f.size > padded:
                        free.append(Slot(f.offset + padded, f.size - padded))
                    break
        if placed is None:
            placed = Slot(top, size)
            top += padded
        slots[n.id] = placed
        for i in set(n.inputs):
            if i in persistent or last_use.get(i) != step or i not in slots:
                continue
            if slots[i].offset == placed.offset:
                continue  # reused in place
            s = slots[i]
            free.append(Slot(s.offset, -(-s.size // _ALIGN) * _ALIGN))
    return MemoryPlan(slots, max(top, _ALIGN),
                      [(i, slots[i]) for i in graph.inputs],
                      [(o, slots[o]) for o in graph.outputs])


# ------------------------------------------------------------------------------ lowering

_KERNEL_BY_KIND = {"I4": "matmul_i4", "I8Scaled": "matmul_i8", "F8": "matmul_f8", "F4": "matmul_f4"}
_EPI = {None: 0, "MatMulAdd": 0, "MatMulAddRelu": 1, "OpRelu": 1, "MatMulAddGelu": 2, "OpGelu": 2,
        "MatMulAddSilu": 3, "OpSilu": 3}
_BINARY = {Opcode.Add: "add", Opcode.Sub: "sub", Opcode.Mul: "mul"}
_UNARY = {Opcode.Relu: "relu_f32", Opcode.Gelu: "gelu_f32", Opcode.Silu: "silu_f32"}
_ACT_SUFFIX = {"OpRelu": "_relu", "OpGelu": "_gelu", "OpSilu": "_silu"}


def _slice(plan: MemoryPlan, nid: int) -> BufferSlice:
    s = plan.slots[nid]
    return BufferSlice(s.offset, s.size)


def lower_to_plan(graph: ComputeGraph, memory_plan: MemoryPlan) -> ExecutablePlan:
    """`CudaBackend::compile`.  Same instruction vocabulary as `CpuBackend::compile`
    (src/backend/cpu/mod.rs:365-640): Constant -> WriteConst / Fill, quantized MatMul ->
    `matmul_{i4,i8,f8,f4}` with params [M,K,N] + `QuantizedWeightMeta` (shape reversed to
    [N,K]).  Unlike the CPU arm it keeps the fusion: params[3] carries the activation and a
    third input slice the bias, and a bias-only `Add` of a 1-D constant that is the MatMul's
    sole consumer is folded into the same kernel."""
    order = graph.topological()
    instructions: List = []
    skip: set = set()
    # Constants first: a kernel that folds a later node (bias add) must find its operand
    # already materialised.
    for n in order:
        if n.opcode == Opcode.Constant:
            out = _slice(memory_plan, n.id)
            if isinstance(n.value, bytes):
                instructions.append(WriteConst(out, n.value))
            else:
                instructions.append(Fill(out, float(n.value)))
    # Add -> RMSNorm / LayerNorm with the Add consumed by nothing else becomes one fused row kernel, as
    # the reference's residual-add-norm fusion does (FusedResidualAddNorm, src/ir/node.rs:136-138;
    # kernels "fused_residual_add_{rms_norm,layer_norm}", src/backend/cpu/mod.rs:2424-2500)
    fused_norm: Dict[int, Tuple[int, int]] = {}
    for n in order:
        if n.opcode in (Opcode.RMSNorm, Opcode.LayerNorm):
            add = graph.get_node(n.inputs[0])
            if (add.opcode == Opcode.Add and "fused_op" not in add.attrs and add.id not in graph.outputs
                    and graph.consumers(add.id) == [n.id] and len(add.inputs) == 2):
                a0, a1 = (graph.get_node(i) for i in add.inputs)
                if list(a0.output_type.shape) == list(a1.output_type.shape) == list(n.output_type.shape):
                    fused_norm[n.id] = (add.inputs[0], add.inputs[1])
                    skip.add(add.id)
    for n in order:
        if n.id in skip:
            continue
        out = _slice(memory_plan, n.id)
        if n.opcode in (Opcode.Input, Opcode.Constant):
            continue
        if n.opcode == Opcode.MatMul:
            a, w = graph.get_node(n.inputs[0]), graph.get_node(n.inputs[1])
            wt = w.output_type
            if not wt.dtype.is_quantized:
                raise BackendError(
                    "UnsupportedOp",
                    "f32 MatMul is outside the CUDA backend's path (weights must be quantized "
                    "constants; runtime inputs and parameters stay f32 in the reference too)")
            # M is the product of the activation's leading dimensions; with a symbolic one among
            # them it is carried as the tuple of all of them and multiplied out once the ShapeEnv
            # is known (ShapeEnv.resolve), like the param_dims of the elementwise and norm arms
            a_shape = a.output_type.shape
            lead = list(a_shape[:-1])
            m_static = 1
            for d in lead:
                m_static *= SYMBOL_DIM_MAX if isinstance(d, str) else int(d)
            symbolic = [d for d in lead if isinstance(d, str)]
            if not symbolic:
                m_dim: DimExpr = m_static
            elif len(lead) == 1:
                m_dim = lead[0]
            else:
                m_dim = tuple(lead)
            k, nn = int(wt.shape[0]), int(wt.shape[1])
            fused = n.attrs.get("fused_op")
            inputs = [_slice(memory_plan, i) for i in n.inputs]
            out_slice, node_id = out, n.id
            if fused is None:
                cons = graph.consumers(n.id)
                if len(cons) == 1 and n.id not in graph.outputs:
                    add = graph.get_node(cons[0])
                    if add.opcode == Opcode.Add and "fused_op" not in add.attrs:
                        other = [i for i in add.inputs if i != n.id]
                        if len(other) == 1:
                            b = graph.get_node(other[0])
                            if (b.opcode == Opcode.Constant and len(b.output_type.shape) == 1
                                    and b.output_type.numel_max() == nn):
                                inputs.append(_slice(memory_plan, b.id))
                                out_slice = _slice(memory_plan, add.id)
                                skip.add(add.id)
                                fused = "MatMulAdd"
            fmt = int(w.attrs.get("packed_fmt", L.FMT_I8))
            dt = wt.dtype
            zp = dt.zero_points if dt.zero_points is not None else np.zeros(0, np.float32)
            if dt.kind == "F8":
                zp = np.zeros(len(dt.scales), np.float32)  # cpu/mod.rs:556-558
            meta = QuantizedWeightMeta(
                bit_width=8 if dt.kind in ("I8Scaled", "F8") else 4, scales=dt.scales,
                zero_points=zp, shape=[nn, k],
                quant_block_size=int(w.attrs.get("quant_block_size", 0)),
                codebooks=list(dt.codebooks), fmt=fmt)
            instructions.append(CallKernel(
                kernel_name=_KERNEL_BY_KIND[dt.kind], input_slices=inputs, output_slice=out_slice,
                params=[m_static, k, nn, _EPI[fused]], node_id=node_id,
                param_dims=[m_dim, k, nn], weight_meta=meta))
            continue
        if n.opcode in _BINARY:
            name = _BINARY[n.opcode] + _ACT_SUFFIX.get(n.attrs.get("fused_op"), "") + "_f32"
            instructions.append(CallKernel(name, [_slice(memory_plan, i) for i in n.inputs], out,
                                           [], node_id=n.id,
                                           param_dims=list(n.output_type.shape)))
            continue
        if n.opcode in _UNARY:
            instructions.append(CallKernel(_UNARY[n.opcode],
                                           [_slice(memory_plan, i) for i in n.inputs], out, [],
                                           node_id=n.id, param_dims=list(n.output_type.shape)))
            continue
        if n.opcode in (Opcode.RMSNorm, Opcode.LayerNorm):
            # "rms_norm" params [eps bits] (src/backend/cpu/mod.rs:1526-1545), "norm_f32" params
            # [eps bits, is_batch_norm = 0] (:980-1001), "fused_residual_add_*" params [eps bits, row size]
            # with inputs [residual, main, weight, bias] (:2424-2500).  The row size (weight length) rides
            # along in every case so that batched inputs normalise rows of the hidden size.
            eps = float(n.attrs.get("eps", "1e-5"))
            hidden = int(graph.get_node(n.inputs[1]).output_type.numel_max())
            bits = struct.unpack("<I", struct.pack("<f", eps))[0]
            rms = n.opcode == Opcode.RMSNorm
            if n.id in fused_norm:
                main, residual = fused_norm[n.id]
                slices = [_slice(memory_plan, residual), _slice(memory_plan, main)] + \
                         [_slice(memory_plan, i) for i in n.inputs[1:]]
                name = "fused_residual_add_rms_norm" if rms else "fused_residual_add_layer_norm"
                params = [bits, hidden]
            else:
                slices = [_slice(memory_plan, i) for i in n.inputs]
                name, params = ("rms_norm", [bits, hidden]) if rms else ("norm_f32", [bits, 0, hidden])
            instructions.append(CallKernel(name, slices, out, params, node_id=n.id,
                                           param_dims=list(n.output_type.shape)))
            continue
        if n.opcode == Opcode.Softmax:
            # kernel "softmax", params [axis_dim, stride] (src/backend/cpu/mod.rs:1002-1050)
            shape = list(n.output_type.shape)
            axis = int(n.attrs.get("axis", "0"))
            axis = axis + len(shape) if axis < 0 else axis
            if not 0 <= axis < len(shape):
                raise BackendError("Compilation", f"softmax axis {axis} outside rank {len(shape)}")
            stride = 1
            for d in shape[axis + 1:]:
                if isinstance(d, str):
                    raise BackendError("UnsupportedOp", "softmax over a non-innermost axis needs static "
                                                        "trailing dimensions")
                stride *= int(d)
            axis_dim = shape[axis]
            instructions.append(CallKernel(
                "softmax", [_slice(memory_plan, n.inputs[0])], out,
                [SYMBOL_DIM_MAX if isinstance(axis_dim, str) else int(axis_dim), stride], node_id=n.id,
                param_dims=[axis_dim, stride] + shape))
            continue
        raise BackendError("UnsupportedOp", f"opcode {n.opcode} is not on the CUDA backend's path")
    return ExecutablePlan(instructions, memory_plan.total_size, list(range(len(instructions))))


# ------------------------------------------------------------------------------ executor


class GraphExecutor:
    """src/backend/executor.rs: pipeline order (:205-321) and `execute_internal` (:599-858)."""

    def __init__(self, backend):
        self.backend = backend
        self.cached_arena = None
        self._static_plan: Optional[ExecutablePlan] = None

    def compile_with_weight_dtype(self, graph: ComputeGraph, weight_dtype: WeightDtype,
                                  calibration=None):
        graph = graph.clone()
        fuse_operators(graph)            # step 2  (:233)
        eliminate_dead_code(graph)       # step 2.5 (:240)
        quantize_weights(graph, weight_dtype)  # (:251-288)
        eliminate_dead_code(graph)       # step 3 (:314)
        memory_plan = plan_memory(graph)  # (:317)
        plan = self.backend.compile(graph, memory_plan)  # (:321)
        return plan, memory_plan, graph

    def compile_with_plan_and_quantize(self, graph: ComputeGraph, quantize: Optional[int],
                                       calibration=None):
        """src/backend/executor.rs:170-188: Some(4) -> I4, Some(8) -> I8, None -> F32."""
        wd = {None: WeightDtype.F32, 4: WeightDtype.I4, 8: WeightDtype.I8}.get(quantize)
        if wd is None:
            raise BackendError("Compilation", f"unsupported quantize bit width {quantize}")
        return self.compile_with_weight_dtype(graph, wd, calibration)

    @staticmethod
    def shape_env_from_inputs(graph: ComputeGraph, inputs: Sequence[bytes]) -> ShapeEnv:
        """`ShapeEnv::from_graph_inputs`: a single symbolic dim per input is solved from the
        input's byte size."""
        env = ShapeEnv()
        for nid, data in zip(graph.inputs, inputs):
            shape = graph.get_node(nid).output_type.shape
            syms = [d for d in shape if isinstance(d, str)]
            known = 1
            for d in shape:
                if not isinstance(d, str):
                    known *= int(d)
            nbytes = len(data) if not isinstance(data, np.ndarray) else data.nbytes
            if not syms:
                if nbytes != known * 4:
                    raise BackendError("Dispatch", f"input {nid}: expected {known * 4} bytes, "
                                                   f"got {nbytes}")
                continue
            if len(syms) > 1 or known == 0 or nbytes % (known * 4) != 0:
                raise BackendError("Dispatch", f"input {nid}: cannot solve symbolic shape {shape} "
                                               f"from {nbytes} bytes")
            val = nbytes // (known * 4)
            if syms[0] in env and env[syms[0]] != val:
                raise BackendError("Dispatch", f"symbol '{syms[0]}' bound to both {env[syms[0]]} "
                                               f"and {val}")
            if val > SYMBOL_DIM_MAX:
                raise BackendError("Dispatch", f"symbol '{syms[0]}'={val} exceeds SYMBOL_DIM_MAX")
            env[syms[0]] = val
        return env

    def execute(self, graph: ComputeGraph, plan: ExecutablePlan, memory_plan: MemoryPlan,
                inputs: Sequence[bytes]) -> List[bytes]:
        if len(inputs) != len(graph.inputs):
            raise BackendError("Dispatch", f"expected {len(graph.inputs)} inputs, "
                                           f"got {len(inputs)}")
        env = self.shape_env_from_inputs(graph, inputs)
        if not graph.has_static_shapes():
            # symbolic shapes: size the slots (and with them the arena) for this call's dimensions
            # (src/backend/executor.rs:599-717); a later, larger call gets a larger arena and
            # materialises the constants again
            tight = tighten(memory_plan, graph, env)
            plan = tighten_slices(plan, memory_plan, tight, env)
            memory_plan = tight
            have = self.cached_arena
            if have is not None and getattr(have, "total_bytes", None) is None:
                have_bytes = len(have)
            else:
                have_bytes = have.total_bytes if have is not None else 0
            if have is not None and have_bytes < tight.total_size:
                if hasattr(have, "close"):
                    have.close()
                self.cached_arena, self._static_plan = None, None
        first = self.cached_arena is None
        if first:
            self.cached_arena = self.backend.allocate_arena(memory_plan.total_size)
        arena = self.cached_arena
        for (nid, slot), data in zip(memory_plan.inputs, inputs):
            self.backend.write_arena(arena, slot.offset, data)
        run = plan
        if not first:   # constants are in place: replay without WriteConst / Fill
            run = ExecutablePlan([i for i in plan.instructions if not isinstance(i, (WriteConst, Fill))],
                                 plan.arena_size, []) if not graph.has_static_shapes() else self._static_plan
        self.backend.dispatch(run, arena, env)
        if first:
            # Constants are materialised once; later calls replay the plan without
            # WriteConst / Fill (src/backend/executor.rs:639-667) -- the device arena persists.
            self._static_plan = ExecutablePlan(
                [i for i in plan.instructions if not isinstance(i, (WriteConst, Fill))],
                plan.arena_size, [])
        outs = []
        for nid, slot in memory_plan.outputs:
            size = self._resolved_size(graph.get_node(nid), env, slot.size)
            outs.append(self.backend.read_arena(arena, slot.offset, size))
        return outs

    def bind_pinned(self, graph: ComputeGraph, memory_plan: MemoryPlan):
        """Replay path for static shapes: pinned host staging buffers for every graph input and
        output, and one captured CUDA graph holding [H2D copies, the static plan, D2H copies].
        Requires one prior `execute` (constants materialised, weights repacked).  Returns
        (inputs, outputs): lists of f32 numpy views over the pinned buffers."""
        if self.cached_arena is None or self._static_plan is None:
            raise BackendError("Dispatch", "bind_pinned: call execute() once first")
        if not graph.has_static_shapes():
            raise BackendError("UnsupportedOp", "bind_pinned needs static shapes")
        be, lib = self.backend, self.backend.lib
        self._pinned_ptrs = []

        def pinned(nbytes):
            p = ctypes.c_void_p()
            rc = lib.fnn_cuda_host_alloc(nbytes, ctypes.byref(p))
            if rc != L.FNN_OK:
                raise BackendError.from_status(rc)
            self._pinned_ptrs.append(p.value)
            return p.value, np.ctypeslib.as_array((ctypes.c_float * (nbytes // 4)).from_address(p.value))

        ins = [pinned(slot.size) for _, slot in memory_plan.inputs]
        outs = [pinned(slot.size) for _, slot in memory_plan.outputs]
        arena, env = self.cached_arena, ShapeEnv()

        def rc_ok(rc):
            if rc != L.FNN_OK:
                raise BackendError.from_status(rc)

        rc_ok(lib.fnn_cuda_graph_begin(be.ctx))
        try:
            for (ptr, _), (_, slot) in zip(ins, memory_plan.inputs):
                rc_ok(lib.fnn_cuda_arena_write_async(arena.handle, slot.offset, ptr, slot.size))
            be.dispatch(self._static_plan, arena, env)
            for (ptr, _), (_, slot) in zip(outs, memory_plan.outputs):
                rc_ok(lib.fnn_cuda_arena_read_async(arena.handle, slot.offset, ptr, slot.size))
        finally:
            g = ctypes.c_void_p()
            rc = lib.fnn_cuda_graph_end(be.ctx, ctypes.byref(g))
        rc_ok(rc)
        self._replay = g.value
        return [a for _, a in ins], [a for _, a in outs]

    def replay_pinned(self) -> None:
        """Launch the captured [H2D, plan, D2H] graph and wait for the result."""
        lib, be = self.backend.lib, self.backend
        rc = lib.fnn_cuda_graph_launch(be.ctx, self._replay)
        if rc == L.FNN_OK:
            rc = lib.fnn_cuda_sync(be.ctx)
        if rc != L.FNN_OK:
            raise BackendError.from_status(rc)

    def execute_profile(self, graph, plan, memory_plan, inputs):
        env = self.shape_env_from_inputs(graph, inputs)
        if self.cached_arena is None:
            self.cached_arena = self.backend.allocate_arena(memory_plan.total_size)
        for (nid, slot), data in zip(memory_plan.inputs, inputs):
            self.backend.write_arena(self.cached_arena, slot.offset, data)
        return self.backend.dispatch_profile(plan, self.cached_arena, env)

    @staticmethod
    def _resolved_size(node: IRNode, env: ShapeEnv, planned: int) -> int:
        n = 1
        for d in node.output_type.shape:
            n *= env.resolve(d)
        return min(n * 4, planned)


class AotExecutor:
    """Python-facing executor with the constructor of fastnn's `AotExecutor`
    (src/python/nn.rs:1221-1364): ONNX-style node dicts + a parameter dict.  `params` become
    `Constant` nodes (src/onnx/converter.rs:114-133), `Gemm` lowers to matmul (+ add)
    (:290-318).  Supported op_types: MatMul, Gemm (transB = 0), Add, Relu, Gelu, Silu, RMSNorm, LayerNorm, Softmax."""

    def __init__(self, nodes: Sequence[Dict[str, object]], params: Dict[str, np.ndarray],
                 input_names: Sequence[str], output_names: Sequence[str],
                 input_shapes: Optional[Dict[str, Sequence[int]]] = None, quantize=None,
                 backend=None):
        weight_dtype = WeightDtype.from_quantize(quantize)
        gb = GraphBuilder()
        env: Dict[str, GraphTensor] = {}
        for name in input_names:
            dims = list((input_shapes or {}).get(name, []))
            if not dims:
                raise ValueError(f"input_shapes must give a shape for '{name}'")
            env[name] = gb.input_with_dims([f"d{-d}" if d < 0 else int(d) for d in dims], F32)
        for name in sorted(params):
            arr = np.ascontiguousarray(params[name], dtype=np.float32)
            env[name] = gb.constant(arr, TensorType.new(list(arr.shape)))

        def names(v):
            if isinstance(v, str):
                return [x.strip() for x in v.strip("[]").split(",") if x.strip()]
            return list(v)

        for nd in nodes:
            op = str(nd.get("op_type", ""))
            ins, outs = names(nd.get("inputs", [])), names(nd.get("outputs", []))
            t = [env[i] for i in ins]
            if op == "MatMul":
                r = gb.matmul(t[0], t[1])
            elif op == "Gemm":
                if str(nd.get("transB", "0")) not in ("0", "0.0"):
                    raise BackendError(
                        "UnsupportedOp", "Gemm with transB=1 leaves a Transpose between the "
                        "constant and the MatMul, which the quantization pass skips; feed [K,N]")
                r = gb.matmul(t[0], t[1])
                if len(t) > 2:
                    r = gb.add(r, t[2])
            elif op == "Add":
                r = gb.add(t[0], t[1])
            elif op == "Relu":
                r = gb.relu(t[0])
            elif op == "Gelu":
                r = gb.gelu(t[0])
            elif op in ("Silu", "Swish"):
                r = gb.silu(t[0])
            elif op in ("RMSNorm", "RmsNorm", "SimplifiedLayerNormalization"):
                r = gb.rms_norm(t[0], t[1], float(nd.get("eps", nd.get("epsilon", 1e-5))))
            elif op in ("LayerNorm", "LayerNormalization"):
                r = gb.layer_norm(t[0], t[1], t[2], float(nd.get("eps", nd.get("epsilon", 1e-5))))
            elif op == "Softmax":
                r = gb.softmax(t[0], int(nd.get("axis", -1)))
            else:
                raise BackendError("UnsupportedOp", f"op_type '{op}' is not on the CUDA path")
            env[outs[0]] = r
        graph = gb.to_graph()
        graph.inputs = gb.recorded_input_ids()
        graph.outputs = [env[o].node_id() for o in output_names]
        self.input_names, self.output_names = list(input_names), list(output_names)
        self.backend = backend if backend is not None else CudaBackend()
        self.executor = GraphExecutor(self.backend)
        self.plan, self.memory_plan, self.graph = self.executor.compile_with_weight_dtype(
            graph, weight_dtype)

    @classmethod
    def from_onnx(cls, source, quantize=None, backend=None,
                  input_shapes: Optional[Dict[str, Sequence[int]]] = None) -> "AotExecutor":
        """Compile an ONNX file (a path or its bytes) -- what fastnn's Python front end does with
        `import_onnx_to_compute_graph` before it builds an `AotExecutor` (fastnn/io/onnx.py:276-466)."""
        from .onnx_import import read_onnx, to_aot_arguments
        nodes, params, ins, outs, shapes = to_aot_arguments(read_onnx(source), input_shapes)
        return cls(nodes, params, ins, outs, shapes, quantize=quantize, backend=backend)

    def forward(self, inputs: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        data = []
        for name in self.input_names:
            if name not in inputs:
                raise ValueError(f"required input '{name}' not found")
            data.append(np.ascontiguousarray(inputs[name], dtype=np.float32).tobytes())
        raw = self.executor.execute(self.graph, self.plan, self.memory_plan, data)
        env = self.executor.shape_env_from_inputs(self.graph, data)
        out = {}
        for name, nid, buf in zip(self.output_names, self.graph.outputs, raw):
            shape = [env.resolve(d) for d in self.graph.get_node(nid).output_type.shape]
            out[name] = np.frombuffer(buf, dtype=np.float32).reshape(shape).copy()
        return out

    def bind_pinned(self) -> None:
        """Prepare `forward_pinned`: inputs are then written into `self.pinned_inputs[name]`
        (pinned host memory) and results appear in the arrays `forward_pinned` returns."""
        ins, outs = self.executor.bind_pinned(self.graph, self.memory_plan)
        self.pinned_inputs, self.pinned_outputs = {}, {}
        for name, nid, arr in zip(self.input_names, self.graph.inputs, ins):
            self.pinned_inputs[name] = arr.reshape(
                [int(d) for d in self.graph.get_node(nid).output_type.shape])
        for name, nid, arr in zip(self.output_names, self.graph.outputs, outs):
            self.pinned_outputs[name] = arr.reshape(
                [int(d) for d in self.graph.get_node(nid).output_type.shape])

    def forward_pinned(self) -> Dict[str, np.ndarray]:
        """One step from host memory to host memory: pinned H2D of the inputs, the plan,
        D2H of the outputs, synchronize.  One CUDA-graph launch."""
        self.executor.replay_pinned()
        return self.pinned_outputs

    def profile(self, inputs: Dict[str, np.ndarray]):
        data = [np.ascontiguousarray(inputs[n], dtype=np.float32).tobytes()
                for n in self.input_names]
        return self.executor.execute_profile(self.graph, self.plan, self.memory_plan, data)

    def save(self, plan_path: str, memory_path: str) -> None:
        """Write the compiled plan as `.fnnc` and its memory plan as JSON, the two files
        `Runtime.load` reads (src/backend/runtime.rs:65-110).  The quantized weights go along as the
        plan's WriteConst payloads and kernel metadata: loading never re-quantizes."""
        from .runtime import Runtime
        Runtime(self.executor.backend, self.plan, self.memory_plan).save(plan_path, memory_path)

    def memory_stats(self) -> Dict[str, int]:
        return {"arena_bytes": self.memory_plan.total_size,
                "slots": len(self.memory_plan.slots)}
