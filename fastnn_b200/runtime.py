"""``Runtime``: load and run a compiled plan without the compiler
(src/backend/runtime.rs:65-151 of fastnn), and the two files it reads.

* ``model.fnnc`` is ``bincode::serialize(&ExecutablePlan)`` (bincode 1.3 defaults: little endian,
  fixed-width integers, ``usize`` as u64, sequences and strings with a u64 length, ``Option`` as
  one tag byte, enum variants as a u32 index, fixed arrays without a length, ``Arc<T>`` as ``T``).
  Field order follows the struct definitions in src/backend/mod.rs:27-107 and
  src/ir/node.rs:163-167.
* ``model.memory.json`` is ``serde_json`` of ``MemoryPlan``
  (src/compiler/passes/memory_planning.rs:6-29): ``total_size``, ``slots`` keyed by the node id as
  a string, ``secondary_slots``, ``outputs``, ``tightened_params``.

Quantized weights travel inside the plan exactly as the compiler produced them: the
``WriteConst`` payload (packed rows + 16 margin words) and the ``QuantizedWeightMeta`` of the
consuming kernel.  Loading a plan therefore never re-quantizes: the first ``run`` writes the
payload into the device arena and the backend builds its kernel layouts from there
(``fnn_cuda_qweight_from_arena``).

The reference's metadata has no format field: the kernel name (``matmul_i8/_i4/_f8/_f4``) and a
non-empty ``codebooks`` list say which packed word type the bytes hold
(src/backend/cpu/mod.rs:406-495).
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib as L
from .backend import (BackendError, BufferSlice, CallKernel, ExecutablePlan, Fill, MemCopy,
                      QuantizedWeightMeta, ShapeEnv, WriteConst)

_KERNEL_FMT = {"matmul_i8": L.FMT_I8, "matmul_i4": L.FMT_I4, "matmul_f8": L.FMT_F8, "matmul_f4": L.FMT_F4}


# ------------------------------------------------------------------------------ bincode writer


class _Writer:
    def __init__(self):
        self.parts: List[bytes] = []

    def u8(self, v):
        self.parts.append(struct.pack("<B", v))

    def u32(self, v):
        self.parts.append(struct.pack("<I", v))

    def u64(self, v):
        self.parts.append(struct.pack("<Q", int(v)))

    def f32(self, v):
        self.parts.append(struct.pack("<f", float(v)))

    def string(self, s: str):
        b = s.encode("utf-8")
        self.u64(len(b))
        self.parts.append(b)

    def slice_(self, s: BufferSlice):
        self.u64(s.offset)
        self.u64(s.size)

    def f32_vec(self, a):
        a = np.ascontiguousarray(a, dtype="<f4").ravel()
        self.u64(a.size)
        self.parts.append(a.tobytes())

    def bytes(self) -> bytes:
        return b"".join(self.parts)


def _write_dim(w: _Writer, d) -> None:
    if isinstance(d, tuple):
        if any(isinstance(f, str) for f in d):
            raise BackendError("Compilation", "a plan with a symbolic batch product must be specialised "
                                              "before it is saved (the format has no product expression)")
        prod = 1
        for f in d:
            prod *= int(f)
        d = prod
    if isinstance(d, str):
        w.u32(1)          # DimExpr::Symbol
        w.string(d)
    else:
        w.u32(0)          # DimExpr::Known
        w.u64(d)


def _write_meta(w: _Writer, m: QuantizedWeightMeta) -> None:
    w.u64(m.bit_width)
    w.f32_vec(m.scales)
    w.f32_vec(m.zero_points)
    w.u64(len(m.shape))
    for d in m.shape:
        w.u64(d)
    w.u64(m.quant_block_size)
    w.u64(len(m.codebooks))
    for cb in m.codebooks:
        cb = np.ascontiguousarray(cb, dtype="<f4").ravel()
        if cb.size != 16:
            raise BackendError("Compilation", "a codebook has 16 centroids")
        w.parts.append(cb.tobytes())


def plan_to_bytes(plan: ExecutablePlan) -> bytes:
    """``bincode::serialize(&ExecutablePlan)``."""
    w = _Writer()
    w.u64(len(plan.instructions))
    for ins in plan.instructions:
        if isinstance(ins, CallKernel):
            w.u32(0)
            w.string(ins.kernel_name)
            w.u64(len(ins.input_slices))
            for s in ins.input_slices:
                w.slice_(s)
            w.slice_(ins.output_slice)
            if ins.secondary_output_slice is None:
                w.u8(0)
            else:
                w.u8(1)
                w.slice_(ins.secondary_output_slice)
            w.u64(len(ins.params))
            for p in ins.params:
                w.u64(p)
            if ins.node_id is None:
                w.u8(0)
            else:
                w.u8(1)
                w.u64(ins.node_id)
            if ins.param_dims is None:
                w.u8(0)
            else:
                w.u8(1)
                w.u64(len(ins.param_dims))
                for d in ins.param_dims:
                    _write_dim(w, d)
            if ins.weight_meta is None:
                w.u8(0)
            else:
                w.u8(1)
                _write_meta(w, ins.weight_meta)
        elif isinstance(ins, MemCopy):
            w.u32(1)
            w.slice_(ins.dst)
            w.slice_(ins.src)
        elif isinstance(ins, Fill):
            w.u32(2)
            w.slice_(ins.dst)
            w.f32(ins.value)
        elif isinstance(ins, WriteConst):
            w.u32(3)
            w.slice_(ins.dst)
            w.u64(len(ins.data))
            w.parts.append(bytes(ins.data))
        else:
            raise BackendError("Compilation", f"unknown instruction {type(ins).__name__}")
    w.u64(plan.arena_size)
    w.u64(len(plan.levels))
    for lv in plan.levels:
        w.u64(lv)
    return w.bytes()


# ------------------------------------------------------------------------------ bincode reader


class _Reader:
    def __init__(self, data: bytes):
        self.d, self.at = memoryview(data), 0

    def take(self, n: int) -> memoryview:
        if n < 0 or self.at + n > len(self.d):
            raise BackendError("Compilation", f"truncated plan file: wanted {n} bytes at offset {self.at} "
                                              f"of {len(self.d)}")
        out = self.d[self.at:self.at + n]
        self.at += n
        return out

    def u8(self):
        return self.take(1)[0]

    def u32(self):
        return struct.unpack("<I", self.take(4))[0]

    def u64(self):
        return struct.unpack("<Q", self.take(8))[0]

    def f32(self):
        return struct.unpack("<f", self.take(4))[0]

    def string(self):
        return bytes(self.take(self.u64())).decode("utf-8")

    def slice_(self):
        return BufferSlice(self.u64(), self.u64())

    def f32_vec(self):
        n = self.u64()
        return np.frombuffer(self.take(4 * n), dtype="<f4").astype(np.float32)

    def option(self) -> bool:
        tag = self.u8()
        if tag > 1:
            raise BackendError("Compilation", f"bad Option tag {tag} at offset {self.at - 1}")
        return tag == 1


def _read_dim(r: _Reader):
    v = r.u32()
    if v == 0:
        return int(r.u64())
    if v == 1:
        return r.string()
    if v == 2:              # DimExpr::Bounded { sym, max }: resolved like a symbol
        sym = r.string()
        r.u64()
        return sym
    raise BackendError("Compilation", f"unknown DimExpr variant {v}")


def _read_meta(r: _Reader, kernel_name: str) -> QuantizedWeightMeta:
    bit_width = r.u64()
    scales, zeros = r.f32_vec(), r.f32_vec()
    shape = [int(r.u64()) for _ in range(r.u64())]
    qblock = r.u64()
    codebooks = [np.frombuffer(r.take(64), dtype="<f4").astype(np.float32) for _ in range(r.u64())]
    fmt = _KERNEL_FMT.get(kernel_name, L.FMT_I8 if bit_width == 8 else L.FMT_I4)
    if fmt == L.FMT_I4 and codebooks:
        fmt = L.FMT_I4CB
    return QuantizedWeightMeta(bit_width=bit_width, scales=scales, zero_points=zeros, shape=shape,
                               quant_block_size=qblock, codebooks=codebooks, fmt=fmt)


def plan_from_bytes(data: bytes) -> ExecutablePlan:
    """``bincode::deserialize::<ExecutablePlan>``."""
    r = _Reader(data)
    instructions = []
    for _ in range(r.u64()):
        variant = r.u32()
        if variant == 0:
            name = r.string()
            inputs = [r.slice_() for _ in range(r.u64())]
            out = r.slice_()
            secondary = r.slice_() if r.option() else None
            params = [int(r.u64()) for _ in range(r.u64())]
            node_id = int(r.u64()) if r.option() else None
            dims = [_read_dim(r) for _ in range(r.u64())] if r.option() else None
            meta = _read_meta(r, name) if r.option() else None
            instructions.append(CallKernel(name, inputs, out, params, node_id, dims, meta, secondary))
        elif variant == 1:
            instructions.append(MemCopy(r.slice_(), r.slice_()))
        elif variant == 2:
            instructions.append(Fill(r.slice_(), r.f32()))
        elif variant == 3:
            dst = r.slice_()
            instructions.append(WriteConst(dst, bytes(r.take(r.u64()))))
        else:
            raise BackendError("Compilation", f"unknown Instruction variant {variant}")
    arena_size = int(r.u64())
    levels = [int(r.u64()) for _ in range(r.u64())]
    if r.at != len(r.d):
        raise BackendError("Compilation", f"{len(r.d) - r.at} trailing bytes after the plan")
    return ExecutablePlan(instructions, arena_size, levels)


# ------------------------------------------------------------------------------ memory plan json


def memory_plan_to_json(memory_plan) -> str:
    slots = {str(nid): {"offset": s.offset, "size": s.size, "node_id": nid, "output_index": 0}
             for nid, s in memory_plan.slots.items()}
    return json.dumps({"total_size": memory_plan.total_size, "slots": slots, "secondary_slots": {},
                       "outputs": [nid for nid, _ in memory_plan.outputs], "tightened_params": {}}, indent=2)


class LoadedMemoryPlan:
    """What ``Runtime`` needs of a ``MemoryPlan``: the slots and the output node ids."""

    def __init__(self, total_size: int, slots: Dict[int, BufferSlice], outputs: List[int]):
        self.total_size, self.slots, self.outputs = total_size, slots, outputs


def memory_plan_from_json(text: str) -> LoadedMemoryPlan:
    d = json.loads(text)
    slots = {int(k): BufferSlice(int(v["offset"]), int(v["size"])) for k, v in d["slots"].items()}
    return LoadedMemoryPlan(int(d["total_size"]), slots, [int(o) for o in d.get("outputs", [])])


# ------------------------------------------------------------------------------ runtime


class Runtime:
    """``Runtime<B>`` (src/backend/runtime.rs:29-151): plan + memory plan + cached arena."""

    def __init__(self, backend, plan: ExecutablePlan, memory_plan):
        self.backend, self.plan = backend, plan
        if not isinstance(memory_plan, LoadedMemoryPlan):
            memory_plan = memory_plan_from_json(memory_plan_to_json(memory_plan))
        self.memory_plan = memory_plan
        self.slots_sorted = sorted(memory_plan.slots.items(), key=lambda kv: kv[1].offset)
        self.cached_arena = None
        self._static_plan: Optional[ExecutablePlan] = None

    @classmethod
    def load(cls, backend, plan_path: str, memory_path: str) -> "Runtime":
        with open(plan_path, "rb") as f:
            plan = plan_from_bytes(f.read())
        with open(memory_path) as f:
            memory_plan = memory_plan_from_json(f.read())
        return cls(backend, plan, memory_plan)

    def save(self, plan_path: str, memory_path: str) -> None:
        with open(plan_path, "wb") as f:
            f.write(plan_to_bytes(self.plan))
        slots = {str(nid): {"offset": s.offset, "size": s.size, "node_id": nid, "output_index": 0}
                 for nid, s in self.memory_plan.slots.items()}
        with open(memory_path, "w") as f:
            json.dump({"total_size": self.memory_plan.total_size, "slots": slots, "secondary_slots": {},
                       "outputs": self.memory_plan.outputs, "tightened_params": {}}, f, indent=2)

    def run(self, inputs: Sequence[bytes]) -> List[bytes]:
        """Inputs go to the first slots by offset (the reference's rule, :118-124); the plan is
        dispatched with an empty ShapeEnv; every graph output slot is read back.  The reference
        clears a reused arena and replays every WriteConst; here the arena keeps its constants and
        the repeat runs skip them (like GraphExecutor's static plan, src/backend/executor.rs:639-667),
        so the device layouts built from the weight slots on the first run stay valid."""
        first = self.cached_arena is None
        if first:
            self.cached_arena = self.backend.allocate_arena(self.plan.arena_size)
            self._static_plan = ExecutablePlan(
                [i for i in self.plan.instructions if not isinstance(i, (WriteConst, Fill))],
                self.plan.arena_size, [])
        arena = self.cached_arena
        for (nid, slot), data in zip(self.slots_sorted, inputs):
            self.backend.write_arena(arena, slot.offset, bytes(data))
        self.backend.dispatch(self.plan if first else self._static_plan, arena, ShapeEnv())
        outs = []
        for nid in self.memory_plan.outputs:
            slot = self.memory_plan.slots.get(nid)
            if slot is not None:
                outs.append(self.backend.read_arena(arena, slot.offset, slot.size))
        return outs

    def close(self) -> None:
        if self.cached_arena is not None:
            self.cached_arena.close()
            self.cached_arena = None
