"""``CudaBackend``: the host-side mirror of fastnn's ``Backend`` trait over the C ABI.

Names, argument meaning and error behaviour follow ``src/backend/mod.rs`` of fastnn:
``BackendError`` (:6-12), ``BufferSlice`` (:27-38), ``QuantizedWeightMeta`` (:43-58),
``Instruction`` (:60-97), ``ExecutablePlan`` (:99-107), ``ProfileEntry`` (:109-115) and the trait
itself (:152-254).  A Rust ``src/backend/cuda`` would be this file's logic over the same
``extern "C"`` symbols.

Differences from ``CpuBackend::compile`` that are deliberate (the CPU backend drops them):
the fused bias/activation of a quantized MatMul is carried to the kernel as an epilogue
(the CPU arm emits ``matmul_i4/i8/f4/f8`` with params ``[M,K,N]`` only,
src/backend/cpu/mod.rs:406-495, and its dispatch ignores a third input slice,
src/backend/cpu/matmul.rs:177).
"""
from __future__ import annotations

import ctypes
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from . import _lib as L

DimExpr = Union[int, str, tuple]  # Known(u64) | Symbol(name) | product of DimExprs
SYMBOL_DIM_MAX = 8192  # src/ir/node.rs:154-160


class BackendError(Exception):
    """``BackendError::{Compilation, Dispatch, Memory, UnsupportedOp}(String)``."""

    def __init__(self, kind: str, msg: str):
        super().__init__(f"{kind} error: {msg}")
        self.kind = kind
        self.msg = msg

    @staticmethod
    def from_status(rc: int) -> "BackendError":
        return BackendError(L.ERR_NAMES.get(rc, f"Status{rc}"), L.last_error())


def _check(rc: int) -> None:
    if rc != L.FNN_OK:
        raise BackendError.from_status(rc)


@dataclass(frozen=True)
class BufferSlice:
    offset: int
    size: int


@dataclass
class QuantizedWeightMeta:
    bit_width: int
    scales: np.ndarray
    zero_points: np.ndarray
    shape: List[int]  # [N, K]: reversed from the node's logical [K, N]
    quant_block_size: int = 0
    codebooks: List[np.ndarray] = field(default_factory=list)
    # which packed word type the bytes hold (the reference encodes this in the kernel name)
    fmt: int = L.FMT_I8


@dataclass
class CallKernel:
    kernel_name: str
    input_slices: List[BufferSlice]
    output_slice: BufferSlice
    params: List[int]
    node_id: Optional[int] = None
    param_dims: Optional[List[DimExpr]] = None
    weight_meta: Optional[QuantizedWeightMeta] = None
    secondary_output_slice: Optional[BufferSlice] = None


@dataclass
class MemCopy:
    dst: BufferSlice
    src: BufferSlice


@dataclass
class Fill:
    dst: BufferSlice
    value: float


@dataclass
class WriteConst:
    dst: BufferSlice
    data: bytes


Instruction = Union[CallKernel, MemCopy, Fill, WriteConst]


@dataclass
class ExecutablePlan:
    instructions: List[Instruction]
    arena_size: int
    levels: List[int] = field(default_factory=list)


@dataclass
class ProfileEntry:
    instruction_index: int
    node_id: Optional[int]
    kernel_name: str
    elapsed_ns: int


class ShapeEnv(dict):
    """Runtime values of symbolic dimension names (src/ir/node.rs:347-495)."""

    def resolve(self, d: DimExpr) -> int:
        if isinstance(d, tuple):   # a product, e.g. the batch rows of a [d1, 8, K] activation
            out = 1
            for f in d:
                out *= self.resolve(f)
            return out
        if isinstance(d, str):
            if d not in self:
                raise BackendError("Dispatch", f"unresolved symbolic dimension '{d}'")
            return int(self[d])
        return int(d)


def resolve_params(params: Sequence[int], param_dims: Optional[Sequence[DimExpr]],
                   env: ShapeEnv, want: int) -> List[int]:
    """src/backend/cpu/params.rs:11-38: re-evaluate symbolic params against the ShapeEnv."""
    if param_dims is not None and len(param_dims) >= want:
        return [env.resolve(d) for d in param_dims[:want]]
    if len(params) < want:
        raise BackendError("Dispatch", f"expected {want} params, got {len(params)}")
    return list(params[:want])


_FUSED_EPILOGUE = {
    None: L.EPI_NONE, "": L.EPI_NONE, "MatMulAdd": L.EPI_NONE,
    "MatMulAddRelu": L.EPI_RELU, "OpRelu": L.EPI_RELU,
    "MatMulAddGelu": L.EPI_GELU, "OpGelu": L.EPI_GELU,
    "MatMulAddSilu": L.EPI_SILU, "OpSilu": L.EPI_SILU,
}

_ELEMENTWISE = {"relu_f32": L.EW_RELU, "gelu_f32": L.EW_GELU, "silu_f32": L.EW_SILU}
for _b, _code in (("add", L.EW_ADD), ("mul", L.EW_MUL), ("sub", L.EW_SUB)):
    _ELEMENTWISE[f"{_b}_f32"] = _code
    for _a, _epi in (("relu", L.EPI_RELU), ("gelu", L.EPI_GELU), ("silu", L.EPI_SILU)):
        _ELEMENTWISE[f"{_b}_{_a}_f32"] = _code | (_epi << 8)  # add_relu_f32, ...

_QMATMUL_KERNELS = ("matmul_i4", "matmul_i8", "matmul_f8", "matmul_f4")


class CudaBuffer:
    """``Backend::Buffer``: one device allocation holding every slot of the MemoryPlan, plus the
    repacked device copies of the quantized weights keyed by their arena slice."""

    def __init__(self, backend: "CudaBackend", total_bytes: int, handle: int, owner=None):
        self.backend = backend
        self.total_bytes = total_bytes
        self.handle = handle
        self._owner = owner  # keeps wrapped external memory alive
        self.qweights: Dict[Tuple[int, int], "QWeightHandle"] = {}
        self.latched_error: Optional[BackendError] = None

    @property
    def device_ptr(self) -> int:
        return int(self.backend.lib.fnn_cuda_arena_device_ptr(self.handle) or 0)

    def close(self) -> None:
        for q in self.qweights.values():
            q.close()
        self.qweights.clear()
        if self.handle and getattr(self.backend, "ctx", None):  # the context outlives its buffers
            self.backend.lib.fnn_cuda_arena_free(self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class QWeightHandle:
    """Device layout of one quantized weight (``fnn_cuda_qweight``)."""

    def __init__(self, backend: "CudaBackend", handle: int, meta: QuantizedWeightMeta):
        self.backend = backend
        self.handle = handle
        self.meta = meta

    def unrepack(self) -> bytes:
        lib = self.backend.lib
        n = lib.fnn_cuda_qweight_packed_bytes(self.handle)
        buf = (ctypes.c_uint8 * n)()
        _check(lib.fnn_cuda_qweight_unrepack(self.handle, buf, n))
        return bytes(buf)

    def close(self) -> None:
        if self.handle and getattr(self.backend, "ctx", None):  # never touch a destroyed context
            self.backend.lib.fnn_cuda_qweight_free(self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CudaBackend:
    """B200 implementation of the ``Backend`` trait (src/backend/mod.rs:152-254)."""

    def __init__(self, device: int = 0, stream: Optional[int] = None, path: int = L.PATH_AUTO):
        self.lib = L.load()
        self.device = device
        self.path = path
        h = ctypes.c_void_p()
        if stream is None:
            _check(self.lib.fnn_cuda_ctx_create(device, ctypes.byref(h)))
        else:
            _check(self.lib.fnn_cuda_ctx_create_on_stream(device, stream, ctypes.byref(h)))
        self.ctx = h.value

    # -- trait ---------------------------------------------------------------------------
    def name(self) -> str:
        return "cuda"

    def allocate_arena(self, total_bytes: int) -> CudaBuffer:
        """Zero-filled, like ``CpuBackend::allocate_arena`` (src/backend/cpu/mod.rs:269-279)."""
        h = ctypes.c_void_p()
        _check(self.lib.fnn_cuda_arena_alloc(self.ctx, total_bytes, ctypes.byref(h)))
        return CudaBuffer(self, total_bytes, h.value)

    def wrap_arena(self, device_ptr: int, total_bytes: int, owner=None) -> CudaBuffer:
        """Arena over device memory owned by the caller (e.g. a torch tensor used for NCCL)."""
        h = ctypes.c_void_p()
        _check(self.lib.fnn_cuda_arena_wrap(self.ctx, device_ptr, total_bytes, ctypes.byref(h)))
        return CudaBuffer(self, total_bytes, h.value, owner)

    def write_arena(self, arena: CudaBuffer, offset: int, data: bytes) -> None:
        """No ``Result`` in the trait: a bad span is clamped and latched for the next dispatch."""
        buf = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data
        rc = self.lib.fnn_cuda_arena_write(arena.handle, offset, buf.ctypes.data, buf.nbytes)
        if rc != L.FNN_OK:
            arena.latched_error = BackendError.from_status(rc)

    def read_arena(self, arena: CudaBuffer, offset: int, size: int) -> bytes:
        out = np.empty(size, dtype=np.uint8)
        rc = self.lib.fnn_cuda_arena_read(arena.handle, offset, out.ctypes.data, size)
        if rc != L.FNN_OK:
            arena.latched_error = BackendError.from_status(rc)
        return out.tobytes()

    def compile(self, graph, memory_plan) -> ExecutablePlan:
        from .compiler import lower_to_plan  # graph-side logic lives with the passes
        return lower_to_plan(graph, memory_plan)

    def dispatch(self, plan: ExecutablePlan, arena: CudaBuffer, shape_env: ShapeEnv) -> None:
        if arena.latched_error is not None:
            err, arena.latched_error = arena.latched_error, None
            raise err
        for instr in plan.instructions:
            self._dispatch_one(instr, arena, shape_env)

    def dispatch_profile(self, plan: ExecutablePlan, arena: CudaBuffer,
                         shape_env: ShapeEnv) -> List[ProfileEntry]:
        """Per-instruction device time from CUDA events (the trait default wall-clocks each
        one-instruction plan, src/backend/mod.rs:178-211, which would time only the launch)."""
        entries = []
        ms = ctypes.c_float()
        for i, instr in enumerate(plan.instructions):
            name = {CallKernel: None, MemCopy: "memcopy", Fill: "fill",
                    WriteConst: "write_const"}[type(instr)]
            if name is None:
                name = instr.kernel_name
            _check(self.lib.fnn_cuda_timer_start(self.ctx, 63))
            self._dispatch_one(instr, arena, shape_env)
            _check(self.lib.fnn_cuda_timer_stop(self.ctx, 63))
            _check(self.lib.fnn_cuda_timer_elapsed_ms(self.ctx, 63, ctypes.byref(ms)))
            entries.append(ProfileEntry(i, getattr(instr, "node_id", None), name,
                                        int(ms.value * 1e6)))
        return entries

    def dispatch_with_persistent_view(self, plan: ExecutablePlan, arena: CudaBuffer,
                                      shape_env: ShapeEnv, persistent_view=None) -> None:
        """The prepared no-copy path strips the WriteConst of every fp32 slot present in the
        view and expects the backend to read those bytes from the view
        (src/backend/executor.rs:737-763, src/backend/prepared.rs:1410-1460).  On a device
        backend that means: upload each (offset, size) -> payload once, then dispatch."""
        if persistent_view:
            done = getattr(arena, "_persistent_uploaded", set())
            for (offset, size), payload in persistent_view.items():
                if (offset, size) not in done:
                    self.write_arena(arena, offset, payload[:size])
                    done.add((offset, size))
            arena._persistent_uploaded = done
        self.dispatch(plan, arena, shape_env)

    # -- extras over the trait ------------------------------------------------------------
    def synchronize(self) -> None:
        _check(self.lib.fnn_cuda_sync(self.ctx))

    def launch_count(self) -> int:
        n = ctypes.c_uint64()
        _check(self.lib.fnn_cuda_launch_count(self.ctx, ctypes.byref(n)))
        return int(n.value)

    def last_path(self) -> str:
        return self.lib.fnn_cuda_last_path(self.ctx).decode()

    def device_info(self) -> dict:
        sm, ma, mi, mem = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
        _check(self.lib.fnn_cuda_device_info(self.ctx, ctypes.byref(sm), ctypes.byref(ma),
                                             ctypes.byref(mi), ctypes.byref(mem)))
        return {"sm_count": sm.value, "cc": (ma.value, mi.value), "total_mem": mem.value}

    def upload_qweight(self, payload: bytes, meta: QuantizedWeightMeta, arena: Optional[CudaBuffer] = None,
                       offset: int = 0, size: int = 0) -> QWeightHandle:
        """``get_or_cache_packed`` + ``packed_tensor_from_meta`` on the device.  With ``arena`` the
        payload is the WriteConst slot ``[offset, offset + size)`` already on the device (``payload``
        is ignored): its rows are used in place or copied device-to-device."""
        data = np.frombuffer(payload, dtype=np.uint8) if arena is None else None
        scales = np.ascontiguousarray(meta.scales, dtype=np.float32)
        zeros = np.ascontiguousarray(meta.zero_points, dtype=np.float32)
        cb = (np.ascontiguousarray(meta.codebooks[0], dtype=np.float32)
              if meta.codebooks else None)
        if len(meta.shape) != 2:
            raise BackendError("UnsupportedOp",
                               f"quantized weight of rank {len(meta.shape)} (only MatMul weights)")
        n, k = meta.shape
        h = ctypes.c_void_p()
        tail = (n, k, scales.ctypes.data if scales.size else None, scales.size,
                zeros.ctypes.data if zeros.size else None, zeros.size, meta.quant_block_size,
                cb.ctypes.data if cb is not None else None, ctypes.byref(h))
        if arena is None:
            _check(self.lib.fnn_cuda_qweight_upload(self.ctx, meta.fmt, data.ctypes.data, data.nbytes, *tail))
        else:
            _check(self.lib.fnn_cuda_qweight_from_arena(self.ctx, meta.fmt, arena.handle, offset, size, *tail))
        qw = QWeightHandle(self, h.value, meta)
        # build the kernel layouts now, so a later graph capture finds them in place
        _check(self.lib.fnn_cuda_qweight_prepare(self.ctx, h.value, self.path))
        return qw

    def close(self) -> None:
        if getattr(self, "ctx", None):
            self.lib.fnn_cuda_ctx_destroy(self.ctx)
            self.ctx = None

    # -- per-instruction dispatch ------------------------------------------------------------
    def _dispatch_one(self, instr: Instruction, arena: CudaBuffer, env: ShapeEnv) -> None:
        lib = self.lib
        if isinstance(instr, WriteConst):
            self.write_arena(arena, instr.dst.offset, instr.data[: instr.dst.size])
            if arena.latched_error is not None:
                err, arena.latched_error = arena.latched_error, None
                raise err
            return
        if isinstance(instr, Fill):
            _check(lib.fnn_cuda_fill(self.ctx, arena.handle, instr.dst.offset, instr.dst.size,
                                     instr.value))
            return
        if isinstance(instr, MemCopy):
            _check(lib.fnn_cuda_memcpy(self.ctx, arena.handle, instr.dst.offset, instr.src.offset,
                                       min(instr.dst.size, instr.src.size)))
            return
        name = instr.kernel_name
        if name in _QMATMUL_KERNELS:
            self._dispatch_qmatmul(instr, arena, env)
            return
        if name in _ELEMENTWISE:
            a = instr.input_slices[0]
            b = instr.input_slices[1] if len(instr.input_slices) > 1 else a
            out_len = instr.output_slice.size // 4
            if instr.param_dims:
                out_len = 1
                for d in instr.param_dims:
                    out_len *= env.resolve(d)
            _check(lib.fnn_cuda_elementwise(self.ctx, _ELEMENTWISE[name], arena.handle, a.offset,
                                            a.size // 4, b.offset, b.size // 4,
                                            instr.output_slice.offset, out_len))
            return
        if name in ("rms_norm", "norm_f32", "fused_residual_add_rms_norm", "fused_residual_add_layer_norm"):
            sl = list(instr.input_slices)
            fused = name.startswith("fused_residual_add_")
            residual = sl.pop(0) if fused else None          # fused: [residual, main, weight, bias]
            data = sl.pop(0)
            weight = sl.pop(0) if sl else None
            bias = sl.pop(0) if sl else None
            if name == "norm_f32" and len(instr.params) > 1 and instr.params[1] == 1:
                raise BackendError("UnsupportedOp", "batch norm is not on the CUDA backend's path")
            n = instr.output_slice.size // 4
            if instr.param_dims:
                n = 1
                for d in instr.param_dims:
                    n *= env.resolve(d)
            eps = struct.unpack("<f", struct.pack("<I", instr.params[0] & 0xFFFFFFFF))[0]
            row_idx = 2 if name == "norm_f32" else 1
            row = instr.params[row_idx] if len(instr.params) > row_idx and instr.params[row_idx] > 0 else \
                (weight.size // 4 if weight is not None else n)
            kind = 0 if name.endswith("rms_norm") else 1
            _check(lib.fnn_cuda_row_norm(
                self.ctx, arena.handle, kind, data.offset, n, residual.offset if residual else -1,
                weight.offset if weight else -1, weight.size // 4 if weight else 0,
                bias.offset if bias else -1, bias.size // 4 if bias else 0, row, eps,
                instr.output_slice.offset))
            return
        if name == "softmax":
            src = instr.input_slices[0]
            dims = resolve_params(instr.params, instr.param_dims[:2] if instr.param_dims else None, env, 2)
            n = instr.output_slice.size // 4
            if instr.param_dims and len(instr.param_dims) > 2:
                n = 1
                for d in instr.param_dims[2:]:
                    n *= env.resolve(d)
            _check(lib.fnn_cuda_softmax(self.ctx, arena.handle, src.offset, n, max(dims[0], 1),
                                        max(dims[1], 1), instr.output_slice.offset))
            return
        # no CPU fallback: anything else is not this backend's job
        raise BackendError("UnsupportedOp", f"kernel '{name}' is not implemented by the CUDA backend")

    def _dispatch_qmatmul(self, instr: CallKernel, arena: CudaBuffer, env: ShapeEnv) -> None:
        name = instr.kernel_name
        if len(instr.input_slices) < 2:
            raise BackendError("Dispatch", f"{name}: expected activation and weight slices")
        m, k, n = resolve_params(instr.params, instr.param_dims, env, 3)
        a_slice, w_slice = instr.input_slices[0], instr.input_slices[1]
        meta = instr.weight_meta
        if meta is None:
            raise BackendError("Dispatch", f"{name}: quantized weight metadata missing")
        if list(meta.shape) != [n, k]:
            raise BackendError(
                "Dispatch", f"{name}: params [M,K,N]=[{m},{k},{n}] disagree with weight shape "
                            f"{list(meta.shape)}")
        if a_slice.size < m * k * 4 or instr.output_slice.size < m * n * 4:
            raise BackendError("Dispatch", f"{name}: slice too small for [M,K,N]=[{m},{k},{n}]")
        key = (w_slice.offset, w_slice.size)
        qw = arena.qweights.get(key)
        if qw is None:
            # Lazily build the kernel layouts from the WriteConst bytes already in the arena (on the
            # device: they never come back to the host), keyed by the weight slice like the CPU
            # backend's packed-weight cache (src/backend/cpu/mod.rs:62-89).
            qw = self.upload_qweight(b"", meta, arena, w_slice.offset, w_slice.size)
            arena.qweights[key] = qw
        epilogue = instr.params[3] if len(instr.params) > 3 else L.EPI_NONE
        bias_off = instr.input_slices[2].offset if len(instr.input_slices) > 2 else -1
        _check(self.lib.fnn_cuda_qmatmul(self.ctx, qw.handle, arena.handle, a_slice.offset,
                                         instr.output_slice.offset, bias_off, m, epilogue,
                                         self.path))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
