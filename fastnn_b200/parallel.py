"""Column sharding of a quantized Linear across the GPUs of one node.

Output columns of `x @ W` are independent and the packed weight is `[N, K]` row-major, so a column
shard is a contiguous range of packed rows plus the matching slice of the per-row metadata
(per-block scales for the codebook format).  Quantize first, then slice: the bytes of every shard
are then identical to the corresponding rows of the single-GPU weight, including the codebook, which
is global per tensor (src/packed_tensor.rs:1257-1260 of fastnn).

One process per GPU; activations are replicated; every rank computes `[M, N/g]` and the outputs are
all-gathered (NCCL on GPUs, any torch.distributed backend for the host logic).
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np

from . import _lib as L
from .backend import BackendError, QuantizedWeightMeta


def shard_bounds(n: int, world: int) -> List[Tuple[int, int]]:
    """Row ranges [n0, n1) per rank: equal shares, the remainder spread over the first ranks."""
    base, rem = divmod(n, world)
    out, start = [], 0
    for r in range(world):
        size = base + (1 if r < rem else 0)
        out.append((start, start + size))
        start += size
    return out


def shard_rows(payload: bytes, meta: QuantizedWeightMeta, rank: int, world: int):
    """The packed rows and metadata of `rank`'s column shard, as (payload, meta).  The payload
    keeps the reference format: rows then 16 zero margin words."""
    n, k = meta.shape
    if not (0 <= rank < world) or world < 1:
        raise BackendError("Dispatch", f"bad shard {rank} of {world}")
    n0, n1 = shard_bounds(n, world)[rank]
    items = 4 if meta.fmt in (L.FMT_I8, L.FMT_F8) else 8
    wpr = -(-k // items)
    words = np.frombuffer(payload, dtype=np.uint32)
    if words.size < n * wpr:
        raise BackendError("Dispatch", "payload shorter than the weight it describes")
    part = np.concatenate([words[n0 * wpr:n1 * wpr], np.zeros(16, dtype=np.uint32)])
    scales = np.asarray(meta.scales, dtype=np.float32)
    zeros = np.asarray(meta.zero_points, dtype=np.float32)
    if meta.fmt == L.FMT_I4CB:
        bpr = scales.size // n
        s, z = scales[n0 * bpr:n1 * bpr], zeros
    elif scales.size == n:
        s, z = scales[n0:n1], (zeros[n0:n1] if zeros.size == n else zeros)
    elif scales.size == 1:
        s, z = scales, zeros
    else:
        raise BackendError("UnsupportedOp", "grouped scales cannot be sliced at arbitrary rows")
    sub = QuantizedWeightMeta(bit_width=meta.bit_width, scales=s.copy(), zero_points=z.copy(),
                              shape=[n1 - n0, k], quant_block_size=meta.quant_block_size,
                              codebooks=list(meta.codebooks), fmt=meta.fmt)
    return part.tobytes(), sub


def assemble_columns(parts: List[np.ndarray]) -> np.ndarray:
    """[g] x [M, N_r] outputs (rank order) -> [M, N]."""
    return np.concatenate(parts, axis=1)


class ColumnShardedLinear:
    """One rank's shard of a quantized Linear on its GPU plus the all-gather of the outputs.

    `forward(x)` takes a replicated f32 CUDA tensor [M, K] and returns the full [M, N] on every
    rank.  Shards may differ by one row, so the gather is padded to the widest shard."""

    def __init__(self, backend, payload: bytes, meta: QuantizedWeightMeta, rank: int, world: int,
                 epilogue: int = L.EPI_NONE, group=None):
        import torch  # plumbing: device tensors and torch.distributed
        self.torch, self.backend, self.group = torch, backend, group
        self.rank, self.world, self.epilogue = rank, world, epilogue
        self.bounds = shard_bounds(meta.shape[0], world)
        self.n, self.k = meta.shape
        sub_payload, sub_meta = shard_rows(payload, meta, rank, world)
        self.n_local = sub_meta.shape[0]
        self.n_max = max(b - a for a, b in self.bounds)
        self.weight = backend.upload_qweight(sub_payload, sub_meta)

    def forward(self, x):
        import torch.distributed as dist
        torch = self.torch
        m = x.shape[0]
        local = torch.zeros((m, self.n_max), dtype=torch.float32, device=x.device)
        out = local if self.n_local == self.n_max else torch.empty(
            (m, self.n_local), dtype=torch.float32, device=x.device)
        rc = self.backend.lib.fnn_cuda_qmatmul_ptr(self.backend.ctx, self.weight.handle, x.data_ptr(),
                                                   out.data_ptr(), None, m, self.epilogue, L.PATH_AUTO)
        if rc != 0:
            raise BackendError.from_status(rc)
        if out is not local:
            local[:, : self.n_local] = out
        gathered = torch.empty((self.world, m, self.n_max), dtype=torch.float32, device=x.device)
        dist.all_gather_into_tensor(gathered, local, group=self.group)
        cols = [gathered[r, :, : b - a] for r, (a, b) in enumerate(self.bounds)]
        return torch.cat(cols, dim=1)


class FusedGatherLinear:
    """Column shard whose GEMV writes its outputs straight into every rank's gathered buffer over
    NVLink peer memory (`fnn_cuda_qmatmul_gather`): one kernel per step, no collective call.

    Set-up exchanges CUDA IPC handles of one shared arena per rank through `torch.distributed`
    (any backend; it is host plumbing).  `forward(a_dev_ptr)` launches the step; afterwards
    `gathered()` returns this step's full [M, N] rows as a numpy array."""

    ROWS = 4  # batch rows a gathered slot holds

    def __init__(self, backend, payload: bytes, meta: QuantizedWeightMeta, rank: int, world: int,
                 m_max: int = 4, epilogue: int = L.EPI_NONE, group=None):
        import ctypes
        import torch.distributed as dist
        self.ctypes, self.backend, self.rank, self.world = ctypes, backend, rank, world
        self.epilogue, self.m_max = epilogue, m_max
        self.bounds = shard_bounds(meta.shape[0], world)
        sub_payload, sub_meta = shard_rows(payload, meta, rank, world)
        self.n_local = sub_meta.shape[0]
        self.n_stride = -(-max(b - a for a, b in self.bounds) // 4) * 4
        self.weight = backend.upload_qweight(sub_payload, sub_meta)
        if not 1 <= m_max <= self.ROWS:
            raise ValueError(f"the fused gather serves 1..{self.ROWS} batch rows, got m_max={m_max}")
        word_bytes = 2 * world * self.ROWS * self.n_stride * 8      # {value, step} words, two slots
        self.gather_off, self.counter_off = 0, -(-word_bytes // 256) * 256
        self.plain_off = self.counter_off + 256                     # f32 [world][M][n_stride] after wait()
        self.a_off = self.plain_off + -(-world * self.ROWS * self.n_stride * 4 // 256) * 256
        self.arena = backend.allocate_arena(self.a_off + m_max * meta.shape[1] * 4)
        backend.synchronize()
        handle = (ctypes.c_uint8 * 64)()
        _check_rc(backend.lib.fnn_cuda_ipc_export(self.arena.handle, handle))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_ptrs = (ctypes.c_void_p * world)()
        self._opened = []
        for r in range(world):
            if r == rank:
                self.peer_ptrs[r] = self.arena.device_ptr
            else:
                p = ctypes.c_void_p()
                buf = (ctypes.c_uint8 * 64).from_buffer_copy(handles[r])
                _check_rc(backend.lib.fnn_cuda_ipc_open(backend.ctx, buf, ctypes.byref(p)))
                self.peer_ptrs[r] = p.value
                self._opened.append(p.value)
        self.calls = 0
        dist.barrier(group=group)  # every rank has mapped every buffer before the first step

    def set_activations(self, x: np.ndarray) -> None:
        x = np.ascontiguousarray(x, dtype=np.float32)
        self.m = x.shape[0]
        self.backend.write_arena(self.arena, self.a_off, x.tobytes())

    def forward(self, m: int = None) -> None:
        m = self.m if m is None else m
        rc = self.backend.lib.fnn_cuda_qmatmul_gather(
            self.backend.ctx, self.weight.handle, self.arena.device_ptr + self.a_off, None, m,
            self.epilogue, self.rank, self.world, self.peer_ptrs, self.gather_off, self.counter_off,
            self.n_stride)
        _check_rc(rc)
        self.calls += 1
        self.m = m

    def wait(self) -> None:
        """Enqueue the consumer-side poll for every rank's shard of the last step; it leaves the
        rows as plain f32 [world][M][n_stride] at `plain_off` of the arena."""
        _check_rc(self.backend.lib.fnn_cuda_gather_wait(
            self.backend.ctx, self.arena.device_ptr, self.gather_off, self.counter_off, self.world,
            self.n_stride, self.arena.device_ptr + self.plain_off))

    def gathered(self) -> np.ndarray:
        self.wait()
        nbytes = self.world * self.m * self.n_stride * 4
        raw = self.backend.read_arena(self.arena, self.plain_off, nbytes)
        full = np.frombuffer(raw, np.float32).reshape(self.world, self.m, self.n_stride)
        return np.concatenate([full[r, :, : b - a] for r, (a, b) in enumerate(self.bounds)], axis=1)

    def close(self) -> None:
        self.backend.synchronize()
        for p in self._opened:
            self.backend.lib.fnn_cuda_ipc_close(self.backend.ctx, p)
        self._opened = []
        self.weight.close()
        self.arena.close()


def _check_rc(rc: int) -> None:
    if rc != 0:
        raise BackendError.from_status(rc)
