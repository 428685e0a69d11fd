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


class PeerArena:
    """One zero-filled device arena per rank, exported with CUDA IPC and mapped by every peer
    (`fnn_cuda_ipc_export/open/close`): plain peer pointers over NVLink, no multicast object.
    `peers[r]` is rank r's arena as seen from this process (`peers[rank]` is the local one)."""

    def __init__(self, backend, nbytes: int, rank: int, world: int, group=None):
        import ctypes
        self.backend, self.rank, self.world, self.group = backend, rank, world, group
        self.arena = backend.allocate_arena(nbytes)
        backend.synchronize()
        self.peers = (ctypes.c_void_p * world)()
        self._opened = []
        if world == 1:   # a single rank is its own and only peer: nothing to exchange
            self.peers[0] = self.arena.device_ptr
            return
        import torch.distributed as dist
        handle = (ctypes.c_uint8 * 64)()
        _check_rc(backend.lib.fnn_cuda_ipc_export(self.arena.handle, handle))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        for r in range(world):
            if r == rank:
                self.peers[r] = self.arena.device_ptr
            else:
                p = ctypes.c_void_p()
                buf = (ctypes.c_uint8 * 64).from_buffer_copy(handles[r])
                _check_rc(backend.lib.fnn_cuda_ipc_open(backend.ctx, buf, ctypes.byref(p)))
                self.peers[r] = p.value
                self._opened.append(p.value)
        dist.barrier(group=group)  # every rank has mapped every buffer before the first step

    @property
    def device_ptr(self) -> int:
        return self.arena.device_ptr

    def close(self) -> None:
        """Unmaps the peers' arenas and frees the local one.  The barriers keep a rank from freeing
        memory a peer's kernel may still be storing into."""
        self.backend.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
            for p in self._opened:
                self.backend.lib.fnn_cuda_ipc_close(self.backend.ctx, p)
            self._opened = []
            dist.barrier(group=self.group)
        self.arena.close()


class AllGatherLinear:
    """Column shard of a quantized Linear for any batch size: the tcgen05 kernel's epilogue stores
    this rank's [M, n_local] block into its column range of every rank's [M, N] rows over NVLink
    (`fnn_cuda_qmatmul_allgather`); the kernel ends only when every rank's block has arrived, so the
    rows at `out_off` of the local arena are the next layer's activations.  Shards are equal (N divisible by
    the number of ranks).  `out_off` / `ctr_off`: offsets inside the PeerArena of the f32 [m_max, N]
    rows and of the 8-byte counter pair; the same on every rank."""

    def __init__(self, backend, payload: bytes, meta: QuantizedWeightMeta, rank: int, world: int,
                 peer_arena: PeerArena, out_off: int, ctr_off: int, epilogue: int = L.EPI_NONE,
                 bias: np.ndarray = None, bias_off: int = None):
        self.backend, self.rank, self.world, self.pa = backend, rank, world, peer_arena
        self.epilogue, self.out_off, self.ctr_off = epilogue, out_off, ctr_off
        self.n, self.k = meta.shape
        if self.n % world:
            raise BackendError("UnsupportedOp", f"{self.n} columns do not split evenly over {world} ranks")
        n0, n1 = shard_bounds(self.n, world)[rank]
        self.col0, self.n_local = n0, n1 - n0
        sub_payload, sub_meta = shard_rows(payload, meta, rank, world)
        self.weight = backend.upload_qweight(sub_payload, sub_meta)
        self.bias_ptr = None
        if bias is not None:
            part = np.ascontiguousarray(bias[n0:n1], dtype=np.float32)
            backend.write_arena(peer_arena.arena, bias_off, part.tobytes())
            self.bias_ptr = peer_arena.device_ptr + bias_off

    def forward(self, a_dev_ptr: int, m: int) -> None:
        lib, b = self.backend.lib, self.backend
        if self.world == 1:   # nothing to gather: the plain call writes the rows where they belong
            _check_rc(lib.fnn_cuda_qmatmul_ptr(b.ctx, self.weight.handle, a_dev_ptr,
                                               self.pa.device_ptr + self.out_off, self.bias_ptr, m,
                                               self.epilogue, L.PATH_AUTO))
            return
        _check_rc(lib.fnn_cuda_qmatmul_allgather(
            b.ctx, self.weight.handle, a_dev_ptr, self.bias_ptr, m, self.epilogue, self.rank, self.world,
            self.pa.peers, self.out_off, self.ctr_off, self.n, self.col0))

    def close(self) -> None:
        self.weight.close()


class ColumnShardedLinear:
    """One rank's shard of a quantized Linear on its GPU plus a collective all-gather of the outputs
    (`torch.distributed.all_gather_into_tensor`, NCCL on GPUs): the plain version of
    `AllGatherLinear`, kept as the baseline it is measured against and for shards of unequal width.

    `forward(x)` takes a replicated f32 CUDA tensor [M, K] (M <= m_max) and returns the full [M, N]
    on every rank.  Every buffer is allocated once; the GEMM, the collective and the one copy that
    turns the gathered [ranks][M][N/ranks] blocks into [M][N] rows all run on the backend's stream,
    which the caller's current stream waits for."""

    def __init__(self, backend, payload: bytes, meta: QuantizedWeightMeta, rank: int, world: int,
                 epilogue: int = L.EPI_NONE, group=None, m_max: int = 64):
        import torch  # plumbing: device tensors and torch.distributed
        self.torch, self.backend, self.group = torch, backend, group
        self.rank, self.world, self.epilogue, self.m_max = rank, world, epilogue, m_max
        self.bounds = shard_bounds(meta.shape[0], world)
        self.n, self.k = meta.shape
        sub_payload, sub_meta = shard_rows(payload, meta, rank, world)
        self.n_local = sub_meta.shape[0]
        self.n_max = max(b - a for a, b in self.bounds)
        self.weight = backend.upload_qweight(sub_payload, sub_meta)
        dev = torch.device("cuda", backend.device)
        self.stream = torch.cuda.ExternalStream(int(backend.lib.fnn_cuda_ctx_stream(backend.ctx) or 0), device=dev)
        self.shard_out = torch.zeros((m_max, self.n_local), dtype=torch.float32, device=dev)
        self.local = torch.zeros((m_max, self.n_max), dtype=torch.float32, device=dev)
        self.gathered = torch.zeros((world, m_max, self.n_max), dtype=torch.float32, device=dev)
        self.out = torch.zeros((m_max, self.n), dtype=torch.float32, device=dev)

    def forward(self, x):
        import torch.distributed as dist
        torch = self.torch
        m = x.shape[0]
        if m > self.m_max or not x.is_contiguous():
            raise BackendError("Dispatch", f"activations must be contiguous with at most {self.m_max} rows")
        caller = torch.cuda.current_stream()
        self.stream.wait_stream(caller)          # x was produced on the caller's stream
        with torch.cuda.stream(self.stream):
            rc = self.backend.lib.fnn_cuda_qmatmul_ptr(self.backend.ctx, self.weight.handle, x.data_ptr(),
                                                       self.shard_out.data_ptr(), None, m, self.epilogue,
                                                       L.PATH_AUTO)
            if rc != 0:
                raise BackendError.from_status(rc)
            self.local[:m, : self.n_local].copy_(self.shard_out.view(-1)[: m * self.n_local].view(m, self.n_local))
            dist.all_gather_into_tensor(self.gathered, self.local, group=self.group)
            for r, (a, b) in enumerate(self.bounds):
                self.out[:m, a:b].copy_(self.gathered[r, :m, : b - a])
        caller.wait_stream(self.stream)
        return self.out[:m]


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
        self.pa = PeerArena(backend, self.a_off + m_max * meta.shape[1] * 4, rank, world, group)
        self.arena, self.peer_ptrs = self.pa.arena, self.pa.peers
        self.calls = 0

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
        self.weight.close()
        self.pa.close()


def _check_rc(rc: int) -> None:
    if rc != 0:
        raise BackendError.from_status(rc)
