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
