"""Host logic of the multi-GPU path on CPU: row sharding of a quantized weight and the column
re-assembly after an all-gather, with two `gloo` ranks.  The per-shard compute is done by the CPU
oracle here (the product has no CPU path); what is under test is that shards are byte-identical to
the matching rows of the single-GPU weight and that gather + assembly reproduce the unsharded result."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200.parallel import assemble_columns, shard_bounds, shard_rows
from helpers import normal


def _meta(q):
    return fnn.QuantizedWeightMeta(bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros,
                                   shape=[q.n, q.k], quant_block_size=q.quant_block_size,
                                   codebooks=[q.codebook] if q.codebook is not None else [], fmt=q.fmt)


def _as_qweight(payload, meta):
    return orc.QWeight(meta.fmt, meta.shape[0], meta.shape[1], np.frombuffer(payload, np.uint32),
                       np.asarray(meta.scales, np.float32), np.asarray(meta.zero_points, np.float32),
                       meta.codebooks[0] if meta.codebooks else None, meta.quant_block_size)


def test_shard_bounds_cover_all_rows():
    assert shard_bounds(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert shard_bounds(11008, 8)[-1] == (9632, 11008)
    assert shard_bounds(3, 8)[3:] == [(3, 3)] * 5


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
def test_shards_are_the_rows_of_the_unsharded_weight(fmt):
    k, n, world = 96, 22, 4
    q = orc.quantize_kn(fmt, normal(7 + fmt, (k, n), 0.02))
    x = normal(8, (3, k), 1.0)
    full = orc.qmatmul(q, x)
    parts = []
    for r in range(world):
        payload, meta = shard_rows(q.payload, _meta(q), r, world)
        n0, n1 = shard_bounds(n, world)[r]
        kp = -(-k // (4 if fmt in (orc.FMT_I8, orc.FMT_F8) else 8))
        assert payload[: (n1 - n0) * kp * 4] == q.payload[n0 * kp * 4: n1 * kp * 4]
        assert len(payload) == ((n1 - n0) * kp + 16) * 4 and not any(payload[-64:])
        parts.append(orc.qmatmul(_as_qweight(payload, meta), x))
    assert np.array_equal(assemble_columns(parts), full)


def _rank_main(rank, world, port, fmt, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        k, n, m = 64, 40, 5
        q = orc.quantize_kn(fmt, normal(21, (k, n), 0.02))       # every rank quantizes the same seed
        x = normal(22, (m, k), 1.0)                              # replicated activations
        payload, meta = shard_rows(q.payload, _meta(q), rank, world)
        local = torch.from_numpy(orc.qmatmul(_as_qweight(payload, meta), x, None, orc.EPI_SILU))
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        full = assemble_columns([g.numpy() for g in gathered])
        want = orc.qmatmul(q, x, None, orc.EPI_SILU)
        ret[rank] = bool(np.array_equal(full, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", [orc.FMT_I8, orc.FMT_I4CB])
def test_two_gloo_ranks_gather_the_unsharded_result(fmt):
    world = 2
    port = 29500 + (os.getpid() % 1000) + fmt
    manager = mp.get_context("spawn").Manager()
    ret = manager.dict()
    mp.spawn(_rank_main, args=(world, port, fmt, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
