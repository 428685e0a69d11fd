"""Column-sharded quantized Linear on 2 / 4 / 8 GPUs: the fused GEMV + peer-store all-gather kernel
and the NCCL all-gather wrapper must both reproduce the unsharded oracle result on every rank.
Needs that many CUDA devices (skipped otherwise); one process per GPU."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    import oracle as orc
    import fastnn_b200 as fnn
    from fastnn_b200 import _lib as L
    from fastnn_b200.parallel import ColumnShardedLinear, FusedGatherLinear
    from helpers import max_err_vs_rms, normal

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        backend = fnn.CudaBackend(rank, stream=torch.cuda.current_stream().cuda_stream)
        k, n = 1024, 1000   # 1000 columns: shards of 500, not a multiple of the 16-row tile
        for fmt in (orc.FMT_I8, orc.FMT_I4, orc.FMT_F8, orc.FMT_F4, orc.FMT_I4CB):
            q = orc.quantize_kn(fmt, normal(31 + fmt, (k, n), 0.02))
            meta = fnn.QuantizedWeightMeta(
                bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros, shape=[q.n, q.k], fmt=q.fmt,
                quant_block_size=32 if fmt == orc.FMT_I4CB else 0,
                codebooks=[q.codebook] if fmt == orc.FMT_I4CB else [])
            tol = 1e-3
            fused = FusedGatherLinear(backend, q.payload, meta, rank, world, m_max=4, epilogue=L.EPI_SILU)
            for step, m in enumerate((1, 3, 1, 2)):   # slots alternate, M changes between steps
                x = normal(40 + step, (m, k), 1.0)
                fused.set_activations(x)
                fused.forward()
                backend.synchronize()   # raises if a bounded wait gave up
                got = fused.gathered()
                want = orc.qmatmul(q, x, None, orc.EPI_SILU)
                ok = ok and got.shape == want.shape and max_err_vs_rms(got, want) <= tol
            # several steps in a row with nothing but the kernels' own polls between them
            x = normal(60, (2, k), 1.0)
            fused.set_activations(x)
            for _ in range(7):
                fused.forward()
            got = fused.gathered()
            backend.synchronize()
            ok = ok and max_err_vs_rms(got, orc.qmatmul(q, x, None, orc.EPI_SILU)) <= tol
            fused.close()
            # NCCL path for what the fused kernel does not serve (here: 16 batch rows)
            lin = ColumnShardedLinear(backend, q.payload, meta, rank, world, epilogue=L.EPI_NONE)
            x = normal(50, (16, k), 1.0)
            y = lin.forward(torch.from_numpy(x).cuda())
            torch.cuda.synchronize()
            ok = ok and max_err_vs_rms(y.cpu().numpy(), orc.qmatmul(q, x)) <= 1e-2
            lin.weight.close()
        backend.close()
    finally:
        ret[rank] = ok
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gather_and_nccl_gather(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 500) + world
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}
