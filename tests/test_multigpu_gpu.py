"""Column-sharded quantized Linear on 2 / 4 / 8 GPUs: the fused GEMV + peer-store all-gather kernel
(up to four batch rows), the fused GEMM + all-gather on the tcgen05 kernel (any batch size, two
layers chained) and the NCCL all-gather wrapper must all reproduce the unsharded oracle result on
every rank.  Needs that many CUDA devices (skipped otherwise); one process per GPU."""
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
    from fastnn_b200.parallel import AllGatherLinear, ColumnShardedLinear, FusedGatherLinear, PeerArena
    from helpers import max_err_vs_rms, normal

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        backend = fnn.CudaBackend(rank)   # its own stream; the NCCL wrapper orders torch's stream against it
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
        # fused GEMM + all-gather on the tcgen05 kernel: two chained layers 1024 -> 1024 -> 1024, the
        # second reading the rows the first one gathered; several steps reuse the same buffers
        k = n = 1024
        al = lambda v: -(-v // 256) * 256
        m_max = 64
        x_off, o1_off = 0, al(m_max * k * 4)
        c1_off = o1_off + al(m_max * n * 4)
        o2_off, c2_off = c1_off + 256, c1_off + 256 + al(m_max * n * 4)
        b_off = c2_off + 256
        pa = PeerArena(backend, b_off + al(n * 4), rank, world)
        for fmt in (orc.FMT_I8, orc.FMT_I4, orc.FMT_F4):
            q1 = orc.quantize_kn(fmt, normal(80 + fmt, (k, n), 0.02))
            q2 = orc.quantize_kn(fmt, normal(90 + fmt, (n, n), 0.02))
            bias = normal(95, (n,), 0.01)
            mk = lambda q: fnn.QuantizedWeightMeta(bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros,
                                                   shape=[q.n, q.k], fmt=q.fmt)
            l1 = AllGatherLinear(backend, q1.payload, mk(q1), rank, world, pa, o1_off, c1_off, L.EPI_SILU,
                                 bias=bias, bias_off=b_off)
            l2 = AllGatherLinear(backend, q2.payload, mk(q2), rank, world, pa, o2_off, c2_off, L.EPI_NONE)
            for step, m in enumerate((64, 20, 64)):
                x = normal(100 + step, (m, k), 1.0)
                backend.write_arena(pa.arena, x_off, x.tobytes())
                l1.forward(pa.device_ptr + x_off, m)
                l2.forward(pa.device_ptr + o1_off, m)
                backend.synchronize()   # raises if a bounded wait gave up
                got = np.frombuffer(backend.read_arena(pa.arena, o2_off, m * n * 4), np.float32).reshape(m, n)
                h = orc.qmatmul(q1, x, bias, orc.EPI_SILU)
                ok = ok and max_err_vs_rms(got, orc.qmatmul(q2, h)) <= 2e-3
            l1.close()
            l2.close()
        pa.close()
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
