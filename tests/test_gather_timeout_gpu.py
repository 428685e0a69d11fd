"""Failure detection of the fused gather, injected on the host: a rank is told that it has a peer,
the peer never runs, so the words it should have stored never arrive.  The consumer-side poll must
give up after its bounded wait (about a second), report through fnn_cuda_sync, and leave the context
usable.  Nothing on the GPU faults or hangs: the poll simply runs out."""
import ctypes
import time

import numpy as np
import pytest

import oracle as orc
from helpers import max_err_vs_rms, normal

pytestmark = pytest.mark.gpu


def test_missing_peer_is_reported_and_context_survives():
    import fastnn_b200 as fnn
    from fastnn_b200 import _lib as L

    backend = fnn.CudaBackend(0)
    lib = backend.lib
    k, n, m = 1024, 512, 2
    q = orc.quantize_kn(orc.FMT_I8, normal(5, (k, n), 0.02))
    meta = fnn.QuantizedWeightMeta(bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros,
                                   shape=[q.n, q.k], fmt=q.fmt)
    w = backend.upload_qweight(q.payload, meta)
    world, rows = 2, 4
    words = 2 * world * rows * n * 8
    counter_off = words
    plain_off = counter_off + 256
    a_off = plain_off + world * rows * n * 4
    arena = backend.allocate_arena(a_off + m * k * 4)
    x = normal(6, (m, k), 1.0)
    backend.write_arena(arena, a_off, x.tobytes())
    # "rank 0 of 2" whose peer is a second view of its own buffer: rank 1's slots are never written
    peers = (ctypes.c_void_p * world)(arena.device_ptr, arena.device_ptr)
    rc = lib.fnn_cuda_qmatmul_gather(backend.ctx, w.handle, arena.device_ptr + a_off, None, m, L.EPI_NONE,
                                     0, world, peers, 0, counter_off, n)
    assert rc == 0
    backend.synchronize()          # the producer never waits: no error yet
    rc = lib.fnn_cuda_gather_wait(backend.ctx, arena.device_ptr, 0, counter_off, world, n,
                                  arena.device_ptr + plain_off)
    assert rc == 0
    t0 = time.time()
    with pytest.raises(fnn.BackendError) as e:
        backend.synchronize()
    waited = time.time() - t0
    assert "bounded wait" in str(e.value)
    assert 0.3 < waited < 10.0, waited
    # rank 0's own rows did arrive
    got = np.frombuffer(backend.read_arena(arena, plain_off, m * n * 4), np.float32).reshape(m, n)
    assert max_err_vs_rms(got, orc.qmatmul(q, x)) <= 1e-3
    # the flag is cleared by the report and the context keeps working
    backend.synchronize()
    out = backend.allocate_arena(m * n * 4)
    rc = lib.fnn_cuda_qmatmul_ptr(backend.ctx, w.handle, arena.device_ptr + a_off, out.device_ptr, None, m,
                                  L.EPI_NONE, L.PATH_AUTO)
    assert rc == 0
    backend.synchronize()
    got = np.frombuffer(backend.read_arena(out, 0, m * n * 4), np.float32).reshape(m, n)
    assert max_err_vs_rms(got, orc.qmatmul(q, x)) <= 1e-3
    out.close()
    arena.close()
    w.close()
    backend.close()
