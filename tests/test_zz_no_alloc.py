"""fnn_cuda_qmatmul_noalloc: the quantized MatMul for hosts that forbid device allocations in
the call (their own allocator owns all device memory, or the call sits in a loop where a
cudaMalloc-induced device synchronization is not acceptable).

The entry point keeps its activation scratch in an array inside the library image instead of
growing the context's scratch buffer.  Checked here through the C ABI against the regular
entry point on the same inputs, on two calls in a row: the second call is smaller than the
first, so it only passes if stale scratch contents from the first call are handled.  A second test
checks the property the entry point is named for: free device memory does not move across a call,
and the context's own scratch buffer is still empty afterwards.

The file name sorts last so that a run that stops at the first failure (-x) has already run
every other test when it gets here; the tests also pass when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200 import _lib as L
from helpers import max_err_vs_rms, normal

pytestmark = pytest.mark.gpu


def _device_rig(backend, q, m_max):
    al = lambda x: -(-x // 256) * 256
    a_off, out_off = 0, al(m_max * q.k * 4)
    ref_off = out_off + al(m_max * q.n * 4)
    bias_off = ref_off + al(m_max * q.n * 4)
    arena = backend.allocate_arena(bias_off + al(q.n * 4))
    meta = fnn.QuantizedWeightMeta(bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros,
                                   shape=[q.n, q.k], fmt=q.fmt, quant_block_size=q.quant_block_size,
                                   codebooks=[q.codebook] if q.codebook is not None else [])
    w = backend.upload_qweight(q.payload, meta)
    return arena, w, (a_off, out_off, ref_off, bias_off)


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
def test_noalloc_entry_matches_regular_entry_on_two_calls(backend, fmt):
    lib = backend.lib
    k, n = 1024, 384
    q = orc.quantize_kn(fmt, normal(900 + fmt, (k, n), 0.02))
    bias = normal(901, (n,), 0.01)
    arena, w, (a_off, out_off, ref_off, bias_off) = _device_rig(backend, q, 200)
    base = arena.device_ptr
    try:
        backend.write_arena(arena, bias_off, bias.tobytes())
        for m, epi, use_bias in ((200, L.EPI_GELU, True), (3, L.EPI_SILU, False)):
            x = normal(910 + m, (m, k), 1.0)
            backend.write_arena(arena, a_off, x.tobytes())
            b_ptr = base + bias_off if use_bias else None
            rc = lib.fnn_cuda_qmatmul_noalloc(backend.ctx, w.handle, base + a_off, base + out_off,
                                              b_ptr, m, epi)
            assert rc == 0, L.last_error()
            assert backend.last_path() == "tc-noalloc"
            rc = lib.fnn_cuda_qmatmul_ptr(backend.ctx, w.handle, base + a_off, base + ref_off,
                                          b_ptr, m, epi, L.PATH_TC)
            assert rc == 0, L.last_error()
            backend.synchronize()
            got = np.frombuffer(backend.read_arena(arena, out_off, m * n * 4), np.float32).reshape(m, n)
            ref = np.frombuffer(backend.read_arena(arena, ref_off, m * n * 4), np.float32).reshape(m, n)
            # same kernel, same arithmetic; the regular entry point may split a tile's K range over
            # several CTAs, which changes the order of the f32 additions only
            assert max_err_vs_rms(got, ref) <= 1e-5
            want = orc.qmatmul(q, x, bias if use_bias else None, epi)
            assert max_err_vs_rms(got, want) <= 1e-2
    finally:
        w.close()
        arena.close()


def test_noalloc_entry_leaves_device_memory_and_context_scratch_untouched():
    """On a fresh context (no scratch yet): after the first call per device (which loads the
    module and looks up the array's address) a call moves cudaMemGetInfo's free bytes by nothing,
    and a regular tcgen05 call of the same size inside a capture still reports that the context's
    scratch would have to grow -- so the entry point did not grow it behind the caller's back."""
    import torch
    fresh = fnn.CudaBackend(0)
    lib = fresh.lib
    k, n, m = 1024, 256, 64
    q = orc.quantize_kn(orc.FMT_I8, normal(930, (k, n), 0.02))
    arena, w, (a_off, out_off, _, _) = _device_rig(fresh, q, m)
    base = arena.device_ptr
    try:
        fresh.write_arena(arena, a_off, normal(931, (m, k), 1.0).tobytes())
        call = lambda: lib.fnn_cuda_qmatmul_noalloc(fresh.ctx, w.handle, base + a_off, base + out_off,
                                                    None, m, L.EPI_NONE)
        assert call() == 0, L.last_error()          # first call on the device: set-up happens here
        fresh.synchronize()
        free_before = torch.cuda.mem_get_info(0)[0]
        assert call() == 0, L.last_error()
        fresh.synchronize()
        assert torch.cuda.mem_get_info(0)[0] == free_before
        assert lib.fnn_cuda_graph_begin(fresh.ctx) == 0
        rc = lib.fnn_cuda_qmatmul_ptr(fresh.ctx, w.handle, base + a_off, base + out_off, None, m,
                                      L.EPI_NONE, L.PATH_TC)
        msg = L.last_error()
        g = ctypes.c_void_p()
        assert lib.fnn_cuda_graph_end(fresh.ctx, ctypes.byref(g)) == 0
        lib.fnn_cuda_graph_free(g)
        assert rc == 3 and "scratch buffer must grow" in msg
    finally:
        w.close()
        arena.close()
        fresh.close()


def test_noalloc_entry_refuses_what_does_not_fit_or_is_not_served(backend):
    lib = backend.lib
    q8 = orc.quantize_kn(orc.FMT_I8, normal(920, (8192, 128), 0.02))
    arena, w, (a_off, out_off, _, _) = _device_rig(backend, q8, 1)
    base = arena.device_ptr
    try:
        # 2 planes x 1024 rows x 8192 bytes = 16 MiB of rewritten activations: beyond the 8 MiB array
        rc = lib.fnn_cuda_qmatmul_noalloc(backend.ctx, w.handle, base + a_off, base + out_off, None,
                                          1024, L.EPI_NONE)
        assert rc == 3 and "built-in" in L.last_error()
    finally:
        w.close()
        arena.close()
    # the codebook format needs whole groups of four scale blocks per row (K a multiple of 128)
    qc = orc.quantize_kn(orc.FMT_I4CB, normal(922, (160, 128), 0.02))
    meta = fnn.QuantizedWeightMeta(bit_width=4, scales=qc.scales, zero_points=qc.zeros, shape=[qc.n, qc.k],
                                   quant_block_size=32, codebooks=[qc.codebook], fmt=qc.fmt)
    wc = backend.upload_qweight(qc.payload, meta)
    arena = backend.allocate_arena(1 << 20)
    try:
        rc = lib.fnn_cuda_qmatmul_noalloc(backend.ctx, wc.handle, arena.device_ptr, arena.device_ptr + 4096,
                                          None, 1, L.EPI_NONE)
        assert rc == 4 and "not served" in L.last_error()
    finally:
        wc.close()
        arena.close()
