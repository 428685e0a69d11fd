"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Bars: packed bytes and dequantized weights bit-exact; outputs within 1e-3 (max error relative to
the RMS of the reference output) for every configuration of 32 batch rows or fewer whatever kernel
family automatic dispatch picks, and on the tcgen05 kernel wherever it carries the activations as
int8 pairs or e4m3 triples; 1e-2 on the tcgen05 kernel from 128 batch rows on for the e4m3
formats (two activation terms) and for the codebook format (fp16 operands).
"""
import ctypes
import os

import numpy as np
import pytest

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200 import _lib as L
from helpers import max_err_vs_rms, normal

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-3   # every skinny configuration; f32-grade operand splits on the tensor cores
TOL_TC = 1e-2    # tcgen05 with two e4m3 terms (M >= 128) or fp16 operands (codebook format)
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qmatmul_small.npz")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def meta_of(q: orc.QWeight) -> fnn.QuantizedWeightMeta:
    return fnn.QuantizedWeightMeta(
        bit_width=q.bit_width, scales=q.scales, zero_points=q.zeros, shape=[q.n, q.k],
        quant_block_size=q.quant_block_size,
        codebooks=[q.codebook] if q.codebook is not None else [], fmt=q.fmt)


class Rig:
    """Arena with [activation | output | bias | dequant] slots around one uploaded weight."""

    def __init__(self, backend, q: orc.QWeight, m: int):
        self.b, self.q, self.m = backend, q, m
        al = lambda x: -(-x // 256) * 256
        self.a_off = 0
        self.out_off = al(m * q.k * 4)
        self.bias_off = self.out_off + al(m * q.n * 4)
        self.deq_off = self.bias_off + al(q.n * 4)
        self.arena = backend.allocate_arena(self.deq_off + al(q.n * q.k * 4))
        self.w = backend.upload_qweight(q.payload, meta_of(q))

    def run(self, x, bias=None, epi=L.EPI_NONE, path=L.PATH_AUTO):
        b = self.b
        b.write_arena(self.arena, self.a_off, np.ascontiguousarray(x, np.float32).tobytes())
        if bias is not None:
            b.write_arena(self.arena, self.bias_off, np.ascontiguousarray(bias, np.float32).tobytes())
        rc = b.lib.fnn_cuda_qmatmul(b.ctx, self.w.handle, self.arena.handle, self.a_off, self.out_off,
                                    self.bias_off if bias is not None else -1, x.shape[0], epi, path)
        if rc != 0:
            raise fnn.BackendError.from_status(rc)
        raw = b.read_arena(self.arena, self.out_off, x.shape[0] * self.q.n * 4)
        return np.frombuffer(raw, np.float32).reshape(x.shape[0], self.q.n)

    def dequant(self):
        b = self.b
        rc = b.lib.fnn_cuda_qweight_dequant(self.w.handle, self.arena.handle, self.deq_off)
        assert rc == 0, L.last_error()
        raw = b.read_arena(self.arena, self.deq_off, self.q.n * self.q.k * 4)
        return np.frombuffer(raw, np.float32).reshape(self.q.n, self.q.k)

    def close(self):
        self.w.close()
        self.arena.close()


SHAPES = [(64, 16), (45, 7), (256, 40), (1000, 33), (4096, 64), (31, 1), (8, 257)]


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
@pytest.mark.parametrize("kn", SHAPES)
def test_repack_preserves_every_bit_and_dequant_is_bit_exact(backend, fmt, kn):
    k, n = kn
    w = normal(10 + k + n, (k, n), 0.02)
    w[:, 0] = 0.5
    q = orc.quantize_kn(fmt, w)
    rig = Rig(backend, q, 1)
    try:
        assert rig.w.unrepack() == q.payload
        assert np.array_equal(bits(rig.dequant()), bits(orc.dequant(q)))
    finally:
        rig.close()


def test_dequant_all_codes_bit_exact(backend):
    """Every 8-bit and 4-bit code, not only those the quantizer emits (e4m3 exponent 15 ->
    NaN, e2m1 0x8 -> +0)."""
    for fmt, nwords in ((orc.FMT_F8, 64), (orc.FMT_I8, 64), (orc.FMT_F4, 2), (orc.FMT_I4, 2)):
        items = 4 if nwords == 64 else 8
        codes = np.arange(256 if items == 4 else 16, dtype=np.uint32)
        shift = 8 if items == 4 else 4
        words = np.zeros(nwords + 16, np.uint32)
        for i, c in enumerate(codes):
            words[i // items] |= c << (shift * (i % items))
        q = orc.QWeight(fmt, 1, len(codes), words, np.array([0.75], np.float32),
                        np.array([0.0 if fmt == orc.FMT_F8 else 0.125], np.float32))
        rig = Rig(backend, q, 1)
        try:
            got, want = rig.dequant(), orc.dequant(q)
            same = (bits(got) == bits(want)) | (np.isnan(got) & np.isnan(want))
            assert same.all(), (fmt, np.nonzero(~same))
        finally:
            rig.close()


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
@pytest.mark.parametrize("kn", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 19])
def test_rows_kernel_parity(backend, fmt, kn, m):
    k, n = kn
    w = normal(20 + k + n, (k, n), 0.02)
    x = normal(30 + m, (m, k), 1.0)
    bias = normal(40 + n, (n,), 0.01)
    q = orc.quantize_kn(fmt, w)
    rig = Rig(backend, q, m)
    try:
        for b, epi in ((None, L.EPI_NONE), (bias, L.EPI_NONE), (bias, L.EPI_GELU), (None, L.EPI_SILU),
                       (bias, L.EPI_RELU)):
            got = rig.run(x, b, epi, L.PATH_ROWS)
            want = orc.qmatmul(q, x, b, epi)
            assert max_err_vs_rms(got, want) <= TOL_F32, (fmt, kn, m, epi)
        assert backend.last_path() == "rows"
    finally:
        rig.close()


def test_golden_vectors_on_device(backend):
    g = np.load(GOLDEN)
    for case in ("aligned", "ragged", "wide"):
        x, bias = g[f"{case}/x"], g[f"{case}/bias"]
        for fmt, name in orc.FMT_NAMES.items():
            p = f"{case}/{name}"
            cb = g[p + "/codebook"] if fmt == orc.FMT_I4CB else None
            k, n = g[f"{case}/w_kn"].shape
            q = orc.QWeight(fmt, n, k, g[p + "/words"], g[p + "/scales"], g[p + "/zeros"], cb,
                            32 if fmt == orc.FMT_I4CB else 0)
            rig = Rig(backend, q, x.shape[0])
            try:
                assert np.array_equal(bits(rig.dequant()), bits(g[p + "/dequant"])), p
                assert max_err_vs_rms(rig.run(x), g[p + "/out_plain"]) <= TOL_F32, p
                assert max_err_vs_rms(rig.run(x, bias, L.EPI_GELU), g[p + "/out_bias_gelu"]) <= TOL_F32, p
                assert max_err_vs_rms(rig.run(x, None, L.EPI_SILU), g[p + "/out_silu"]) <= TOL_F32, p
            finally:
                rig.close()


def test_exact_integer_kat_on_device(backend):
    """microkernels/tests.rs:504-533: zero point contributes zero * sum(input)."""
    q = orc.from_f32_slice(orc.FMT_I8, [12.0, 14.0, 16.0, 18.0], 1, 4, 2.0, 10.0)
    rig = Rig(backend, q, 2)
    try:
        out = rig.run(np.array([[1.0, 2.0, 3.0, 4.0], [-1.0, 0.5, 2.0, -3.0]], np.float32))
        assert abs(out[0, 0] - 160.0) < 1e-4 and abs(out[1, 0] - (-27.0)) < 1e-4
    finally:
        rig.close()


def test_per_tensor_and_grouped_metadata_are_broadcast(backend):
    w = normal(3, (8, 64), 0.02)  # [N,K]
    q = orc.quantize_nk(orc.FMT_I8, w)
    # one scale/zero per group of 4 rows: rows % n_scales == 0 (matmul.rs:108-113)
    grouped = orc.QWeight(orc.FMT_I8, 8, 64, q.words, q.scales[::4].copy(), q.zeros[::4].copy())
    full = orc.QWeight(orc.FMT_I8, 8, 64, q.words, np.repeat(grouped.scales, 4),
                       np.repeat(grouped.zeros, 4))
    x = normal(4, (2, 64), 1.0)
    rig = Rig(backend, grouped, 2)
    try:
        assert max_err_vs_rms(rig.run(x), orc.qmatmul(full, x)) <= TOL_F32
    finally:
        rig.close()


@pytest.mark.parametrize("fmt,m,epi", [(orc.FMT_I4, 8, L.EPI_NONE),      # config 1 (+bias)
                                       (orc.FMT_I4, 1, L.EPI_NONE),
                                       (orc.FMT_I8, 1, L.EPI_SILU),      # config 2
                                       (orc.FMT_I8, 4, L.EPI_SILU),
                                       (orc.FMT_I8, 16, L.EPI_SILU)])
def test_baseline_config_sizes_against_oracle(backend, fmt, m, epi):
    k, n = (4096, 4096) if fmt == orc.FMT_I4 else (4096, 11008)
    w = normal(0, (k, n), 0.02)
    x = normal(1, (m, k), 1.0)
    bias = normal(2, (n,), 0.01) if fmt == orc.FMT_I4 else None
    packed, scales, zeros, cb = fnn.quantize_weight_constant(w, fmt)   # library host pass
    q = orc.QWeight(fmt, n, k, np.frombuffer(packed.tobytes(), np.uint32), scales, zeros)
    rig = Rig(backend, q, m)
    try:
        got = rig.run(x, bias, epi)
        want = orc.qmatmul(q, x, bias, epi)
        assert max_err_vs_rms(got, want) <= TOL_F32, backend.last_path()   # whatever kernel ran
    finally:
        rig.close()


@pytest.mark.parametrize("fmt", [orc.FMT_F8, orc.FMT_F4])
def test_config3_full_size_row_slices_and_linearity(backend, fmt):
    """K=8192, N=28672 (Llama-style FFN).  Output columns are independent, so the oracle checks
    random column slices exactly; linearity in the activations covers the whole output."""
    k, n, m = 8192, 28672, 2
    w = normal(7, (k, n), 0.015)
    packed, scales, zeros, _ = fnn.quantize_weight_constant(w, fmt)
    words = np.frombuffer(packed.tobytes(), np.uint32)
    q = orc.QWeight(fmt, n, k, words, scales, zeros if fmt == orc.FMT_F4 else np.zeros(0, np.float32))
    x1, x2 = normal(8, (m, k), 1.0), normal(9, (m, k), 1.0)
    rig = Rig(backend, q, m)
    try:
        y1, y2, y12 = rig.run(x1).copy(), rig.run(x2).copy(), rig.run(x1 + x2).copy()
        scale = np.sqrt(np.mean(y12.astype(np.float64) ** 2))
        assert np.max(np.abs(y12 - (y1 + y2))) <= 2e-3 * scale
        kp = k // (4 if fmt == orc.FMT_F8 else 8)
        rows = np.concatenate([np.arange(0, 64), np.arange(14000, 14064), np.arange(n - 64, n)])
        sub_words = np.concatenate([words[: n * kp].reshape(n, kp)[rows].reshape(-1),
                                    np.zeros(16, np.uint32)])
        sub = orc.QWeight(fmt, len(rows), k, sub_words, scales[rows],
                          zeros[rows] if fmt == orc.FMT_F4 else np.zeros(0, np.float32))
        assert max_err_vs_rms(y1[:, rows], orc.qmatmul(sub, x1)) <= TOL_F32, backend.last_path()
    finally:
        rig.close()


# ---- error behaviour: BackendError::Dispatch with the reference's messages --------------------------

def _upload_raises(backend, q, meta, match):
    with pytest.raises(fnn.BackendError, match=match):
        backend.upload_qweight(q.payload, meta)


def test_metadata_validation_matches_packed_tensor_from_meta(backend):
    q = orc.quantize_nk(orc.FMT_I8, normal(1, (6, 32), 0.02))
    m = meta_of(q)
    m.scales = np.zeros(0, np.float32)
    _upload_raises(backend, q, m, "missing scales")
    m = meta_of(q)
    m.zero_points = q.zeros[:3]
    _upload_raises(backend, q, m, "length mismatch")
    m = meta_of(q)
    m.scales, m.zero_points = q.scales[:4], q.zeros[:4]   # 6 % 4 != 0
    _upload_raises(backend, q, m, "incompatible with shape")
    m = meta_of(q)
    with pytest.raises(fnn.BackendError, match="payload too short"):
        backend.upload_qweight(q.payload[:40], m)
    m = meta_of(q)
    m.fmt = 9
    _upload_raises(backend, q, m, "unknown format")


def test_out_of_range_slices_are_rejected(backend):
    q = orc.quantize_nk(orc.FMT_I8, normal(1, (16, 64), 0.02))
    rig = Rig(backend, q, 1)
    try:
        lib = backend.lib
        rc = lib.fnn_cuda_qmatmul(backend.ctx, rig.w.handle, rig.arena.handle, 0,
                                  rig.arena.total_bytes - 16, -1, 1, 0, 0)
        assert rc == 2 and "outside arena" in L.last_error()
        rc = lib.fnn_cuda_qmatmul(backend.ctx, rig.w.handle, rig.arena.handle, 0, rig.out_off, -1, 1, 7, 0)
        assert rc == 2 and "epilogue" in L.last_error()
        rc = lib.fnn_cuda_qmatmul(backend.ctx, rig.w.handle, rig.arena.handle, 4, rig.out_off, -1, 1, 0, 0)
        assert rc == 2 and "aligned" in L.last_error()
        # write_arena has no Result: the error is latched and raised by the next dispatch
        backend.write_arena(rig.arena, rig.arena.total_bytes - 4, b"\0" * 64)
        with pytest.raises(fnn.BackendError, match="out of range"):
            backend.dispatch(fnn.ExecutablePlan([], 0), rig.arena, fnn.ShapeEnv())
    finally:
        rig.close()


def test_arena_is_zero_filled_and_round_trips(backend):
    arena = backend.allocate_arena(4096 + 12)
    try:
        assert backend.read_arena(arena, 0, 4108) == bytes(4108)
        data = bytes(range(256)) * 4
        backend.write_arena(arena, 64, data)
        assert backend.read_arena(arena, 64, 1024) == data
    finally:
        arena.close()


def test_elementwise_fill_memcpy(backend):
    lib = backend.lib
    arena = backend.allocate_arena(3 * 4096)
    try:
        a, b = normal(1, (1024,), 1.0), normal(2, (32,), 1.0)
        backend.write_arena(arena, 0, a.tobytes())
        backend.write_arena(arena, 4096, b.tobytes())
        for op, f in ((L.EW_ADD, lambda u, v: u + v), (L.EW_MUL, lambda u, v: u * v),
                      (L.EW_SUB, lambda u, v: u - v)):
            assert lib.fnn_cuda_elementwise(backend.ctx, op, arena.handle, 0, 1024, 4096, 32, 8192, 1024) == 0
            got = np.frombuffer(backend.read_arena(arena, 8192, 4096), np.float32)
            assert np.array_equal(got, f(a, np.tile(b, 32)))  # broadcast by modulo, exact f32 op
        op = L.EW_ADD | (L.EPI_GELU << 8)   # add_gelu_f32, in place on a
        assert lib.fnn_cuda_elementwise(backend.ctx, op, arena.handle, 0, 1024, 4096, 32, 0, 1024) == 0
        got = np.frombuffer(backend.read_arena(arena, 0, 4096), np.float32)
        want = orc.epilogue(a.reshape(1, -1), 32, b, orc.EPI_GELU).ravel()
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
        assert lib.fnn_cuda_fill(backend.ctx, arena.handle, 8192, 4096, 2.5) == 0
        assert lib.fnn_cuda_memcpy(backend.ctx, arena.handle, 4096, 8192, 2048) == 0
        got = np.frombuffer(backend.read_arena(arena, 4096, 2048), np.float32)
        assert np.all(got == 2.5)
        assert lib.fnn_cuda_elementwise(backend.ctx, 77, arena.handle, 0, 4, 0, 4, 0, 4) == 4
    finally:
        arena.close()


def test_graph_replay_and_launch_count(backend):
    q = orc.quantize_nk(orc.FMT_I4, normal(1, (32, 128), 0.02))
    rig = Rig(backend, q, 4)
    lib = backend.lib
    try:
        x = normal(2, (4, 128), 1.0)
        want = rig.run(x).copy()                      # warm (allocations happen outside capture)
        before = backend.launch_count()
        assert lib.fnn_cuda_graph_begin(backend.ctx) == 0
        for _ in range(3):
            assert lib.fnn_cuda_qmatmul(backend.ctx, rig.w.handle, rig.arena.handle, rig.a_off,
                                        rig.out_off, -1, 4, 0, 0) == 0
        g = ctypes.c_void_p()
        assert lib.fnn_cuda_graph_end(backend.ctx, ctypes.byref(g)) == 0
        assert backend.launch_count() == before       # captured, not executed
        assert lib.fnn_cuda_fill(backend.ctx, rig.arena.handle, rig.out_off, 4 * 32 * 4, 0.0) == 0
        assert lib.fnn_cuda_graph_launch(backend.ctx, g) == 0
        backend.synchronize()
        assert backend.launch_count() == before + 1 + 3
        got = np.frombuffer(backend.read_arena(rig.arena, rig.out_off, 4 * 32 * 4), np.float32)
        assert np.array_equal(got.reshape(4, 32), want)
        lib.fnn_cuda_graph_free(g)
    finally:
        rig.close()


# ---- skinny tensor-core kernel (fragment-major weights, mma.sync, fp16 hi/lo activations) ------------

MMA_SHAPES = [(512, 64), (4096, 256), (1000, 33), (45, 7), (640, 1040), (8192, 96), (2048, 272)]


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
@pytest.mark.parametrize("kn", MMA_SHAPES)
def test_mma_kernel_parity(backend, fmt, kn):
    k, n = kn
    w = normal(50 + k + n, (k, n), 0.02)
    bias = normal(60 + n, (n,), 0.01)
    q = orc.quantize_kn(fmt, w)
    ms = [1, 2, 4, 5, 8, 13, 16, 17, 32, 33, 64, 65, 100]
    rig = Rig(backend, q, max(ms))
    try:
        for m in ms:
            x = normal(70 + m, (m, k), 1.0)
            b, epi = ((bias, L.EPI_GELU) if m % 2 else (None, L.EPI_SILU))
            got = rig.run(x, b, epi, L.PATH_MMA)
            assert backend.last_path() in ("mma", "mma8")
            want = orc.qmatmul(q, x, b, epi)
            # up to 32 rows every format is f32-grade: int8 activation pairs up to 16 rows for the
            # integer-valued formats (the codebook format at any M, 16 rows at a time), fp16 hi + lo
            # terms otherwise; beyond 32 rows the fp16 kernel keeps one term (the tcgen05 kernel
            # is the intended path there)
            tol = TOL_F32 if (m <= 32 or fmt == orc.FMT_I4CB) else TOL_TC
            err = max_err_vs_rms(got, want)
            assert err <= tol, (orc.FMT_NAMES[fmt], kn, m, err)
        backend.synchronize()
    finally:
        rig.close()


def test_mma_kernel_is_deterministic(backend):
    q = orc.quantize_kn(orc.FMT_I4, normal(1, (4096, 512), 0.02))
    rig = Rig(backend, q, 4)
    try:
        x = normal(2, (4, 4096), 1.0)
        a = rig.run(x, None, L.EPI_NONE, L.PATH_MMA).copy()
        for _ in range(3):
            assert np.array_equal(a, rig.run(x, None, L.EPI_NONE, L.PATH_MMA))
    finally:
        rig.close()


@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
@pytest.mark.parametrize("m", [1, 6])
def test_fragment_kernels_take_any_activation_magnitude(backend, fmt, m):
    """Rows are rescaled by a power of two (fp16 operands) or by their maximum (int8 pairs) before
    they are narrowed: 1e6, 1e-6 and a row of mixed magnitudes give the oracle's answer."""
    q = orc.quantize_kn(fmt, normal(1, (512, 64), 0.02))
    rig = Rig(backend, q, m)
    try:
        for scale in (1e6, 1e-6, 1.0):
            x = normal(2, (m, 512), scale)
            x[0, 3] = 12.0 * scale   # a heavy-tailed element; the int8 pairs resolve 1/16256 of the row maximum
            got = rig.run(x, None, L.EPI_NONE, L.PATH_MMA)
            backend.synchronize()
            assert max_err_vs_rms(got, orc.qmatmul(q, x)) <= TOL_F32, (fmt, m, scale)
    finally:
        rig.close()


# ---- tcgen05 / TMEM / TMA kernel (native I8 and FP8 codes) ---------------------------------------------

TC_SHAPES = [(128, 128), (4096, 256), (1000, 200), (512, 1040), (8192, 384)]


@pytest.mark.parametrize("fmt", [orc.FMT_I8, orc.FMT_F8, orc.FMT_I4, orc.FMT_F4, orc.FMT_I4CB])
@pytest.mark.parametrize("kn", TC_SHAPES)
def test_tcgen05_kernel_parity(backend, fmt, kn):
    k, n = kn
    if fmt == orc.FMT_I4CB and k % 128:
        pytest.skip("the codebook format's block scales reach the tcgen05 kernel four per row and stage")
    w = normal(150 + k + n, (k, n), 0.02)
    bias = normal(160 + n, (n,), 0.01)
    q = orc.quantize_kn(fmt, w)
    ms = [1, 5, 16, 100, 128, 300, 512]
    rig = Rig(backend, q, max(ms))
    try:
        for m in ms:
            x = normal(170 + m, (m, k), 1.0)
            b, epi = ((bias, L.EPI_GELU) if m % 2 else (None, L.EPI_SILU))
            got = rig.run(x, b, epi, L.PATH_TC)
            backend.synchronize()  # a bounded wait that gave up would raise here
            assert backend.last_path() == "tc"
            want = orc.qmatmul(q, x, b, epi)
            err = max_err_vs_rms(got, want)
            # int8 pairs and e4m3 triples of the activations are f32-grade; from 128 batch rows
            # on the e4m3 formats use two terms (tensor-core tolerance)
            # (the codebook format runs on an fp16 copy with one fp16 activation term)
            tol = TOL_TC if ((m >= 128 and fmt in (orc.FMT_F8, orc.FMT_F4)) or fmt == orc.FMT_I4CB) \
                else TOL_F32
            assert err <= tol, (orc.FMT_NAMES[fmt], kn, m, err)
    finally:
        rig.close()


def test_tcgen05_path_rejects_shapes_it_does_not_cover(backend):
    q = orc.quantize_kn(orc.FMT_I8, normal(1, (64, 128), 0.02))   # K below one 128-byte swizzle row
    rig = Rig(backend, q, 1)
    try:
        with pytest.raises(fnn.BackendError, match="tcgen05 path does not cover"):
            rig.run(normal(2, (1, 64), 1.0), None, L.EPI_NONE, L.PATH_TC)
    finally:
        rig.close()
