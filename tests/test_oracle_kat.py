"""Pins the CPU oracle against the reference's own known-answer tests for this path.

Each test restates one `#[test]` of fastnn (cited by file:line) with the same inputs and
the same expectations.  The reference pins no packed bytes for random weights; these KATs
plus the bit-for-bit agreement with the NumPy twin (test_oracle_twin.py) are what anchors
the oracle.
"""
import math

import numpy as np
import pytest

import oracle as orc
from helpers import assert_close, seeded_values


# ---- src/dtypes/f4x8.rs:185-278 ---------------------------------------------------------

def test_fp4_to_f32_table():
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert [orc.fp4_to_f32(c) for c in range(8)] == want


def test_fp4_negative():
    v = orc.fp4_to_f32(0x8)
    assert v == 0.0 and math.copysign(1.0, v) == 1.0  # -0 is treated as +0
    assert orc.fp4_to_f32(0x9) == -0.5
    assert orc.fp4_to_f32(0xF) == -6.0


def test_f32_to_fp4_roundtrip():
    for v in [0.0, 0.5, 1.0, -1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -6.0, -0.5]:
        assert abs(orc.fp4_to_f32(orc.f32_to_fp4(v)) - v) < 0.01


def test_f32_to_fp4_clamp():
    c = orc.f32_to_fp4(100.0)
    assert c & 7 == 7 and orc.fp4_to_f32(c) == 6.0
    c = orc.f32_to_fp4(-100.0)
    assert c & 7 == 7 and orc.fp4_to_f32(c) == -6.0


def test_f32_to_fp4_ties_keep_lower_index_and_nan():
    # strict '<' in the search: 0.25 is equidistant from 0 and 0.5 -> index 0
    assert orc.f32_to_fp4(0.25) == 0
    assert orc.f32_to_fp4(2.5) == 4      # between 2 and 3 -> 2.0
    assert orc.f32_to_fp4(float("nan")) == 0
    assert orc.f32_to_fp4(-0.0) == 0     # sign only when magnitude index != 0


def test_f4x8_pack_unpack_and_zero_word():
    vals = [1.0, -1.0, 0.5, 6.0, -6.0, 0.0, 3.0, -3.0]
    w = orc.pack_word(orc.FMT_F4, vals)
    assert np.allclose(orc.unpack_word(orc.FMT_F4, w), vals, atol=0.01)
    assert orc.pack_word(orc.FMT_F4, [0.0] * 8) == 0


# ---- src/dtypes/f8x4.rs:173-292 ---------------------------------------------------------

def test_e4m3_specials():
    assert orc.e4m3_to_f32(0x00) == 0.0
    z = orc.e4m3_to_f32(0x80)
    assert z == 0.0 and math.copysign(1.0, z) == -1.0
    assert abs(orc.e4m3_to_f32(0x38) - 1.0) < 0.1
    assert abs(orc.e4m3_to_f32(0x77) - 240.0) < 1.0
    assert math.isnan(orc.e4m3_to_f32(0x7F)) and math.isnan(orc.e4m3_to_f32(0xFF))
    assert 0.0 < orc.e4m3_to_f32(0x01) < 0.1
    assert orc.f32_to_e4m3(float("nan")) == 0x7F
    # every exponent-15 code is NaN in the reference decoder, whatever the mantissa
    assert all(math.isnan(orc.e4m3_to_f32(c)) for c in range(0x78, 0x80))


def test_e4m3_roundtrip_extensive():
    vals = [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -2.0, 4.0, 8.0, 16.0, 32.0, 64.0, 128.0, -128.0,
            240.0, -240.0, 0.25, 0.125, 1.5, 2.5, 3.5, 7.0, 15.0, 31.0, 63.0, 127.0]
    for v in vals:
        d = orc.e4m3_to_f32(orc.f32_to_e4m3(v))
        assert abs(d - v) < 0.5 * max(abs(v), 1.0)


def test_e4m3_encoder_never_exceeds_0x77():
    codes = {orc.f32_to_e4m3(v) & 0x7F for v in [240.0, 250.0, 1e9, 239.9, 232.0, 248.0]}
    assert max(codes) <= 0x77


def test_f8x4_pack_unpack_all_representable():
    w = orc.pack_word(orc.FMT_F8, [0.0, 240.0, -240.0, float("nan")])
    u = orc.unpack_word(orc.FMT_F8, w)
    assert u[0] == 0.0 and abs(u[1] - 240) < 1 and abs(u[2] + 240) < 1 and math.isnan(u[3])


# ---- src/dtypes/i4x8.rs:82-121, i8x4.rs:52-86 ------------------------------------------------

def test_i4x8_roundtrip_clamp_zero():
    vals = [0.0, 1.0, 2.0, 3.0, -1.0, -4.0, 7.0, -8.0]
    assert list(orc.unpack_word(orc.FMT_I4, orc.pack_word(orc.FMT_I4, vals))) == vals
    u = orc.unpack_word(orc.FMT_I4, orc.pack_word(orc.FMT_I4, [100.0, -100.0, 0, 1, 2, 3, 4, 5]))
    assert u[0] == 7.0 and u[1] == -8.0
    assert orc.pack_word(orc.FMT_I4, [0.0] * 8) == 0


def test_i8x4_roundtrip_clamp_zero():
    assert list(orc.unpack_word(orc.FMT_I8, orc.pack_word(orc.FMT_I8, [0.0, 1.0, -1.0, 127.0]))) \
        == [0.0, 1.0, -1.0, 127.0]
    u = orc.unpack_word(orc.FMT_I8, orc.pack_word(orc.FMT_I8, [200.0, -200.0, 50.0, -50.0]))
    assert u[0] == 127.0 and u[1] == -128.0
    assert orc.pack_word(orc.FMT_I8, [0.0] * 4) == 0


def test_round_half_away_from_zero_after_clamp():
    # f32::round is half-away; clamp happens first (src/dtypes/i4x8.rs:36)
    u = orc.unpack_word(orc.FMT_I4, orc.pack_word(orc.FMT_I4, [0.5, -0.5, 1.5, -1.5, 2.5, 6.5, 7.4, -8.5]))
    assert list(u) == [1.0, -1.0, 2.0, -2.0, 3.0, 7.0, 7.0, -8.0]


# ---- src/packed_tensor.rs:1751-1759, 1887-2014 ---------------------------------------------------

def test_packed_len_has_16_word_margin():
    # 8 FP4 values pack into 1 u32 + 16 SIMD margin words
    assert orc.packed_words(orc.FMT_F4, 1, 8) == 17
    q = orc.quantize_nk(orc.FMT_I8, np.ones((3, 5), np.float32))
    assert q.words.size == 3 * 2 + 16 and not q.words[-16:].any()


def test_zero_range_row_gets_scale_one_zero_zero():
    for fmt in (orc.FMT_I8, orc.FMT_I4, orc.FMT_F4):
        q = orc.quantize_nk(fmt, np.full((2, 16), 1.0, np.float32))
        assert list(q.scales) == [1.0, 1.0] and list(q.zeros) == [0.0, 0.0]
        assert np.all(orc.dequant(q) == 1.0)


def test_f4x8_asymmetric_per_channel_scale_zp_values():
    row0 = [-5.0 + i * 10.0 / 63.0 for i in range(64)]
    row1 = [1.0 + i * 4.0 / 63.0 for i in range(64)]
    data = np.array([row0, row1], dtype=np.float32)
    q = orc.quantize_nk(orc.FMT_F4, data)
    assert q.scales.size == 2
    assert abs(q.scales[0] - 10.0 / 8.0) < 1e-5   # clipped FP4 range is 8 (+-4)
    assert abs(q.zeros[0] - 0.0) < 1e-5           # uniform -> mean == midpoint
    assert abs(q.scales[1] - 4.0 / 8.0) < 1e-5
    assert abs(q.zeros[1] - 3.0) < 1e-5


def test_f8_per_channel_scale_is_maxabs_over_240():
    data = np.array([[1.0, -2.0, 0.5, 0.25], [0.0, 0.0, 0.0, 0.0]], np.float32)
    q = orc.quantize_nk(orc.FMT_F8, data)
    assert q.scales[0] == np.float32(2.0) / np.float32(240.0) and q.scales[1] == 1.0
    assert q.zeros.size == 0  # IrDType::F8 carries scales only


# ---- src/backend/cpu/microkernels/tests.rs:504-533, 680-816 ----------------------------------------

def test_gemm_i8_asymmetric_zero_is_per_input_sum():
    # dequantized weight = q*2 + 10 = [12,14,16,18]; offset term is 10*sum(input), not +10
    q = orc.from_f32_slice(orc.FMT_I8, [12.0, 14.0, 16.0, 18.0], 1, 4, 2.0, 10.0)
    act = np.array([[1.0, 2.0, 3.0, 4.0], [-1.0, 0.5, 2.0, -3.0]], np.float32)
    out = orc.qmatmul(q, act)
    e0 = 12 * 1 + 14 * 2 + 16 * 3 + 18 * 4
    e1 = -12 + 14 * 0.5 + 16 * 2 + 18 * -3
    assert abs(out[0, 0] - e0) < 1e-4 and abs(out[1, 0] - e1) < 1e-4


def test_gemv_i4_asymmetric_zero_matches_dequant():
    w = [12.0, 14.0, 16.0, 18.0, 0.0, 2.0, 4.0, 6.0]
    q = orc.from_f32_slice(orc.FMT_I4, w, 1, 8, 2.0, 10.0)
    deq = orc.dequant(q)
    act = np.array([[1.0, 2.0, 3.0, 4.0, 0.5, -1.0, 2.0, -3.0]], np.float32)
    assert abs(orc.qmatmul(q, act)[0, 0] - float((deq[0] * act[0]).sum())) < 1e-4


def test_gemv_i8_per_row_scale_zero_negative_activations():
    scales, zeros = np.array([2.0, 3.0], np.float32), np.array([10.0, -5.0], np.float32)
    w = np.array([[12.0, 4.0, 20.0, -6.0], [7.0, -14.0, 1.0, 13.0]], np.float32)
    words = np.zeros(orc.packed_words(orc.FMT_I8, 2, 4), np.uint32)
    for r in range(2):
        words[r] = orc.pack_word(orc.FMT_I8, (w[r] - zeros[r]) / scales[r])
    q = orc.QWeight(orc.FMT_I8, 2, 4, words, scales, zeros)
    out = orc.qmatmul(q, np.array([[2.0, -3.0, 1.0, -2.0]], np.float32))
    assert abs(out[0, 0] - (12 * 2 + 4 * -3 + 20 * 1 + -6 * -2)) < 1e-4
    assert abs(out[0, 1] - (7 * 2 + -14 * -3 + 1 * 1 + 13 * -2)) < 1e-4


# ---- src/compiler/passes/quantization.rs:698-789 (shape facts of the pass) ---------------------------

@pytest.mark.parametrize("fmt", [orc.FMT_I8, orc.FMT_I4, orc.FMT_F8, orc.FMT_F4])
def test_pass_transposes_kn_to_nk_and_scales_are_per_output_channel(fmt):
    k, n = 8, 4
    w_kn = (np.arange(k * n, dtype=np.float32) / 8.0).reshape(k, n)
    q = orc.quantize_kn(fmt, w_kn)
    assert (q.n, q.k) == (n, k) and q.scales.size == n
    # row r of the packed tensor is column r of the graph constant
    assert np.abs(orc.dequant(q) - w_kn.T).max() <= 0.13 * np.abs(w_kn).max()


def test_codebook_pass_facts():
    k, n = 70, 3  # partial last block (70 = 2*32 + 6)
    w_kn = np.linspace(-1, 1, k * n, dtype=np.float32).reshape(k, n)
    q = orc.quantize_kn(orc.FMT_I4CB, w_kn)
    assert q.quant_block_size == 32 and q.scales.size == n * 3 and q.zeros.size == 0
    assert q.codebook.size == 16 and np.all(np.diff(q.codebook) >= 0)
    assert q.kernel_name == "matmul_i4"  # I4CB is `matmul_i4` with non-empty codebooks
    # block scale is the block's max |w|
    w_nk = w_kn.T
    assert q.scales[0] == np.abs(w_nk[0, :32]).max() and q.scales[2] == np.abs(w_nk[0, 64:]).max()


def test_kernel_names():
    # src/compiler/passes/quantization.rs:835-873, tests/quantized_pipeline.rs:608-620
    w = np.eye(4, dtype=np.float32)
    names = {f: orc.quantize_nk(f, w).kernel_name for f in orc.FMT_NAMES}
    assert names == {orc.FMT_I8: "matmul_i8", orc.FMT_I4: "matmul_i4", orc.FMT_F8: "matmul_f8",
                     orc.FMT_F4: "matmul_f4", orc.FMT_I4CB: "matmul_i4"}


# ---- tests/quantized_pipeline.rs:102-176, 825-869 ----------------------------------------------------

def _pipeline(fmt, w_kn, x):
    return orc.qmatmul(orc.quantize_kn(fmt, w_kn), x)


def test_matmul_u4_u8_end_to_end_bounds():
    w = (np.arange(32, dtype=np.float32) / 8.0).reshape(8, 4)
    x = np.full((2, 8), 0.5, np.float32)
    ref = x @ w
    for fmt, rel in ((orc.FMT_I4, 0.5), (orc.FMT_I8, 0.15)):
        out = _pipeline(fmt, w, x)
        small = np.abs(ref) <= 0.1
        assert np.all(np.abs(out - ref)[small] < 0.05)
        assert np.all((np.abs(out - ref) / np.abs(ref))[~small] < rel)


def test_matmul_i4codebook_and_f4_identity_roundtrip():
    w = np.eye(4, dtype=np.float32)
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    assert np.all(np.abs(_pipeline(orc.FMT_I4CB, w, x) - x) <= 1.0)
    assert np.all(np.abs(_pipeline(orc.FMT_F4, w, x) - x) <= 1.5)


# ---- tests/cpu_reference_oracle.rs:188-276 (tail-K cases, seeded xorshift inputs) -------------------

@pytest.mark.parametrize("fmt,cases,abs_tol,rel_tol", [
    (orc.FMT_I4, [(23, 2, 7, 5), (29, 3, 9, 4)], 0.45, 0.40),
    (orc.FMT_I8, [(41, 2, 7, 5), (43, 4, 9, 3)], 0.12, 0.10),
])
def test_reference_oracle_tail_k(fmt, cases, abs_tol, rel_tol):
    for seed, m, k, n in cases:
        w = seeded_values(seed + 1, k * n).reshape(k, n)
        x = seeded_values(seed, m * k).reshape(m, k)
        assert_close(f"seed={seed}", _pipeline(fmt, w, x), x @ w, abs_tol, rel_tol)


# ---- epilogue semantics: src/backend/cpu/matmul.rs:61-71, cpu/mod.rs:3140-3171 -------------------------

def test_epilogue_formulas():
    x = np.array([[-2.0, -0.5, 0.0, 0.5, 2.0, 3.0]], np.float32)
    b = np.array([0.5, -0.5, 0.0, 0.25, -1.0, 1.0], np.float32)
    y = (x + b).astype(np.float64)
    assert np.allclose(orc.epilogue(x, 6, b, orc.EPI_RELU), np.maximum(y, 0), atol=1e-6)
    gelu = 0.5 * y * (1 + np.tanh(0.7978846 * (y + 0.044715 * y ** 3)))
    assert np.allclose(orc.epilogue(x, 6, b, orc.EPI_GELU), gelu, atol=1e-6)
    assert np.allclose(orc.epilogue(x, 6, b, orc.EPI_SILU), y / (1 + np.exp(-y)), atol=1e-6)
    assert np.array_equal(orc.epilogue(x, 6, None, orc.EPI_NONE), x)


def test_add_broadcast_by_modulo():
    a = np.arange(6, dtype=np.float32)
    b = np.array([10.0, 20.0, 30.0], np.float32)
    assert list(orc.add_broadcast(a, b, 6)) == [10, 21, 32, 13, 24, 35]


# ---- what the reference CPU backend does today, kept measurable --------------------------------------

def test_as_written_mode_reproduces_dropped_epilogue_and_misstrided_codebook():
    rng = np.random.default_rng(5)
    w = rng.standard_normal((16, 8)).astype(np.float32)  # [K,N], non-square
    x = rng.standard_normal((3, 16)).astype(np.float32)
    b = rng.standard_normal(8).astype(np.float32)
    q8 = orc.quantize_kn(orc.FMT_I8, w)
    plain = orc.qmatmul(q8, x)
    # Op* fusion: the activation is silently not applied
    assert np.array_equal(orc.qmatmul(q8, x, None, orc.EPI_SILU, orc.MODE_AS_WRITTEN), plain)
    # MatMulAdd* fusion: a 3-input quantized MatMul writes nothing
    assert orc.qmatmul(q8, x, b, orc.EPI_GELU, orc.MODE_AS_WRITTEN) is None
    # bias without activation is a separate add_f32 and stays correct
    assert np.allclose(orc.qmatmul(q8, x, b, orc.EPI_NONE, orc.MODE_AS_WRITTEN),
                       orc.qmatmul(q8, x, b, orc.EPI_NONE, orc.MODE_INTENDED))
    # codebook GEMM reads the [N,K] buffer as [K,N]
    qc = orc.quantize_kn(orc.FMT_I4CB, w)
    wdeq = orc.dequant(qc)  # [N,K]
    assert np.allclose(orc.qmatmul(qc, x), x @ wdeq.T, atol=1e-4)
    assert np.allclose(orc.qmatmul(qc, x, mode=orc.MODE_AS_WRITTEN), x @ wdeq.reshape(16, 8), atol=1e-4)
