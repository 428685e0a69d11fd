"""The C oracle, its NumPy twin and the committed golden vectors must agree bit for bit.

The reference pins no packed bytes, scales or codebooks for random weights, so two separately
written restatements (oracle/fastnn_oracle.c and oracle/np_twin.py) cross-check each other,
and tests/golden/qmatmul_small.npz freezes their output.
"""
import os

import numpy as np
import pytest

import oracle as orc
from oracle import np_twin as tw
from helpers import normal

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qmatmul_small.npz")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def twin_quantize(name, w_nk):
    if name == "i8":
        return (*tw.quantize_int_asym(w_nk, 8), None)
    if name == "i4":
        return (*tw.quantize_int_asym(w_nk, 4), None)
    if name == "f4":
        return (*tw.quantize_fp4_asym(w_nk), None)
    if name == "f8":
        words, s = tw.quantize_f8_sym(w_nk)
        return words, s, np.zeros(0, np.float32), None
    words, s, cb = tw.quantize_codebook(w_nk)
    return words, s, np.zeros(0, np.float32), cb


@pytest.mark.parametrize("shape", [(5, 7), (16, 64), (33, 100), (8, 257), (1, 32), (40, 1)])
@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
def test_c_oracle_equals_numpy_twin(fmt, shape):
    n, k = shape
    w = normal(1000 + n * 7 + k, (n, k), 0.02)
    w[0, :] = 0.25                      # zero-range row
    if n > 2:
        w[2, : min(k, 32)] = 0.0        # all-zero codebook block / row start
    name = orc.FMT_NAMES[fmt]
    q = orc.quantize_nk(fmt, w)
    words, s, z, cb = twin_quantize(name, w)
    assert np.array_equal(words, q.words)
    assert np.array_equal(bits(s), bits(q.scales))
    assert np.array_equal(bits(z), bits(q.zeros))
    if cb is not None:
        assert np.array_equal(bits(cb), bits(q.codebook))
    d_c = orc.dequant(q)
    d_np = tw.dequant(name, q.words, n, k, q.scales, q.zeros, q.codebook)
    assert np.array_equal(bits(d_c), bits(d_np))


def test_e4m3_decode_tables_agree():
    table = tw.e4m3_decode_table()
    for c in range(256):
        a, b = orc.e4m3_to_f32(c), float(table[c])
        assert (np.isnan(a) and np.isnan(b)) or (a == b and np.signbit(a) == np.signbit(b))
    ft = tw.fp4_decode_table()
    assert [orc.fp4_to_f32(c) for c in range(16)] == list(ft)


def test_e4m3_encoders_agree_on_a_dense_sweep():
    rng = np.random.default_rng(3)
    v = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 100,
        rng.standard_normal(20000).astype(np.float32) * 0.01,
        np.array([0.0, -0.0, 240.0, -240.0, 1e9, 0.015625, 0.0156249, 2 ** -9, 2 ** -10, 2 ** -11,
                  np.nan, 1.0, 0.99999994, 1.9999999, 232.0, 248.0], np.float32)])
    got = tw.e4m3_encode(v)
    want = np.array([orc.f32_to_e4m3(float(x)) for x in v], np.uint8)
    assert np.array_equal(got, want)


def test_golden_vectors_are_reproduced():
    g = np.load(GOLDEN)
    cases = sorted({k.split("/")[0] for k in g.files})
    assert cases == ["aligned", "ragged", "wide"]
    for case in cases:
        w_kn, x, bias = g[f"{case}/w_kn"], g[f"{case}/x"], g[f"{case}/bias"]
        for fmt, name in orc.FMT_NAMES.items():
            p = f"{case}/{name}"
            q = orc.quantize_kn(fmt, w_kn)
            assert np.array_equal(q.words, g[p + "/words"]), p
            assert np.array_equal(bits(q.scales), bits(g[p + "/scales"])), p
            assert np.array_equal(bits(q.zeros), bits(g[p + "/zeros"])), p
            if q.codebook is not None:
                assert np.array_equal(bits(q.codebook), bits(g[p + "/codebook"])), p
            assert np.array_equal(bits(orc.dequant(q)), bits(g[p + "/dequant"])), p
            # GEMM results depend on the host's SIMD width (sum order): tolerance, not bits
            for key, args in (("out_plain", (None, orc.EPI_NONE)),
                              ("out_bias_gelu", (bias, orc.EPI_GELU)),
                              ("out_silu", (None, orc.EPI_SILU))):
                got = orc.qmatmul(q, x, *args)
                assert np.allclose(got, g[f"{p}/{key}"], rtol=1e-5, atol=1e-5), (p, key)


def test_oracle_gemm_matches_dequantized_f64_reference():
    """acc*scale + zero*sum(a) (gemm.rs:2048-2087) equals A . Wdeq^T up to f32 rounding."""
    for fmt in orc.FMT_NAMES:
        w = normal(77 + fmt, (96, 24), 0.02)
        x = normal(88 + fmt, (5, 96), 1.0)
        q = orc.quantize_kn(fmt, w)
        ref = x.astype(np.float64) @ orc.dequant(q).astype(np.float64).T
        got = orc.qmatmul(q, x)
        assert np.max(np.abs(got - ref)) <= 1e-5 * max(1.0, np.abs(ref).max())
