"""CPU oracle for fastnn's quantized-weight MatMul path -- TEST INFRASTRUCTURE ONLY.

ctypes front-end of ``oracle/fastnn_oracle.c`` (a plain-C restatement of the reference's
Rust algorithm; every C function cites the reference file:line it follows).  Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark may import this package;
the CUDA product path never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfastnn_oracle.so")

FMT_I8, FMT_I4, FMT_F8, FMT_F4, FMT_I4CB = 0, 1, 2, 3, 4
FMT_NAMES = {FMT_I8: "i8", FMT_I4: "i4", FMT_F8: "f8", FMT_F4: "f4", FMT_I4CB: "i4cb"}
FMT_BY_NAME = {v: k for k, v in FMT_NAMES.items()}
EPI_NONE, EPI_RELU, EPI_GELU, EPI_SILU = 0, 1, 2, 3
MODE_INTENDED, MODE_AS_WRITTEN = 0, 1
SIMD_MARGIN_WORDS = 16
CODEBOOK_BLOCK = 32


def build(force: bool = False) -> str:
    """Compile the C oracle with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "fastnn_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_LIB_PATH)
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libfastnn_oracle.so"])
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = ctypes.CDLL(_LIB_PATH)
    c_sz, c_int, c_f, c_vp = ctypes.c_size_t, ctypes.c_int, ctypes.c_float, ctypes.c_void_p
    L.orc_items_per_word.argtypes = [c_int]
    L.orc_items_per_word.restype = c_int
    L.orc_words_per_row.argtypes = [c_int, c_sz]
    L.orc_words_per_row.restype = c_sz
    L.orc_packed_words.argtypes = [c_int, c_sz, c_sz]
    L.orc_packed_words.restype = c_sz
    L.orc_f32_to_e4m3.argtypes = [c_f]
    L.orc_f32_to_e4m3.restype = ctypes.c_uint8
    L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
    L.orc_e4m3_to_f32.restype = c_f
    L.orc_f32_to_fp4.argtypes = [c_f]
    L.orc_f32_to_fp4.restype = ctypes.c_uint8
    L.orc_fp4_to_f32.argtypes = [ctypes.c_uint8]
    L.orc_fp4_to_f32.restype = c_f
    L.orc_pack_word.argtypes = [c_int, c_vp]
    L.orc_pack_word.restype = ctypes.c_uint32
    L.orc_unpack_word.argtypes = [c_int, ctypes.c_uint32, c_vp]
    L.orc_unpack_word.restype = None
    L.orc_transpose_kn_to_nk.argtypes = [c_vp, c_sz, c_sz, c_vp]
    L.orc_transpose_kn_to_nk.restype = None
    L.orc_from_f32_slice.argtypes = [c_int, c_vp, c_sz, c_sz, c_f, c_f, c_vp]
    L.orc_from_f32_slice.restype = None
    L.orc_quantize.argtypes = [c_int, c_vp, c_sz, c_sz, c_vp, c_vp, c_vp, c_vp]
    L.orc_quantize.restype = c_int
    L.orc_kmeans16.argtypes = [c_vp, c_sz, c_int, c_vp]
    L.orc_kmeans16.restype = None
    L.orc_dequant.argtypes = [c_int, c_vp, c_sz, c_sz, c_vp, c_vp, c_vp, c_vp]
    L.orc_dequant.restype = c_int
    L.orc_qmatmul.argtypes = [c_int, c_vp, c_sz, c_sz, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp,
                              c_int, c_int, c_vp]
    L.orc_qmatmul.restype = c_int
    L.orc_epilogue.argtypes = [c_vp, c_sz, c_sz, c_vp, c_int]
    L.orc_epilogue.restype = None
    L.orc_add_broadcast.argtypes = [c_vp, c_sz, c_vp, c_sz, c_vp, c_sz]
    L.orc_add_broadcast.restype = None
    L.orc_rms_norm.argtypes = [c_vp, c_sz, c_vp, c_sz, c_sz, ctypes.c_float, c_vp]
    L.orc_rms_norm.restype = None
    L.orc_layer_norm.argtypes = [c_vp, c_vp, c_sz, c_vp, c_sz, c_vp, c_sz, c_sz, ctypes.c_float, c_vp]
    L.orc_layer_norm.restype = None
    L.orc_softmax.argtypes = [c_vp, c_sz, c_sz, c_sz, c_vp]
    L.orc_softmax.restype = None
    L.orc_simd_level.restype = c_int
    L.orc_physical_cores.restype = c_int
    L.orc_k_block_size.restype = c_sz
    _lib = L
    return L


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


@dataclass
class QWeight:
    """What the reference's quantization pass leaves on a weight Constant: the packed
    `[N, ceil(K/ITEMS)]` u32 rows plus 16 margin words, and the metadata that
    `QuantizedWeightMeta` (src/backend/mod.rs:43-58) carries to the kernel."""

    fmt: int
    n: int
    k: int
    words: np.ndarray  # uint32, len rows*k_packed + 16
    scales: np.ndarray  # float32
    zeros: np.ndarray  # float32 (empty for F8 / I4CB in the IR dtype)
    codebook: Optional[np.ndarray] = None  # float32[16] for I4CB
    quant_block_size: int = 0

    @property
    def bit_width(self) -> int:
        return 8 if self.fmt in (FMT_I8, FMT_F8) else 4

    @property
    def payload(self) -> bytes:
        """`pt.as_bytes()`: what WriteConst carries (margin included)."""
        return self.words.tobytes()

    @property
    def kernel_name(self) -> str:
        return {FMT_I8: "matmul_i8", FMT_I4: "matmul_i4", FMT_F8: "matmul_f8",
                FMT_F4: "matmul_f4", FMT_I4CB: "matmul_i4"}[self.fmt]


def items_per_word(fmt: int) -> int:
    return lib().orc_items_per_word(fmt)


def packed_words(fmt: int, rows: int, inner: int) -> int:
    return lib().orc_packed_words(fmt, rows, inner)


def f32_to_e4m3(v: float) -> int:
    return int(lib().orc_f32_to_e4m3(ctypes.c_float(v)))


def e4m3_to_f32(b: int) -> float:
    return float(lib().orc_e4m3_to_f32(b))


def f32_to_fp4(v: float) -> int:
    return int(lib().orc_f32_to_fp4(ctypes.c_float(v)))


def fp4_to_f32(c: int) -> float:
    return float(lib().orc_fp4_to_f32(c))


def pack_word(fmt: int, vals) -> int:
    a = _f32(vals)
    assert a.size == items_per_word(fmt)
    return int(lib().orc_pack_word(fmt, _p(a)))


def unpack_word(fmt: int, word: int) -> np.ndarray:
    out = np.zeros(8, dtype=np.float32)
    lib().orc_unpack_word(fmt, ctypes.c_uint32(word), _p(out))
    return out[: items_per_word(fmt)].copy()


def transpose_kn_to_nk(w_kn: np.ndarray) -> np.ndarray:
    w_kn = _f32(w_kn)
    K, N = w_kn.shape
    out = np.empty((N, K), dtype=np.float32)
    lib().orc_transpose_kn_to_nk(_p(w_kn), K, N, _p(out))
    return out


def from_f32_slice(fmt: int, data, rows: int, inner: int, scale: float, zero: float) -> QWeight:
    data = _f32(data).reshape(-1)
    words = np.zeros(packed_words(fmt, rows, inner), dtype=np.uint32)
    lib().orc_from_f32_slice(fmt, _p(data), rows, inner, ctypes.c_float(scale),
                             ctypes.c_float(zero), _p(words))
    return QWeight(fmt, rows, inner, words, np.array([scale], np.float32),
                   np.array([zero], np.float32))


def quantize_nk(fmt: int, w_nk: np.ndarray) -> QWeight:
    """Quantize an [N,K] f32 weight (already transposed) like the compiler pass."""
    w_nk = _f32(w_nk)
    N, K = w_nk.shape
    words = np.zeros(packed_words(fmt, N, K), dtype=np.uint32)
    if fmt == FMT_I4CB:
        scales = np.zeros(N * ((K + CODEBOOK_BLOCK - 1) // CODEBOOK_BLOCK), dtype=np.float32)
        zeros = np.zeros(0, dtype=np.float32)
        codebook = np.zeros(16, dtype=np.float32)
        rc = lib().orc_quantize(fmt, _p(w_nk), N, K, _p(words), _p(scales), None, _p(codebook))
        assert rc == 0
        return QWeight(fmt, N, K, words, scales, zeros, codebook, CODEBOOK_BLOCK)
    scales = np.zeros(N, dtype=np.float32)
    zeros = np.zeros(N, dtype=np.float32)
    rc = lib().orc_quantize(fmt, _p(w_nk), N, K, _p(words), _p(scales), _p(zeros), None)
    assert rc == 0
    if fmt == FMT_F8:
        zeros = np.zeros(0, dtype=np.float32)  # IrDType::F8 carries scales only
    return QWeight(fmt, N, K, words, scales, zeros)


def quantize_kn(fmt: int, w_kn: np.ndarray) -> QWeight:
    """Graph-level entry: constant is [K,N]; the pass transposes to [N,K] first
    (src/compiler/passes/quantization.rs:144-156)."""
    return quantize_nk(fmt, transpose_kn_to_nk(w_kn))


def kmeans16(values, iters: int = 30) -> np.ndarray:
    values = _f32(values).reshape(-1)
    out = np.zeros(16, dtype=np.float32)
    lib().orc_kmeans16(_p(values), values.size, iters, _p(out))
    return out


def _zeros_full(q: QWeight) -> Optional[np.ndarray]:
    if q.fmt == FMT_I4CB:
        return None
    if q.zeros.size == 0:
        return np.zeros(q.scales.size, dtype=np.float32)
    return q.zeros


def _expand_per_row(q: QWeight):
    """Per-tensor (scale, zero) -> per-row arrays (scale_for_row, packed_tensor.rs:439-462)."""
    s, z = q.scales, _zeros_full(q)
    if q.fmt != FMT_I4CB and s.size == 1 and q.n > 1:
        s = np.full(q.n, s[0], np.float32)
        z = np.full(q.n, z[0], np.float32)
    return s, z


def dequant(q: QWeight) -> np.ndarray:
    out = np.empty((q.n, q.k), dtype=np.float32)
    s, z = _expand_per_row(q)
    rc = lib().orc_dequant(q.fmt, _p(q.words), q.n, q.k, _p(s), _p(z), _p(q.codebook), _p(out))
    assert rc == 0
    return out


def qmatmul(q: QWeight, act: np.ndarray, bias: Optional[np.ndarray] = None,
            epilogue: int = EPI_NONE, mode: int = MODE_INTENDED) -> Optional[np.ndarray]:
    act = _f32(act)
    M, K = act.shape
    assert K == q.k
    out = np.zeros((M, q.n), dtype=np.float32)
    b = None if bias is None else _f32(bias)
    s, z = _expand_per_row(q)
    rc = lib().orc_qmatmul(q.fmt, _p(q.words), q.n, q.k, _p(s), _p(z), _p(q.codebook), _p(act),
                           M, _p(b), epilogue, mode, _p(out))
    assert rc >= 0
    if rc == 1:
        return None  # the reference writes nothing on this path
    return out


def epilogue(x: np.ndarray, n: int, bias: Optional[np.ndarray], epi: int) -> np.ndarray:
    out = _f32(x).copy()
    b = None if bias is None else _f32(bias)
    lib().orc_epilogue(_p(out), out.size, n, _p(b), epi)
    return out


def add_broadcast(a: np.ndarray, b: np.ndarray, out_len: int) -> np.ndarray:
    a, b = _f32(a).reshape(-1), _f32(b).reshape(-1)
    out = np.empty(out_len, dtype=np.float32)
    lib().orc_add_broadcast(_p(a), a.size, _p(b), b.size, _p(out), out_len)
    return out


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float, mode: int = MODE_INTENDED) -> np.ndarray:
    """Rows of weight.size elements (the hidden size; one row when weight is empty).  MODE_AS_WRITTEN
    reproduces the unfused dispatch arm's row size x.size // weight.size
    (src/backend/cpu/mod.rs:5053-5075)."""
    x, weight = _f32(x), _f32(weight).reshape(-1)
    row = x.size if weight.size == 0 else (weight.size if mode == MODE_INTENDED else x.size // weight.size)
    out = np.empty(x.size, dtype=np.float32)
    lib().orc_rms_norm(_p(x.reshape(-1)), x.size, _p(weight) if weight.size else None, weight.size,
                       row, ctypes.c_float(eps), _p(out))
    return out.reshape(x.shape)


def layer_norm(x: np.ndarray, weight, bias, eps: float, residual=None) -> np.ndarray:
    """Rows of the last dimension; x + residual is normalised when a residual is given."""
    x = _f32(x)
    row = x.shape[-1]
    w = _f32(weight).reshape(-1) if weight is not None else np.zeros(0, np.float32)
    b = _f32(bias).reshape(-1) if bias is not None else np.zeros(0, np.float32)
    r = _f32(residual).reshape(-1) if residual is not None else None
    out = np.empty(x.size, dtype=np.float32)
    lib().orc_layer_norm(_p(x.reshape(-1)), _p(r) if r is not None else None, x.size,
                         _p(w) if w.size else None, w.size, _p(b) if b.size else None, b.size, row,
                         ctypes.c_float(eps), _p(out))
    return out.reshape(x.shape)


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    x = _f32(x)
    axis = axis % x.ndim
    stride = int(np.prod(x.shape[axis + 1:], dtype=np.int64)) if axis + 1 < x.ndim else 1
    out = np.empty(x.size, dtype=np.float32)
    lib().orc_softmax(_p(x.reshape(-1)), x.size, x.shape[axis], stride, _p(out))
    return out.reshape(x.shape)


def host_info() -> dict:
    L = lib()
    return {"simd_level": L.orc_simd_level(), "physical_cores": L.orc_physical_cores(),
            "k_block_size": int(L.orc_k_block_size())}
