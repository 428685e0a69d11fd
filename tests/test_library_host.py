"""CPU-side checks of the shipped library: the C ABI exports what the header declares, and the
library's host quantization pass is bit-identical to the oracle.  No kernel is launched."""
import ctypes
import os
import re

import numpy as np
import pytest

import oracle as orc
from fastnn_b200 import _lib as L
from fastnn_b200.compiler import quantize_weight_constant
from helpers import normal

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "qmatmul_small.npz")


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fastnn_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fnn_(?:cuda|quant|quantize)_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(L.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/fastnn_cuda.h but not exported"
    assert sorted(L.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_no_device_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import fastnn_b200 as fnn
    with pytest.raises(fnn.BackendError):
        fnn.CudaBackend(0)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("shape", [(7, 5), (64, 16), (100, 33), (257, 8), (32, 1), (1, 40)])
@pytest.mark.parametrize("fmt", list(orc.FMT_NAMES))
def test_host_quantizer_is_bit_identical_to_oracle(fmt, shape):
    k, n = shape
    w = normal(500 + k * 3 + n, (k, n), 0.02)
    w[:, 0] = -0.125  # zero-range output channel
    q = orc.quantize_kn(fmt, w)
    packed, scales, zeros, codebook = quantize_weight_constant(w, fmt)
    assert packed.tobytes() == q.payload
    assert np.array_equal(bits(scales), bits(q.scales))
    if fmt in (orc.FMT_I8, orc.FMT_I4, orc.FMT_F4):
        assert np.array_equal(bits(zeros), bits(q.zeros))
    if fmt == orc.FMT_I4CB:
        assert np.array_equal(bits(codebook), bits(q.codebook))


def test_host_quantizer_reproduces_golden_vectors():
    g = np.load(GOLDEN)
    for case in ("aligned", "ragged", "wide"):
        for fmt, name in orc.FMT_NAMES.items():
            packed, scales, zeros, codebook = quantize_weight_constant(g[f"{case}/w_kn"], fmt)
            p = f"{case}/{name}"
            assert packed.tobytes() == g[p + "/words"].tobytes(), p
            assert np.array_equal(bits(scales), bits(g[p + "/scales"])), p


def test_quant_size_helpers():
    lib = L.load()
    assert lib.fnn_quant_packed_bytes(L.FMT_I4, 3, 20) == (3 * 3 + 16) * 4
    assert lib.fnn_quant_packed_bytes(L.FMT_F8, 3, 20) == (3 * 5 + 16) * 4
    assert lib.fnn_quant_num_scales(L.FMT_I4CB, 3, 70) == 9
    assert lib.fnn_quant_packed_bytes(99, 3, 20) == 0
