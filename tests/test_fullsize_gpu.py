"""Parity at the sizes the benchmark quotes numbers for, on a B200, through the C ABI.

Output columns are independent, so the CPU oracle checks slices of output channels exactly (the
first, a middle and the last 64 channels of every layer: the first and last weight tiles of the
persistent kernels and one from a later wave); linearity in the activations, run without an
activation function, covers every element of the output.  Weights are quantized by the library's
host pass; the oracle is only handed the rows of the slices.
"""
import numpy as np
import pytest

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200 import _lib as L
from helpers import max_err_vs_rms, normal

pytestmark = pytest.mark.gpu


class _Arena:
    """Activation / output / bias slots around an uploaded weight (no dequant slot: these layers
    are up to 28672 x 8192)."""

    def __init__(self, backend, meta, payload, m):
        self.b, self.m = backend, m
        self.n, self.k = meta.shape
        al = lambda x: -(-x // 256) * 256
        self.a_off, self.out_off = 0, al(m * self.k * 4)
        self.bias_off = self.out_off + al(m * self.n * 4)
        self.arena = backend.allocate_arena(self.bias_off + al(self.n * 4))
        self.w = backend.upload_qweight(payload, meta)

    def run(self, x, bias=None, epi=L.EPI_NONE, path=L.PATH_AUTO):
        b, m = self.b, x.shape[0]
        b.write_arena(self.arena, self.a_off, np.ascontiguousarray(x, np.float32).tobytes())
        if bias is not None:
            b.write_arena(self.arena, self.bias_off, np.ascontiguousarray(bias, np.float32).tobytes())
        rc = b.lib.fnn_cuda_qmatmul(b.ctx, self.w.handle, self.arena.handle, self.a_off, self.out_off,
                                    self.bias_off if bias is not None else -1, m, epi, path)
        if rc != 0:
            raise fnn.BackendError.from_status(rc)
        b.synchronize()   # a bounded wait that gave up raises here
        raw = b.read_arena(self.arena, self.out_off, m * self.n * 4)
        return np.frombuffer(raw, np.float32).reshape(m, self.n).copy()

    def close(self):
        self.w.close()
        self.arena.close()


def quantized_layer(fmt, k, n, sigma, seed):
    """(payload bytes, meta, oracle-side slicer) of a [K, N] layer quantized by the library."""
    w = normal(seed, (k, n), sigma)
    packed, scales, zeros, cb = fnn.quantize_weight_constant(w, fmt)
    words = np.frombuffer(packed.tobytes(), np.uint32)
    zp = zeros if fmt in (L.FMT_I8, L.FMT_I4, L.FMT_F4) else np.zeros(0, np.float32)
    meta = fnn.QuantizedWeightMeta(
        bit_width=8 if fmt in (L.FMT_I8, L.FMT_F8) else 4, scales=scales, zero_points=zp, shape=[n, k],
        quant_block_size=32 if fmt == L.FMT_I4CB else 0, codebooks=[cb] if fmt == L.FMT_I4CB else [], fmt=fmt)
    wpr = k // (4 if fmt in (L.FMT_I8, L.FMT_F8) else 8)
    bpr = k // 32

    def rows_of(rows):
        sub_words = np.concatenate([words[: n * wpr].reshape(n, wpr)[rows].reshape(-1), np.zeros(16, np.uint32)])
        if fmt == L.FMT_I4CB:
            return orc.QWeight(fmt, len(rows), k, sub_words, scales.reshape(n, bpr)[rows].reshape(-1).copy(),
                               np.zeros(0, np.float32), cb, 32)
        return orc.QWeight(fmt, len(rows), k, sub_words, scales[rows].copy(),
                           zp[rows].copy() if zp.size else np.zeros(0, np.float32))

    return packed.tobytes(), meta, rows_of


def slice_rows(n, width=64):
    mid = (n // 2) // 16 * 16 + 8   # not aligned to a 128-row tile
    return np.concatenate([np.arange(0, width), np.arange(mid, mid + width), np.arange(n - width, n)])


# (label, format, K, N, sigma, [(M, epilogue, bias?, error bar)]); the bar is 1e-3 except where the
# tcgen05 kernel runs two e4m3 activation terms (M >= 128) or the codebook format's fp16 operand
CASES = [
    ("c2_i8", L.FMT_I8, 4096, 11008, 0.02, [(128, L.EPI_SILU, False, 1e-3), (512, L.EPI_SILU, False, 1e-3)]),
    ("c3_f8", L.FMT_F8, 8192, 28672, 0.015, [(32, L.EPI_NONE, False, 1e-3), (512, L.EPI_NONE, False, 1e-2),
                                             (4096, L.EPI_NONE, False, 1e-2)]),
    ("c3_f4", L.FMT_F4, 8192, 28672, 0.015, [(32, L.EPI_NONE, False, 1e-3), (512, L.EPI_NONE, False, 1e-2),
                                             (4096, L.EPI_NONE, False, 1e-2)]),
    ("c5_i4_gateup", L.FMT_I4, 4096, 28672, 0.02, [(64, L.EPI_NONE, False, 1e-3)]),
    ("c5_i4_down", L.FMT_I4, 14336, 4096, 0.02, [(64, L.EPI_NONE, False, 1e-3)]),
    ("c5_i4_qkv", L.FMT_I4, 4096, 6144, 0.02, [(64, L.EPI_NONE, False, 1e-3)]),
    ("c4_i4cb_up", L.FMT_I4CB, 2048, 8192, 0.02, [(64, L.EPI_GELU, True, 1e-2), (1, L.EPI_GELU, True, 1e-3)]),
    ("c4_i4cb_down", L.FMT_I4CB, 8192, 2048, 0.02, [(64, L.EPI_NONE, True, 1e-2), (8, L.EPI_NONE, True, 1e-3)]),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_benchmark_sizes_against_oracle_slices(backend, case):
    label, fmt, k, n, sigma, points = case
    payload, meta, rows_of = quantized_layer(fmt, k, n, sigma, 7)
    rows = slice_rows(n)
    sub = rows_of(rows)
    bias = normal(8, (n,), 0.01)
    m_max = max(p[0] for p in points)
    rig = _Arena(backend, meta, payload, m_max)
    try:
        for m, epi, use_bias, tol in points:
            x = normal(9 + m, (m, k), 1.0)
            got = rig.run(x, bias if use_bias else None, epi)
            path = backend.last_path()
            # the oracle's cost grows with M: at 4096 rows it checks a quarter of them
            ms = np.arange(m) if m <= 512 else np.arange(0, m, 4)
            want = orc.qmatmul(sub, x[ms], bias[rows] if use_bias else None, epi)
            err = max_err_vs_rms(got[np.ix_(ms, rows)], want)
            assert err <= tol, (label, m, path, err)
            # whole output: linearity in the activations (no activation function, no bias)
            x2 = normal(90 + m, (m, k), 1.0)
            y1 = got if (epi == L.EPI_NONE and not use_bias) else rig.run(x)
            y2, y12 = rig.run(x2), rig.run(x + x2)
            scale = np.sqrt(np.mean(y12.astype(np.float64) ** 2))
            lin = float(np.max(np.abs(y12 - (y1 + y2))) / scale)
            assert lin <= 3 * tol, (label, m, path, lin)
    finally:
        rig.close()


def test_config4_stack_at_full_size_through_aot_executor(backend):
    """Config 4 as stated: 12 Linear layers alternating 2048 -> 8192 (bias, GELU) and 8192 -> 2048
    (bias) with a residual Add, quantize='i4cb', input [64, 2048], compiled through AotExecutor
    with fusion and the arena plan.  The oracle follows the whole chain on the CPU."""
    d, h, m, pairs = 2048, 8192, 64, 6
    params, nodes, cur = {}, [], "x"
    for i in range(pairs):
        params[f"w_up{i}"], params[f"b_up{i}"] = normal(10 + i, (d, h), 0.02), normal(20 + i, (h,), 0.01)
        params[f"w_dn{i}"], params[f"b_dn{i}"] = normal(30 + i, (h, d), 0.02), normal(40 + i, (d,), 0.01)
        nodes += [
            {"op_type": "Gemm", "name": f"up{i}", "inputs": f"[{cur}, w_up{i}, b_up{i}]", "outputs": f"[u{i}]"},
            {"op_type": "Gelu", "name": f"act{i}", "inputs": f"[u{i}]", "outputs": f"[g{i}]"},
            {"op_type": "Gemm", "name": f"dn{i}", "inputs": f"[g{i}, w_dn{i}, b_dn{i}]", "outputs": f"[v{i}]"},
            {"op_type": "Add", "name": f"res{i}", "inputs": f"[v{i}, {cur}]", "outputs": f"[r{i}]"},
        ]
        cur = f"r{i}"
    aot = fnn.AotExecutor(nodes, params, ["x"], [cur], {"x": [m, d]}, quantize="i4cb", backend=backend)
    names = [i.kernel_name for i in aot.plan.instructions if isinstance(i, fnn.CallKernel)]
    assert names == ["matmul_i4", "matmul_i4", "add_f32"] * pairs
    x = normal(50, (m, d), 1.0)
    got = aot.forward({"x": x})[cur]
    again = aot.forward({"x": x})[cur]        # second call: the captured replay of the static plan
    assert np.array_equal(got, again)
    # the oracle runs on the packed bytes and metadata the plan itself carries (the library's host
    # pass, whose bits the host tests pin against the oracle's own quantizer)
    consts = {i.dst.offset: i.data for i in aot.plan.instructions if isinstance(i, fnn.WriteConst)}
    layers = []
    for call in aot.plan.instructions:
        if isinstance(call, fnn.CallKernel) and call.kernel_name == "matmul_i4":
            meta = call.weight_meta
            words = np.frombuffer(consts[call.input_slices[1].offset], np.uint32)
            layers.append(orc.QWeight(orc.FMT_I4CB, meta.shape[0], meta.shape[1], words, meta.scales,
                                      np.zeros(0, np.float32), meta.codebooks[0], 32))
    assert len(layers) == 2 * pairs
    ref = x
    for i in range(pairs):
        up = orc.qmatmul(layers[2 * i], ref, params[f"b_up{i}"], orc.EPI_GELU)
        dn = orc.qmatmul(layers[2 * i + 1], up, params[f"b_dn{i}"], orc.EPI_NONE)
        ref = dn + ref
    # twelve fp16-operand tcgen05 layers in a row: the tensor-core bar
    assert max_err_vs_rms(got, ref) <= 1e-2
