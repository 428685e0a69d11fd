"""rms_norm and softmax plan instructions on a B200: the C-ABI entry points against the oracle's
restatement of the reference's scalar kernels (src/backend/cpu/microkernels/ops.rs:979-1008,
1363-1397), and a decoder-style block (rms_norm -> quantized MatMul + SiLU -> quantized MatMul ->
softmax) through GraphBuilder and AotExecutor."""
import numpy as np
import pytest

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200 import GraphBuilder, TensorType
from fastnn_b200.backend import _check
from helpers import max_err_vs_rms, normal

pytestmark = pytest.mark.gpu


def _run(backend, fn, x, extra=None):
    """x at offset 0, optional weight after it, output after that."""
    al = lambda v: -(-v // 256) * 256
    w_off = al(x.nbytes)
    out_off = w_off + al(extra.nbytes if extra is not None else 4)
    arena = backend.allocate_arena(out_off + al(x.nbytes))
    try:
        backend.write_arena(arena, 0, x.tobytes())
        if extra is not None:
            backend.write_arena(arena, w_off, extra.tobytes())
        fn(arena, w_off, out_off)
        backend.synchronize()
        return np.frombuffer(backend.read_arena(arena, out_off, x.nbytes), np.float32).reshape(x.shape)
    finally:
        arena.close()


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (3, 1000), (64, 8192), (5, 7), (2, 1)])
def test_rms_norm_matches_oracle(backend, rows, hidden):
    x = normal(700 + hidden, (rows, hidden), 2.0)
    w = normal(701 + hidden, (hidden,), 1.0)
    lib = backend.lib
    got = _run(backend, lambda a, w_off, out_off: _check(lib.fnn_cuda_rms_norm(
        backend.ctx, a.handle, 0, x.size, w_off, hidden, hidden, 1e-5, out_off)), x, w)
    want = orc.rms_norm(x, w, 1e-5)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-6), np.abs(got - want).max()
    # no weight: w = 1
    got = _run(backend, lambda a, w_off, out_off: _check(lib.fnn_cuda_rms_norm(
        backend.ctx, a.handle, 0, x.size, -1, 0, hidden, 1e-5, out_off)), x, None)
    assert np.allclose(got, orc.rms_norm(x, np.ones(hidden, np.float32), 1e-5), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("shape,axis", [((1, 32000), -1), ((16, 4, 128), 2), ((3, 5, 7), 1), ((6, 9), 0),
                                        ((4, 1), 1)])
def test_softmax_matches_oracle(backend, shape, axis):
    x = normal(710 + len(shape) + shape[-1], shape, 3.0)
    ax = axis % len(shape)
    stride = int(np.prod(shape[ax + 1:])) if ax + 1 < len(shape) else 1
    lib = backend.lib
    got = _run(backend, lambda a, w_off, out_off: _check(lib.fnn_cuda_softmax(
        backend.ctx, a.handle, 0, x.size, shape[ax], stride, out_off)), x)
    want = orc.softmax(x, axis)
    # the oracle adds the row sequentially in f32 like the reference's scalar kernel; over 32000 terms
    # that order alone moves the sum by ~1e-5 relative, so the bar is 2e-4 relative
    assert np.allclose(got, want, rtol=2e-4, atol=1e-9), np.abs(got - want).max()
    assert np.allclose(got.astype(np.float64).sum(ax), 1.0, atol=1e-5)


def test_row_ops_work_in_place_and_reject_bad_slices(backend):
    x = normal(720, (4, 256), 1.0)
    arena = backend.allocate_arena(x.nbytes)
    try:
        backend.write_arena(arena, 0, x.tobytes())
        _check(backend.lib.fnn_cuda_softmax(backend.ctx, arena.handle, 0, x.size, 256, 1, 0))
        backend.synchronize()
        got = np.frombuffer(backend.read_arena(arena, 0, x.nbytes), np.float32).reshape(x.shape)
        assert np.allclose(got, orc.softmax(x, -1), rtol=2e-4, atol=1e-9)
        with pytest.raises(fnn.BackendError, match="outside arena"):
            _check(backend.lib.fnn_cuda_softmax(backend.ctx, arena.handle, 256, x.size, 256, 1, 0))
        with pytest.raises(fnn.BackendError, match="whole rows"):
            _check(backend.lib.fnn_cuda_rms_norm(backend.ctx, arena.handle, 0, x.size, -1, 0, 100, 1e-5, 0))
    finally:
        arena.close()


def test_decoder_style_block_through_the_graph_builder(backend):
    """rms_norm -> W1 (I8, SiLU fused) -> W2 (I8) -> softmax, batch 3, against the oracle chain."""
    m, k, h, v = 3, 512, 1024, 640
    x = normal(730, (m, k), 1.0)
    g = np.abs(normal(731, (k,), 1.0)) + 0.5
    w1, w2 = normal(732, (k, h), 0.03), normal(733, (h, v), 0.03)
    gb = GraphBuilder()
    inp = gb.input_with_dims([m, k])
    t = gb.rms_norm(inp, gb.constant(g.tobytes(), TensorType.new([k])), 1e-6)
    t = gb.silu(gb.matmul(t, gb.constant(w1, TensorType.new([k, h]))))
    t = gb.softmax(gb.matmul(t, gb.constant(w2, TensorType.new([h, v]))), -1)
    out = gb.compile_and_execute_with_quantize([t], backend, [x.tobytes()], 8)
    got = np.frombuffer(out[0], np.float32).reshape(m, v)
    a = orc.rms_norm(x, g, 1e-6)
    a = orc.qmatmul(orc.quantize_kn(orc.FMT_I8, w1), a, None, orc.EPI_SILU)
    a = orc.qmatmul(orc.quantize_kn(orc.FMT_I8, w2), a)
    want = orc.softmax(a, -1)
    assert np.allclose(got.sum(-1), 1.0, atol=1e-5)
    assert max_err_vs_rms(got, want) <= 2e-3


def test_aot_executor_accepts_rms_norm_and_softmax_nodes(backend):
    m, k, n = 2, 256, 384
    x, g, w = normal(740, (m, k), 1.0), np.abs(normal(741, (k,), 1.0)) + 0.5, normal(742, (k, n), 0.05)
    nodes = [{"op_type": "RMSNorm", "inputs": "[x, g]", "outputs": "[h]", "eps": "1e-5"},
             {"op_type": "MatMul", "inputs": "[h, w]", "outputs": "[z]"},
             {"op_type": "Softmax", "inputs": "[z]", "outputs": "[y]", "axis": "-1"}]
    ex = fnn.AotExecutor(nodes, {"g": g, "w": w}, ["x"], ["y"], {"x": [m, k]}, quantize=8, backend=backend)
    got = ex.forward({"x": x})["y"]
    a = orc.qmatmul(orc.quantize_kn(orc.FMT_I8, w), orc.rms_norm(x, g, 1e-5))
    assert max_err_vs_rms(got, orc.softmax(a, -1)) <= 2e-3


@pytest.mark.parametrize("kind", ["rms", "layer"])
@pytest.mark.parametrize("rows,hidden", [(1, 4096), (7, 1000), (3, 5)])
def test_row_norm_with_residual_matches_oracle(backend, kind, rows, hidden):
    """fnn_cuda_row_norm: x = in + residual, then rms_norm or layer_norm with weight (and bias)."""
    x, r = normal(750 + hidden, (rows, hidden), 1.5), normal(751 + hidden, (rows, hidden), 0.7)
    w, b = normal(752 + hidden, (hidden,), 1.0), normal(753 + hidden, (hidden,), 0.2)
    al = lambda v: -(-v // 256) * 256
    offs, top = {}, 0
    for name, arr in (("x", x), ("r", r), ("w", w), ("b", b), ("y", x)):
        offs[name], top = top, top + al(arr.nbytes)
    arena = backend.allocate_arena(top)
    try:
        for name, arr in (("x", x), ("r", r), ("w", w), ("b", b)):
            backend.write_arena(arena, offs[name], arr.tobytes())
        k = 0 if kind == "rms" else 1
        _check(backend.lib.fnn_cuda_row_norm(backend.ctx, arena.handle, k, offs["x"], x.size, offs["r"],
                                             offs["w"], hidden, offs["b"] if k else -1, hidden if k else 0,
                                             hidden, 1e-5, offs["y"]))
        backend.synchronize()
        got = np.frombuffer(backend.read_arena(arena, offs["y"], x.nbytes), np.float32).reshape(x.shape)
    finally:
        arena.close()
    want = orc.rms_norm(x + r, w, 1e-5) if kind == "rms" else orc.layer_norm(x, w, b, 1e-5, r)
    assert np.allclose(got, want, rtol=1e-4, atol=2e-6), np.abs(got - want).max()


def test_residual_block_through_the_graph_builder(backend):
    """h = x + W_o(a); y = W_up(layer_norm(h)) with GELU: the Add feeds the norm and is fused into it."""
    m, k, n = 4, 512, 768
    x, a = normal(760, (m, k), 1.0), normal(761, (m, k), 1.0)
    wo, wu = normal(762, (k, k), 0.04), normal(763, (k, n), 0.04)
    g, beta = np.abs(normal(764, (k,), 1.0)) + 0.5, normal(765, (k,), 0.1)
    gb = GraphBuilder()
    xi, ai = gb.input_with_dims([m, k]), gb.input_with_dims([m, k])
    h = gb.add(xi, gb.matmul(ai, gb.constant(wo, TensorType.new([k, k]))))
    t = gb.layer_norm(h, gb.constant(g.tobytes(), TensorType.new([k])),
                      gb.constant(beta.tobytes(), TensorType.new([k])), 1e-5)
    y = gb.gelu(gb.matmul(t, gb.constant(wu, TensorType.new([k, n]))))
    out = gb.compile_and_execute_with_quantize([y], backend, [x.tobytes(), a.tobytes()], 8)
    got = np.frombuffer(out[0], np.float32).reshape(m, n)
    o = orc.qmatmul(orc.quantize_kn(orc.FMT_I8, wo), a)
    ln = orc.layer_norm(x, g, beta, 1e-5, o)
    want = orc.qmatmul(orc.quantize_kn(orc.FMT_I8, wu), ln, None, orc.EPI_GELU)
    assert max_err_vs_rms(got, want) <= 2e-3
