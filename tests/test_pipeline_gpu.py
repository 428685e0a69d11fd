"""End-to-end through the reference-facing API on a B200: GraphBuilder ->
compile_and_execute_with_quantize -> CudaBackend, and AotExecutor(quantize=...).
Same graphs as the reference's tests/quantized_pipeline.rs and tests/wgpu_quantized.rs
(`run_matmul<B: Backend>`), checked against the CPU oracle."""
import numpy as np
import pytest

import oracle as orc
import fastnn_b200 as fnn
from fastnn_b200 import GraphBuilder, GraphExecutor, TensorType, WeightDtype
from helpers import assert_close, max_err_vs_rms, normal, seeded_values

pytestmark = pytest.mark.gpu


def run_matmul(backend, m, k, n, w, x, quantize):
    """tests/quantized_pipeline.rs:20-49 with the backend as a parameter."""
    gb = GraphBuilder()
    inp = gb.input_with_dims([m, k])
    weight = gb.constant(np.asarray(w, np.float32).tobytes(), TensorType.new([k, n]))
    out = gb.matmul(inp, weight)
    res = gb.compile_and_execute_with_quantize([out], backend, [np.asarray(x, np.float32).tobytes()],
                                               quantize)
    return np.frombuffer(res[0], np.float32).reshape(m, n)


def test_matmul_u4_u8_end_to_end(backend):
    w = (np.arange(32, dtype=np.float32) / 8.0).reshape(8, 4)
    x = np.full((2, 8), 0.5, np.float32)
    ref = x @ w
    for quantize, rel, fmt in ((4, 0.5, orc.FMT_I4), (8, 0.15, orc.FMT_I8)):
        out = run_matmul(backend, 2, 8, 4, w, x, quantize)
        assert out.shape == (2, 4)
        assert np.all(np.abs(out - ref) / np.abs(ref) < rel)
        assert max_err_vs_rms(out, orc.qmatmul(orc.quantize_kn(fmt, w), x)) <= 1e-3


@pytest.mark.parametrize("quantize,cases,abs_tol,rel_tol", [
    (4, [(23, 2, 7, 5), (29, 3, 9, 4)], 0.45, 0.40),
    (8, [(41, 2, 7, 5), (43, 4, 9, 3)], 0.12, 0.10)])
def test_reference_oracle_tail_k_cases(backend, quantize, cases, abs_tol, rel_tol):
    """tests/cpu_reference_oracle.rs:188-276."""
    for seed, m, k, n in cases:
        w = seeded_values(seed + 1, k * n).reshape(k, n)
        x = seeded_values(seed, m * k).reshape(m, k)
        assert_close(f"seed={seed}", run_matmul(backend, m, k, n, w, x, quantize), x @ w,
                     abs_tol, rel_tol)


def test_config1_linear_i4_bias_through_graph_builder(backend):
    """Config 1: x[8,4096] @ W[4096,4096] (quantize=4) + bias, seed 0 (smaller N for speed is
    not used: this is the reference's own CPU-runnable case at full size)."""
    m, k, n = 8, 4096, 4096
    w, x, b = normal(0, (k, n), 0.02), normal(1, (m, k), 1.0), normal(2, (n,), 0.01)
    gb = GraphBuilder()
    inp = gb.input_with_dims([m, k])
    y = gb.add(gb.matmul(inp, gb.constant(w, TensorType.new([k, n]))),
               gb.constant(b, TensorType.new([n])))
    out = gb.compile_and_execute_with_quantize([y], backend, [x.tobytes()], 4)
    got = np.frombuffer(out[0], np.float32).reshape(m, n)
    want = orc.qmatmul(orc.quantize_kn(orc.FMT_I4, w), x, b, orc.EPI_NONE)
    assert max_err_vs_rms(got, want) <= 1e-3
    # the quantized result is also close to the f32 layer (tests/quantized_pipeline.rs bounds)
    ref = x @ w + b
    assert np.sqrt(np.mean((got - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)) < 0.2


@pytest.mark.parametrize("wd", [WeightDtype.F8x4, WeightDtype.F4x8, WeightDtype.I4Codebook])
def test_compile_with_weight_dtype_fp_formats(backend, wd):
    m, k, n = 4, 256, 96
    w, x = normal(5, (k, n), 0.015), normal(6, (m, k), 1.0)
    gb = GraphBuilder()
    inp = gb.input_with_dims([m, k])
    y = gb.silu(gb.matmul(inp, gb.constant(w, TensorType.new([k, n]))))
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    ex = GraphExecutor(backend)
    plan, mp, cg = ex.compile_with_weight_dtype(g, wd)
    fmt = {WeightDtype.F8x4: orc.FMT_F8, WeightDtype.F4x8: orc.FMT_F4,
           WeightDtype.I4Codebook: orc.FMT_I4CB}[wd]
    want = orc.qmatmul(orc.quantize_kn(fmt, w), x, None, orc.EPI_SILU)
    for _ in range(2):  # second call replays the static plan without WriteConst
        got = np.frombuffer(ex.execute(cg, plan, mp, [x.tobytes()])[0], np.float32).reshape(m, n)
        assert max_err_vs_rms(got, want) <= 1e-3
    prof = ex.execute_profile(cg, plan, mp, [x.tobytes()])
    assert [p.kernel_name for p in prof][-1].startswith("matmul_") and prof[-1].elapsed_ns > 0


def test_aot_executor_i4cb_mlp_stack_with_residual(backend):
    """Config 4 in miniature: Linear(+bias, GELU) up, Linear(+bias) down, residual add, twice;
    quantize='i4cb'.  The oracle runs the intended semantics (the reference CPU backend writes
    nothing for the fused up-projection and mis-strides non-square codebook GEMMs)."""
    d, h, m, layers = 64, 256, 6, 2
    params, nodes = {}, []
    cur = "x"
    for i in range(layers):
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
    assert names == ["matmul_i4", "matmul_i4", "add_f32"] * layers
    x = normal(50, (m, d), 1.0)
    got = aot.forward({"x": x})[cur]
    ref = x
    for i in range(layers):
        up = orc.qmatmul(orc.quantize_kn(orc.FMT_I4CB, params[f"w_up{i}"]), ref, params[f"b_up{i}"], orc.EPI_GELU)
        dn = orc.qmatmul(orc.quantize_kn(orc.FMT_I4CB, params[f"w_dn{i}"]), up, params[f"b_dn{i}"], orc.EPI_NONE)
        ref = dn + ref
    assert max_err_vs_rms(got, ref) <= 1e-3
    assert aot.memory_stats()["arena_bytes"] > 0


def test_symbolic_batch_dimension(backend):
    k, n = 128, 48
    w = normal(3, (k, n), 0.02)
    aot = fnn.AotExecutor([{"op_type": "MatMul", "inputs": "[x, w]", "outputs": "[y]"}], {"w": w},
                          ["x"], ["y"], {"x": [-1, k]}, quantize=8, backend=backend)
    q = orc.quantize_kn(orc.FMT_I8, w)
    for m in (1, 5, 3):
        x = normal(60 + m, (m, k), 1.0)
        got = aot.forward({"x": x})["y"]
        assert got.shape == (m, n) and max_err_vs_rms(got, orc.qmatmul(q, x)) <= 1e-3


def test_unsupported_paths_fail_loudly(backend):
    gb = GraphBuilder()
    x = gb.input_with_dims([2, 8])
    y = gb.matmul(x, gb.constant(np.ones((8, 4), np.float32), TensorType.new([8, 4])))
    with pytest.raises(fnn.BackendError, match="Unsupported"):
        gb.compile_and_execute_with_quantize([y], backend, [bytes(64)], None)  # f32 MatMul
    arena = backend.allocate_arena(256)
    bogus = fnn.CallKernel("conv2d_i4", [fnn.BufferSlice(0, 64)], fnn.BufferSlice(64, 64), [])
    with pytest.raises(fnn.BackendError, match="not implemented by the CUDA backend"):
        backend.dispatch(fnn.ExecutablePlan([bogus], 256), arena, fnn.ShapeEnv())
    arena.close()


@pytest.mark.parametrize("quantize", [8, 4, "f8", "f4", "i4cb"])
def test_saved_plan_runs_through_runtime_without_requantizing(backend, tmp_path, quantize):
    """AotExecutor.save -> `.fnnc` + `.memory.json` -> Runtime.load on a CudaBackend -> run
    (src/backend/runtime.rs:65-151): same bits as the executor that compiled the plan, twice (the
    second run replays the plan without its WriteConst instructions)."""
    m, k, n = 5, 512, 192
    w, b, x = normal(70, (k, n), 0.02), normal(71, (n,), 0.01), normal(72, (m, k), 1.0)
    nodes = [{"op_type": "Gemm", "inputs": "[x, w, b]", "outputs": "[h]"},
             {"op_type": "Gelu", "inputs": "[h]", "outputs": "[y]"}]
    aot = fnn.AotExecutor(nodes, {"w": w, "b": b}, ["x"], ["y"], {"x": [m, k]}, quantize=quantize,
                          backend=backend)
    want = aot.forward({"x": x})["y"]
    aot.save(str(tmp_path / "m.fnnc"), str(tmp_path / "m.memory.json"))
    rt = fnn.Runtime.load(backend, str(tmp_path / "m.fnnc"), str(tmp_path / "m.memory.json"))
    try:
        for _ in range(2):
            got = np.frombuffer(rt.run([x.tobytes()])[0], np.float32).reshape(m, n)
            assert np.array_equal(got, want)
    finally:
        rt.close()


@pytest.mark.parametrize("quantize,fmt", [(8, orc.FMT_I8), ("f8", orc.FMT_F8)])
def test_onnx_file_with_torch_style_linear_layers(backend, quantize, fmt, tmp_path):
    """An ONNX file as PyTorch exports an MLP block -- Gemm(transB=1) + bias, SiLU as Sigmoid x Mul,
    a second Gemm, symbolic batch -- through `AotExecutor.from_onnx`: both weights land on the
    quantized MatMul with the epilogue fused, and the result follows the oracle."""
    import onnx_wire as ow
    k, h, n, m = 256, 512, 192, 5
    w1, b1 = normal(60, (h, k), 0.05), normal(61, (h,), 0.01)       # torch layout [out, in]
    w2, b2 = normal(62, (n, h), 0.05), normal(63, (n,), 0.01)
    nodes = [ow.node("Gemm", ["x", "fc1.weight", "fc1.bias"], ["h1"], "fc1", transB=1),
             ow.node("Sigmoid", ["h1"], ["s1"]), ow.node("Mul", ["h1", "s1"], ["a1"]),
             ow.node("Gemm", ["a1", "fc2.weight", "fc2.bias"], ["y"], "fc2", transB=1, alpha=1.0, beta=1.0)]
    path = tmp_path / "mlp.onnx"
    path.write_bytes(ow.model(nodes, {"fc1.weight": w1, "fc1.bias": b1, "fc2.weight": w2, "fc2.bias": b2},
                              [("x", ["batch", k])], ["y"], initializers_as_inputs=True))
    aot = fnn.AotExecutor.from_onnx(str(path), quantize=quantize, backend=backend)
    names = [i.kernel_name for i in aot.plan.instructions if isinstance(i, fnn.CallKernel)]
    assert [nm for nm in names if nm.startswith("matmul_")] == ["matmul_" + ("i8" if quantize == 8 else "f8")] * 2, names
    assert "silu_f32" not in names and "sigmoid_f32" not in names, names     # the activation is fused
    x = normal(64, (m, k), 1.0)
    got = aot.forward({"x": x})["y"]
    q1, q2 = orc.quantize_kn(fmt, np.ascontiguousarray(w1.T)), orc.quantize_kn(fmt, np.ascontiguousarray(w2.T))
    want = orc.qmatmul(q2, orc.qmatmul(q1, x, b1, orc.EPI_SILU), b2, orc.EPI_NONE)
    assert got.shape == (m, n)
    assert max_err_vs_rms(got, want) <= 1e-3
