"""Host logic of the pipeline (fusion, quantization pass, memory plan, lowering), on CPU with a
recording stand-in for the device.  Mirrors the structural tests of the reference:
src/compiler/passes/quantization.rs:698-873, tests/quantized_pipeline.rs:608-620,
tests/memory_planning_tests.rs."""
import numpy as np
import pytest

import fastnn_b200 as fnn
from fastnn_b200 import _lib as L
from fastnn_b200.compiler import (GraphBuilder, GraphExecutor, TensorType, WeightDtype,
                                  eliminate_dead_code, fuse_operators, lower_to_plan, plan_memory,
                                  quantize_weights)
from fastnn_b200.backend import CallKernel
from helpers import normal


class RecordingBackend:
    """Implements the Backend trait surface without a device: records what it is given."""

    def __init__(self):
        self.arena = None
        self.dispatched = []

    def name(self):
        return "recording"

    def allocate_arena(self, total_bytes):
        self.arena = bytearray(total_bytes)
        return self.arena

    def compile(self, graph, memory_plan):
        return lower_to_plan(graph, memory_plan)

    def write_arena(self, arena, offset, data):
        arena[offset:offset + len(data)] = bytes(data)

    def read_arena(self, arena, offset, size):
        return bytes(arena[offset:offset + size])

    def dispatch(self, plan, arena, env):
        self.dispatched.append([type(i).__name__ if not hasattr(i, "kernel_name") else i.kernel_name
                                for i in plan.instructions])


def linear_graph(m, k, n, bias=False, act=None, residual=False):
    gb = GraphBuilder()
    x = gb.input_with_dims([m, k])
    w = gb.constant(normal(1, (k, n), 0.02), TensorType.new([k, n]))
    y = gb.matmul(x, w)
    if bias:
        y = gb.add(y, gb.constant(normal(2, (n,), 0.01), TensorType.new([n])))
    if act:
        y = getattr(gb, act)(y)
    if residual:
        r = gb.input_with_dims([m, n])
        y = gb.add(y, r)
    g = gb.to_graph()
    g.inputs = gb.recorded_input_ids()
    g.outputs = [y.node_id()]
    return g


def compile_graph(g, wd):
    ex = GraphExecutor(RecordingBackend())
    return ex.compile_with_weight_dtype(g, wd)


def kernels(plan):
    return [i.kernel_name for i in plan.instructions if isinstance(i, fnn.CallKernel)]


@pytest.mark.parametrize("wd,name", [(WeightDtype.I4, "matmul_i4"), (WeightDtype.I8, "matmul_i8"),
                                     (WeightDtype.F8x4, "matmul_f8"), (WeightDtype.F4x8, "matmul_f4"),
                                     (WeightDtype.I4Codebook, "matmul_i4")])
def test_kernel_name_and_meta_per_weight_dtype(wd, name):
    plan, mp, g = compile_graph(linear_graph(2, 64, 16), wd)
    assert kernels(plan) == [name]
    call = [i for i in plan.instructions if isinstance(i, fnn.CallKernel)][0]
    meta = call.weight_meta
    assert call.params[:3] == [2, 64, 16] and meta.shape == [16, 64]  # [N,K]: reversed
    if wd == WeightDtype.I4Codebook:
        assert meta.quant_block_size == 32 and len(meta.codebooks) == 1
        assert meta.scales.size == 16 * 2 and meta.zero_points.size == 0
    else:
        assert meta.quant_block_size == 0 and meta.scales.size == 16
    assert meta.bit_width == (8 if wd in (WeightDtype.I8, WeightDtype.F8x4) else 4)
    # the WriteConst payload is the reference byte stream: rows + 16 margin words
    wc = [i for i in plan.instructions if isinstance(i, fnn.WriteConst)][0]
    items = 4 if meta.bit_width == 8 else 8
    assert len(wc.data) == (16 * (64 // items) + 16) * 4 == wc.dst.size


def test_only_constant_weights_are_quantized():
    gb = GraphBuilder()
    x = gb.input_with_dims([2, 8])
    w = gb.input_with_dims([8, 4])  # a runtime input stays f32 (quantization.rs:47-89)
    y = gb.matmul(x, w)
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    quantize_weights(g, WeightDtype.I8)
    assert all(not n.output_type.dtype.is_quantized for n in g.nodes)
    with pytest.raises(fnn.BackendError, match="Unsupported"):
        lower_to_plan(g, plan_memory(g))  # f32 MatMul is not this backend's path


def test_fusion_matmul_add_act_and_op_act():
    g = linear_graph(2, 64, 16, bias=True, act="gelu")
    fuse_operators(g)
    mm = [n for n in g.nodes if n.opcode.value == "MatMul"]
    assert len(mm) == 1 and mm[0].attrs["fused_op"] == "MatMulAddGelu" and len(mm[0].inputs) == 3
    g = linear_graph(2, 64, 16, act="silu")
    fuse_operators(g)
    mm = [n for n in g.nodes if n.opcode.value == "MatMul"]
    assert mm[0].attrs["fused_op"] == "OpSilu" and len(g.nodes) == 3
    # bias without activation is not fused by the graph passes (no MatMul+Add-only fusion)
    g = linear_graph(2, 64, 16, bias=True)
    fuse_operators(g)
    assert [n.opcode.value for n in g.nodes].count("Add") == 1


def test_lowering_keeps_the_epilogue_the_cpu_backend_drops():
    plan, _, _ = compile_graph(linear_graph(2, 64, 16, bias=True, act="gelu"), WeightDtype.I8)
    call = [i for i in plan.instructions if isinstance(i, fnn.CallKernel)]
    assert len(call) == 1 and len(call[0].input_slices) == 3 and call[0].params[3] == L.EPI_GELU
    plan, _, _ = compile_graph(linear_graph(2, 64, 16, act="silu"), WeightDtype.I8)
    call = [i for i in plan.instructions if isinstance(i, fnn.CallKernel)]
    assert len(call) == 1 and len(call[0].input_slices) == 2 and call[0].params[3] == L.EPI_SILU
    # bias-only add of a 1-D constant folds into the matmul kernel (C1's MatMul+Add)
    plan, _, _ = compile_graph(linear_graph(8, 64, 16, bias=True), WeightDtype.I4)
    assert kernels(plan) == ["matmul_i4"]
    # a residual add (rank 2) stays a separate elementwise instruction
    plan, _, _ = compile_graph(linear_graph(2, 64, 16, residual=True), WeightDtype.I4)
    assert kernels(plan) == ["matmul_i4", "add_f32"]


def test_memory_plan_alignment_persistence_and_inplace_reuse():
    g = linear_graph(4, 64, 16, residual=True)
    quantize_weights(g, WeightDtype.I8)
    mp = plan_memory(g)
    assert all(s.offset % 64 == 0 for s in mp.slots.values())
    spans = sorted((s.offset, s.offset + s.size, nid) for nid, s in mp.slots.items())
    mm = [n for n in g.nodes if n.opcode.value == "MatMul"][0]
    add = [n for n in g.nodes if n.opcode.value == "Add"][0]
    assert mp.slots[add.id].offset == mp.slots[mm.id].offset      # in-place elementwise reuse
    others = [(a, b) for a, b, nid in spans if nid != add.id]
    for (a0, b0), (a1, b1) in zip(others, others[1:]):
        assert b0 <= a1, "live slots overlap"
    assert mp.total_size >= max(b for _, b, _ in spans)


def test_static_plan_drops_writeconst_after_first_execute():
    be = RecordingBackend()
    ex = GraphExecutor(be)
    g = linear_graph(2, 64, 16)
    plan, mp, cg = ex.compile_with_weight_dtype(g, WeightDtype.I8)
    x = normal(3, (2, 64), 1.0).tobytes()
    ex.execute(cg, plan, mp, [x])
    ex.execute(cg, plan, mp, [x])
    assert be.dispatched[0] == ["WriteConst", "matmul_i8"] and be.dispatched[1] == ["matmul_i8"]


def test_symbolic_batch_resolves_from_input_bytes():
    gb = GraphBuilder()
    x = gb.input_with_dims(["d1", 64])
    w = gb.constant(normal(1, (64, 16), 0.02), TensorType.new([64, 16]))
    y = gb.matmul(x, w)
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    env = GraphExecutor.shape_env_from_inputs(g, [bytes(5 * 64 * 4)])
    assert env["d1"] == 5
    plan, mp, cg = compile_graph(g, WeightDtype.I8)
    call = [i for i in plan.instructions if isinstance(i, fnn.CallKernel)][0]
    assert call.param_dims == ["d1", 64, 16]
    assert fnn.backend.resolve_params(call.params, call.param_dims, env, 3) == [5, 64, 16]
    with pytest.raises(fnn.BackendError):
        GraphExecutor.shape_env_from_inputs(g, [bytes(5 * 64 * 4 + 4)])


@pytest.mark.parametrize("shape,rows", [(["d1", 8, 64], 40), ([4, "d1", 64], 20), ([3, 2, 64], 6)])
def test_batch_rows_are_the_product_of_all_leading_dims(shape, rows):
    """A symbolic leading dimension next to other leading dimensions: M = their product."""
    gb = GraphBuilder()
    x = gb.input_with_dims(shape)
    w = gb.constant(normal(1, (64, 16), 0.02), TensorType.new([64, 16]))
    y = gb.matmul(x, w)
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    plan, mp, cg = compile_graph(g, WeightDtype.I8)
    call = [i for i in plan.instructions if isinstance(i, fnn.CallKernel)][0]
    env = fnn.ShapeEnv({"d1": 5})
    assert fnn.backend.resolve_params(call.params, call.param_dims, env, 3) == [rows, 64, 16]


def test_tighten_shrinks_symbolic_slots_and_the_arena():
    """memory_planning.rs:44-236 / executor.rs:1194-1284: at d1 = 3 an activation slot holds 3 rows,
    not SYMBOL_DIM_MAX; offsets stay; a larger batch later gets a larger arena and its constants again."""
    from fastnn_b200.compiler import tighten, tighten_slices
    gb = GraphBuilder()
    x = gb.input_with_dims(["d1", 64])
    y = gb.silu(gb.matmul(x, gb.constant(normal(1, (64, 16), 0.02), TensorType.new([64, 16]))))
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    be = RecordingBackend()
    ex = GraphExecutor(be)
    plan, mp, cg = ex.compile_with_weight_dtype(g, WeightDtype.I8)
    env = fnn.ShapeEnv({"d1": 3})
    tight = tighten(mp, cg, env)
    assert {k: v.offset for k, v in tight.slots.items()} == {k: v.offset for k, v in mp.slots.items()}
    out_id = cg.outputs[0]
    assert mp.slots[out_id].size == fnn.backend.SYMBOL_DIM_MAX * 16 * 4 and tight.slots[out_id].size == 3 * 16 * 4
    assert tight.total_size < mp.total_size
    tplan = tighten_slices(plan, mp, tight, env)
    call = [i for i in tplan.instructions if isinstance(i, fnn.CallKernel)][0]
    assert call.params[:3] == [3, 64, 16] and call.output_slice.size == 3 * 16 * 4
    ex.execute(cg, plan, mp, [bytes(3 * 64 * 4)])
    small = len(be.arena)
    assert small == tight.total_size < mp.total_size
    ex.execute(cg, plan, mp, [bytes(2 * 64 * 4)])
    assert len(be.arena) == small and be.dispatched[-1] == ["matmul_i8"]          # constants stay
    ex.execute(cg, plan, mp, [bytes(50 * 64 * 4)])
    assert len(be.arena) > small and be.dispatched[-1][0] == "WriteConst"          # regrown: constants again


def test_quantize_argument_validation():
    assert WeightDtype.from_quantize(4) == WeightDtype.I4
    assert WeightDtype.from_quantize("i4cb") == WeightDtype.I4Codebook
    assert WeightDtype.from_quantize(None) == WeightDtype.F32
    with pytest.raises(ValueError):
        WeightDtype.from_quantize(5)
    with pytest.raises(ValueError):
        WeightDtype.from_quantize("fp16")
    gb = GraphBuilder()
    with pytest.raises(fnn.BackendError):
        gb.compile_and_execute_with_quantize([], RecordingBackend(), [], 3)


# ---- rms_norm / softmax plan instructions (host side: lowering and the oracle's restatement) ----------


def test_rms_norm_and_softmax_lower_to_the_reference_kernel_names():
    import struct
    gb = GraphBuilder()
    x = gb.input(["batch", 8])
    w = gb.constant(np.linspace(0.5, 1.5, 8, dtype=np.float32).tobytes(), TensorType.new([8]))
    y = gb.softmax(gb.rms_norm(x, w, 1e-6), -1)
    graph = gb.to_graph()
    graph.inputs, graph.outputs = gb.recorded_input_ids(), [y.node_id()]
    mp = plan_memory(graph)
    plan = lower_to_plan(graph, mp)
    calls = [i for i in plan.instructions if isinstance(i, CallKernel)]
    assert [c.kernel_name for c in calls] == ["rms_norm", "softmax"]
    assert calls[0].params[0] == struct.unpack("<I", struct.pack("<f", 1e-6))[0]   # eps as f32 bits
    assert calls[0].params[1] == 8 and len(calls[0].input_slices) == 2
    assert calls[1].params == [8, 1] and calls[1].param_dims[:2] == [8, 1]


def test_softmax_stride_for_an_inner_axis():
    gb = GraphBuilder()
    x = gb.input([2, 5, 3])
    y = gb.softmax(x, 1)
    graph = gb.to_graph()
    graph.inputs, graph.outputs = gb.recorded_input_ids(), [y.node_id()]
    plan = lower_to_plan(graph, plan_memory(graph))
    call = [i for i in plan.instructions if isinstance(i, CallKernel)][0]
    assert call.params == [5, 3]


def test_oracle_rms_norm_matches_the_reference_fused_test_vector():
    """tests/residual_add_norm.rs:327-355 (hidden row size 4, batch 2): x = main + residual."""
    import oracle as orc
    main = np.array([1.0, -2.0, 3.5, -4.5, 2.25, -1.0, 0.5, 3.0], np.float32)
    residual = np.array([-0.25, 0.5, -1.5, 2.0, 1.25, -0.75, 2.5, -3.5], np.float32)
    weight = np.array([0.75, -1.25, 1.5, 0.5], np.float32)
    x = (main + residual).reshape(2, 4)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * weight
    got = orc.rms_norm(x, weight, 1e-5)
    assert np.allclose(got, want, rtol=0, atol=1e-5)
    # the unfused dispatch arm as written takes rows of len / w_len = 2 elements instead
    as_written = orc.rms_norm(x, weight, 1e-5, orc.MODE_AS_WRITTEN)
    assert not np.allclose(as_written, want, atol=1e-3)


def test_oracle_softmax_rows_sum_to_one_on_any_axis():
    import oracle as orc
    x = np.random.default_rng(3).standard_normal((2, 5, 3)).astype(np.float32) * 4
    for axis in (0, 1, 2, -1):
        s = orc.softmax(x, axis)
        e = np.exp(x - x.max(axis, keepdims=True))
        assert np.allclose(s, e / e.sum(axis, keepdims=True), atol=1e-6)
        assert np.allclose(s.sum(axis), 1.0, atol=1e-5)


def test_add_feeding_a_norm_becomes_the_fused_residual_kernel():
    """Kernel names and input order [residual, main, weight, bias] of the reference's
    FusedResidualAddNorm lowering (src/backend/cpu/mod.rs:2424-2500)."""
    for norm in ("rms", "layer"):
        gb = GraphBuilder()
        main, res = gb.input([2, 4]), gb.input([2, 4])
        w = gb.constant(np.ones(4, np.float32).tobytes(), TensorType.new([4]))
        b = gb.constant(np.zeros(4, np.float32).tobytes(), TensorType.new([4]))
        s = gb.add(main, res)
        y = gb.rms_norm(s, w, 1e-5) if norm == "rms" else gb.layer_norm(s, w, b, 1e-5)
        graph = gb.to_graph()
        graph.inputs, graph.outputs = gb.recorded_input_ids(), [y.node_id()]
        mp = plan_memory(graph)
        calls = [i for i in lower_to_plan(graph, mp).instructions if isinstance(i, CallKernel)]
        assert [c.kernel_name for c in calls] == [f"fused_residual_add_{norm}_norm"]
        assert len(calls[0].input_slices) == (3 if norm == "rms" else 4)
        assert calls[0].params[1] == 4
        # residual first, main second
        assert calls[0].input_slices[0].offset == mp.slots[res.node_id()].offset
        assert calls[0].input_slices[1].offset == mp.slots[main.node_id()].offset


def test_layer_norm_alone_lowers_to_norm_f32():
    gb = GraphBuilder()
    x = gb.input([3, 8])
    w = gb.constant(np.ones(8, np.float32).tobytes(), TensorType.new([8]))
    b = gb.constant(np.zeros(8, np.float32).tobytes(), TensorType.new([8]))
    y = gb.layer_norm(x, w, b, 1e-5)
    graph = gb.to_graph()
    graph.inputs, graph.outputs = gb.recorded_input_ids(), [y.node_id()]
    calls = [i for i in lower_to_plan(graph, plan_memory(graph)).instructions if isinstance(i, CallKernel)]
    assert calls[0].kernel_name == "norm_f32" and calls[0].params[1] == 0 and calls[0].params[2] == 8


def test_oracle_layer_norm_matches_the_reference_fused_test_vector():
    """tests/residual_add_norm.rs:357-390: main + residual, weight and bias of length 4."""
    import oracle as orc
    main = np.array([0.5, -1.0, 2.0, -3.0, 1.5, 2.5, -0.75, -1.25], np.float32).reshape(2, 4)
    residual = np.array([1.0, 0.25, -0.5, 1.75, -2.0, 0.5, 1.25, -0.25], np.float32).reshape(2, 4)
    weight = np.array([1.25, 0.75, -0.5, 1.5], np.float32)
    bias = np.array([0.1, -0.2, 0.3, -0.4], np.float32)
    x = (main + residual).astype(np.float64)
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * weight + bias
    got = orc.layer_norm(main, weight, bias, 1e-5, residual)
    assert np.allclose(got, want, atol=1e-5)
