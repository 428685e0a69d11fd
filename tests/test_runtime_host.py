"""The `.fnnc` + `.memory.json` pair (src/backend/runtime.rs:65-151): bincode layout of
`ExecutablePlan` checked byte for byte on a hand-built plan, round trip of a compiled quantized
plan, and `Runtime.run` against a recording stand-in for the device."""
import json
import struct

import numpy as np
import pytest

import fastnn_b200 as fnn
from fastnn_b200 import _lib as L
from fastnn_b200.backend import BufferSlice, CallKernel, ExecutablePlan, Fill, MemCopy, QuantizedWeightMeta, WriteConst
from fastnn_b200.compiler import WeightDtype
from fastnn_b200.runtime import Runtime, memory_plan_from_json, memory_plan_to_json, plan_from_bytes, plan_to_bytes
from helpers import normal
from test_compiler_host import RecordingBackend, linear_graph, compile_graph


def u64(v):
    return struct.pack("<Q", v)


def test_bincode_layout_of_every_instruction_variant():
    """bincode 1.3 defaults applied to src/backend/mod.rs:27-107 by hand."""
    meta = QuantizedWeightMeta(bit_width=4, scales=np.array([0.5, 2.0], np.float32),
                               zero_points=np.zeros(0, np.float32), shape=[2, 32], quant_block_size=32,
                               codebooks=[np.arange(16, dtype=np.float32)], fmt=L.FMT_I4CB)
    plan = ExecutablePlan([
        WriteConst(BufferSlice(64, 3), b"\x01\x02\x03"),
        Fill(BufferSlice(128, 8), 1.5),
        MemCopy(BufferSlice(0, 4), BufferSlice(8, 4)),
        CallKernel("matmul_i4", [BufferSlice(0, 256), BufferSlice(64, 96)], BufferSlice(512, 16),
                   [2, 32, 2, 1], node_id=7, param_dims=["d1", 32, 2], weight_meta=meta),
        CallKernel("add_f32", [], BufferSlice(1, 2), [], node_id=None, param_dims=None, weight_meta=None,
                   secondary_output_slice=BufferSlice(3, 4)),
    ], 1024, [0, 0, 1, 2, 3])
    want = b"".join([
        u64(5),
        struct.pack("<I", 3), u64(64), u64(3), u64(3), b"\x01\x02\x03",
        struct.pack("<I", 2), u64(128), u64(8), struct.pack("<f", 1.5),
        struct.pack("<I", 1), u64(0), u64(4), u64(8), u64(4),
        struct.pack("<I", 0), u64(9), b"matmul_i4", u64(2), u64(0), u64(256), u64(64), u64(96),
        u64(512), u64(16), b"\x00", u64(4), u64(2), u64(32), u64(2), u64(1), b"\x01", u64(7),
        b"\x01", u64(3), struct.pack("<I", 1), u64(2), b"d1", struct.pack("<I", 0), u64(32),
        struct.pack("<I", 0), u64(2),
        b"\x01", u64(4), u64(2), struct.pack("<2f", 0.5, 2.0), u64(0), u64(2), u64(2), u64(32), u64(32),
        u64(1), struct.pack("<16f", *range(16)),
        struct.pack("<I", 0), u64(7), b"add_f32", u64(0), u64(1), u64(2), b"\x01", u64(3), u64(4), u64(0),
        b"\x00", b"\x00", b"\x00",
        u64(1024), u64(5), u64(0), u64(0), u64(1), u64(2), u64(3),
    ])
    got = plan_to_bytes(plan)
    assert got == want
    back = plan_from_bytes(got)
    assert plan_to_bytes(back) == want
    call = back.instructions[3]
    assert call.weight_meta.fmt == L.FMT_I4CB and call.param_dims == ["d1", 32, 2]
    with pytest.raises(fnn.BackendError, match="truncated"):
        plan_from_bytes(got[:-3])
    with pytest.raises(fnn.BackendError, match="trailing"):
        plan_from_bytes(got + b"\0")


@pytest.mark.parametrize("wd,kernel,fmt", [(WeightDtype.I8, "matmul_i8", L.FMT_I8), (WeightDtype.I4, "matmul_i4", L.FMT_I4),
                                           (WeightDtype.F8x4, "matmul_f8", L.FMT_F8), (WeightDtype.F4x8, "matmul_f4", L.FMT_F4),
                                           (WeightDtype.I4Codebook, "matmul_i4", L.FMT_I4CB)])
def test_compiled_quantized_plan_round_trips_with_its_weights(tmp_path, wd, kernel, fmt):
    plan, mp, cg = compile_graph(linear_graph(3, 64, 16, bias=True, act="silu"), wd)
    rt = Runtime(RecordingBackend(), plan, mp)
    rt.save(str(tmp_path / "m.fnnc"), str(tmp_path / "m.memory.json"))
    rt2 = Runtime.load(RecordingBackend(), str(tmp_path / "m.fnnc"), str(tmp_path / "m.memory.json"))
    a = [i for i in plan.instructions if isinstance(i, CallKernel)][0]
    b = [i for i in rt2.plan.instructions if isinstance(i, CallKernel)][0]
    assert b.kernel_name == kernel and b.weight_meta.fmt == fmt        # format recovered from name + codebooks
    assert b.params == a.params and b.input_slices == a.input_slices and b.output_slice == a.output_slice
    assert np.array_equal(b.weight_meta.scales, a.weight_meta.scales)
    assert np.array_equal(b.weight_meta.zero_points, a.weight_meta.zero_points)
    assert [c.tolist() for c in b.weight_meta.codebooks] == [np.asarray(c).tolist() for c in a.weight_meta.codebooks]
    consts_a = [(i.dst, i.data) for i in plan.instructions if isinstance(i, WriteConst)]
    consts_b = [(i.dst, i.data) for i in rt2.plan.instructions if isinstance(i, WriteConst)]
    assert consts_a == consts_b                                        # packed bytes incl. the margin words
    d = json.loads((tmp_path / "m.memory.json").read_text())
    assert set(d) == {"total_size", "slots", "secondary_slots", "outputs", "tightened_params"}
    assert d["total_size"] == mp.total_size and d["outputs"] == [o for o, _ in mp.outputs]
    again = memory_plan_from_json(memory_plan_to_json(mp))
    assert {k: (v.offset, v.size) for k, v in again.slots.items()} == {k: (v.offset, v.size) for k, v in mp.slots.items()}


def test_runtime_run_writes_inputs_first_dispatches_and_reads_outputs():
    plan, mp, cg = compile_graph(linear_graph(2, 64, 16), WeightDtype.I8)
    be = RecordingBackend()
    rt = Runtime(be, plan, mp)
    x = normal(3, (2, 64), 1.0).tobytes()
    outs = rt.run([x])
    first = min(mp.slots.values(), key=lambda s: s.offset)
    assert bytes(be.arena[first.offset:first.offset + len(x)]) == x      # inputs go to the first slots by offset
    assert len(outs) == 1 and len(outs[0]) == 2 * 16 * 4
    rt.run([x])
    assert be.dispatched[0] == ["WriteConst", "matmul_i8"] and be.dispatched[1] == ["matmul_i8"]


def test_symbolic_batch_product_cannot_be_saved():
    gb = fnn.GraphBuilder()
    x = gb.input_with_dims(["d1", 8, 64])
    y = gb.matmul(x, gb.constant(normal(1, (64, 16), 0.02), fnn.TensorType.new([64, 16])))
    g = gb.to_graph()
    g.inputs, g.outputs = gb.recorded_input_ids(), [y.node_id()]
    plan, mp, cg = compile_graph(g, WeightDtype.I8)
    with pytest.raises(fnn.BackendError, match="specialised"):
        plan_to_bytes(plan)
