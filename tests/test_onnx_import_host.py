"""ONNX import on the host: wire-format reader and the rewrites that put exporter output on the
quantized MatMul (no GPU)."""
import numpy as np
import pytest

import onnx_wire as ow
from fastnn_b200.backend import BackendError
from fastnn_b200.onnx_import import read_onnx, to_aot_arguments


def rng(seed, shape, s=1.0):
    return (np.random.Generator(np.random.Philox(seed)).standard_normal(shape) * s).astype(np.float32)


def linear_model(trans_b=1, alpha=1.0, beta=1.0, batch="batch"):
    w, b = rng(1, (24, 16)), rng(2, (24,))         # torch layout [N, K]
    w_file = w if trans_b else np.ascontiguousarray(w.T)
    attrs = {"transB": trans_b}
    if alpha != 1.0:
        attrs["alpha"] = alpha
    if beta != 1.0:
        attrs["beta"] = beta
    nodes = [ow.node("Gemm", ["x", "fc.weight", "fc.bias"], ["h"], "fc", **attrs),
             ow.node("Sigmoid", ["h"], ["s"], "sig"),
             ow.node("Mul", ["h", "s"], ["y"], "mul")]
    data = ow.model(nodes, {"fc.weight": w_file, "fc.bias": b}, [("x", [batch, 16])], ["y"],
                    initializers_as_inputs=True)
    return data, w, b


def test_reader_decodes_nodes_initializers_and_shapes():
    data, w, b = linear_model()
    m = read_onnx(data)
    assert [n.op_type for n in m.nodes] == ["Gemm", "Sigmoid", "Mul"]
    assert m.nodes[0].inputs == ["x", "fc.weight", "fc.bias"] and m.nodes[0].attrs["transB"] == 1
    assert m.inputs == [("x", ["batch", 16])]       # initializers listed as inputs are not inputs
    assert m.outputs == ["y"]
    assert np.array_equal(m.initializers["fc.weight"], w) and np.array_equal(m.initializers["fc.bias"], b)


@pytest.mark.parametrize("raw", [True, False])
def test_tensor_payload_forms(raw):
    a = rng(3, (3, 5))
    i = np.arange(-3, 4, dtype=np.int64)
    d = np.linspace(-1, 1, 6).reshape(2, 3)
    data = ow.model([ow.node("Relu", ["x"], ["y"])],
                    {"a": ow.tensor("a", a, raw), "i": ow.tensor("i", i, raw), "d": ow.tensor("d", d, raw)},
                    [("x", [2, 2])], ["y"])
    m = read_onnx(data)
    assert np.array_equal(m.initializers["a"], a)
    assert np.array_equal(m.initializers["i"], i) and m.initializers["i"].dtype == np.int64
    assert np.array_equal(m.initializers["d"], d)


def test_gemm_transb_is_folded_into_the_constant_and_silu_is_recognised():
    data, w, b = linear_model(trans_b=1)
    nodes, params, ins, outs, shapes = to_aot_arguments(read_onnx(data))
    assert [n["op_type"] for n in nodes] == ["Gemm", "Silu"]
    assert nodes[0]["transB"] == "0" and nodes[0]["inputs"] == "[x, fc.weight, fc.bias]"
    assert nodes[1]["inputs"] == "[h]" and nodes[1]["outputs"] == "[y]"
    assert params["fc.weight"].shape == (16, 24) and np.array_equal(params["fc.weight"], w.T)
    assert ins == ["x"] and outs == ["y"] and shapes == {"x": [-1, 16]}


def test_alpha_and_beta_fold_into_constants():
    data, w, b = linear_model(trans_b=0, alpha=0.5, beta=2.0, batch=4)
    nodes, params, _, _, shapes = to_aot_arguments(read_onnx(data))
    assert np.array_equal(params["fc.weight"], (w.T * np.float32(0.5)).astype(np.float32))
    assert np.array_equal(params["fc.bias"], (b * np.float32(2.0)).astype(np.float32))
    assert shapes == {"x": [4, 16]}


def test_input_shapes_override_and_symbols_number_per_name():
    nodes = [ow.node("Add", ["a", "b"], ["y"])]
    data = ow.model(nodes, {}, [("a", ["n", "seq", 8]), ("b", ["n", "seq", 8])], ["y"])
    _, _, ins, _, shapes = to_aot_arguments(read_onnx(data))
    assert ins == ["a", "b"] and shapes == {"a": [-1, -2, 8], "b": [-1, -2, 8]}
    _, _, _, _, shapes = to_aot_arguments(read_onnx(data), {"a": [2, 3, 8]})
    assert shapes["a"] == [2, 3, 8] and shapes["b"] == [-1, -2, 8]


def test_constant_nodes_become_parameters_and_identity_disappears():
    w = rng(5, (8, 4))
    nodes = [ow.node("Constant", [], ["w"], value=w), ow.node("Dropout", ["x"], ["xd"]),
             ow.node("MatMul", ["xd", "w"], ["h"]), ow.node("Identity", ["h"], ["y"])]
    data = ow.model(nodes, {}, [("x", [2, 8])], ["y"])
    out_nodes, params, _, outs, _ = to_aot_arguments(read_onnx(data))
    assert [n["op_type"] for n in out_nodes] == ["MatMul"] and out_nodes[0]["inputs"] == "[x, w]"
    assert np.array_equal(params["w"], w) and outs == ["h"]


def test_refusals():
    with pytest.raises(BackendError):
        read_onnx(b"\x08\x08")                                  # no graph
    data = ow.model([ow.node("Conv", ["x", "w"], ["y"])], {"w": rng(6, (1, 1, 1, 1))}, [("x", [1, 1, 4, 4])], ["y"])
    with pytest.raises(BackendError, match="Conv"):
        to_aot_arguments(read_onnx(data))
    data = ow.model([ow.node("Gemm", ["x", "w"], ["y"], transA=1)], {"w": rng(7, (4, 4))}, [("x", [4, 4])], ["y"])
    with pytest.raises(BackendError, match="transA"):
        to_aot_arguments(read_onnx(data))
    whole = linear_model()[0]
    with pytest.raises(BackendError):
        read_onnx(whole[:len(whole) // 2])                       # cut in the middle of the graph
