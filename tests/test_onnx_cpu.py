"""ONNX entry: models are built with the wire-format writer (no `onnx` package here), decoded by the reader, translated
to LLH, compiled through the C ABI and executed by the CPU plan interpreter; results are compared with PyTorch eager."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import InterpreterCompiler
from llcompiler_b200.importer import onnx_wire as W
from oracle.models import max_rel_err


def _np(*shape, seed=0, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def test_wire_format_round_trip():
    w = _np(3, 5)
    data = W.build_model([("Gemm", ["x", "w"], ["y"], {"transB": 1, "alpha": 1.0}), ("MaxPool", ["y"], ["z"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]})],
                         {"w": w, "s": np.array([2, -1], dtype=np.int64)}, [("x", [4, 5])], [("z", ["B", 3])])
    g = W.parse_model(data)
    assert [(n.op_type, n.inputs, n.outputs) for n in g.nodes] == [("Gemm", ["x", "w"], ["y"]), ("MaxPool", ["y"], ["z"])]
    assert g.nodes[0].attrs == {"transB": 1, "alpha": 1.0} and g.nodes[1].attrs["pads"] == [1, 1, 1, 1]
    assert np.array_equal(g.initializers["w"], w) and list(g.initializers["s"]) == [2, -1]
    assert g.inputs[0].dims == [4, 5] and g.outputs[0].dims == ["B", 3]


def test_onnx_mlp():
    w1, b1, w2, b2 = _np(512, 784, scale=0.05), _np(512, seed=1), _np(10, 512, seed=2, scale=0.05), _np(10, seed=3)
    data = W.build_model([("Gemm", ["x", "w1", "b1"], ["h"], {"transB": 1}), ("Relu", ["h"], ["r"], {}), ("Gemm", ["r", "w2", "b2"], ["y"], {"transB": 1})],
                         {"w1": w1, "b1": b1, "w2": w2, "b2": b2}, [("x", [64, 784])], [("y", [64, 10])])
    comp = InterpreterCompiler()
    fn = comp.compile_onnx(data)
    x = torch.randn(64, 784)
    want = F.linear(F.relu(F.linear(x, torch.from_numpy(w1), torch.from_numpy(b1))), torch.from_numpy(w2), torch.from_numpy(b2))
    assert max_rel_err(fn(x), want) < 1e-5
    plan = comp.compiled[0].engine.text
    assert plan.count("step gemm") == 2 and "step eltwise" not in plan           # bias and ReLU ride in the epilogues


def test_onnx_residual_cnn():
    c1, c2, fc, fb = _np(16, 3, 3, 3, scale=0.2), _np(16, 16, 3, 3, seed=1, scale=0.1), _np(10, 16, seed=2, scale=0.2), _np(10, seed=3)
    g, bt, mu, var = np.abs(_np(16, seed=4)) + 0.5, _np(16, seed=5), _np(16, seed=6, scale=0.1), np.abs(_np(16, seed=7)) + 0.5
    nodes = [("Conv", ["x", "c1"], ["a"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 2]}),
             ("BatchNormalization", ["a", "g", "bt", "mu", "var"], ["b"], {"epsilon": 1e-5}), ("Relu", ["b"], ["c"], {}),
             ("MaxPool", ["c"], ["d"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 2]}),
             ("Conv", ["d", "c2"], ["e"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1]}), ("Add", ["e", "d"], ["f"], {}), ("Relu", ["f"], ["h"], {}),
             ("GlobalAveragePool", ["h"], ["p"], {}), ("Flatten", ["p"], ["q"], {"axis": 1}), ("Gemm", ["q", "fc", "fb"], ["y"], {"transB": 1})]
    data = W.build_model(nodes, {"c1": c1, "c2": c2, "g": g, "bt": bt, "mu": mu, "var": var, "fc": fc, "fb": fb}, [("x", [2, 3, 32, 32])], [("y", [2, 10])])
    fn = InterpreterCompiler().compile_onnx(data)
    x = torch.randn(2, 3, 32, 32)
    t = torch.from_numpy
    d = F.max_pool2d(F.relu(F.batch_norm(F.conv2d(x, t(c1), None, 2, 1), t(mu), t(var), t(g), t(bt), False, 0.0, 1e-5)), 3, 2, 1)
    h = F.relu(F.conv2d(d, t(c2), None, 1, 1) + d)
    want = F.linear(h.mean((2, 3)), t(fc), t(fb))
    assert max_rel_err(fn(x), want) < 1e-4


def test_onnx_refuses_what_it_does_not_cover():
    data = W.build_model([("LSTM", ["x"], ["y"], {})], {}, [("x", [2, 8])], [("y", [2, 8])])
    with pytest.raises(NotImplementedError, match="LSTM"):
        InterpreterCompiler().compile_onnx(data)


def test_onnx_symbolic_batch():
    """`dim_param` extents become symbols bound from the input at run time: one plan serves every batch size."""
    c1, fc, fb = _np(8, 3, 3, 3, scale=0.2), _np(10, 8 * 4 * 4, seed=2, scale=0.1), _np(10, seed=3)
    nodes = [("Conv", ["x", "c1"], ["a"], {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [2, 2]}), ("Relu", ["a"], ["b"], {}),
             ("MaxPool", ["b"], ["c"], {"kernel_shape": [2, 2], "strides": [2, 2]}), ("Flatten", ["c"], ["d"], {"axis": 1}),
             ("Gemm", ["d", "fc", "fb"], ["e"], {"transB": 1}), ("Reshape", ["e", "s"], ["y"], {})]
    data = W.build_model(nodes, {"c1": c1, "fc": fc, "fb": fb, "s": np.array([-1, 2, 5], dtype=np.int64)}, [("x", ["batch", 3, 16, 16])], [("y", ["batch", 2, 5])])
    comp = InterpreterCompiler()
    fn = comp.compile_onnx(data)
    assert 'func.input_symbol_0 = "batch"' in comp._mlir_module and "tensor<?x3x16x16xf32>" in comp._mlir_module
    t = torch.from_numpy
    for batch in (1, 5, 16):
        x = torch.randn(batch, 3, 16, 16, generator=torch.Generator().manual_seed(batch))
        want = F.linear(F.max_pool2d(F.relu(F.conv2d(x, t(c1), None, 2, 1)), 2, 2).flatten(1), t(fc), t(fb)).reshape(-1, 2, 5)
        got = fn(x)
        assert tuple(got.shape) == (batch, 2, 5) and max_rel_err(got, want) < 1e-4
    assert len(comp.compiled) == 1
