"""The C-ABI library without a GPU: it loads, exports every symbol the headers declare, reports
errors through status codes, and refuses to run without a CUDA device (there is no CPU path)."""
import ctypes
import os
import re

import pytest

from llcompiler_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(llc_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported():
    lib = _capi.lib()
    declared = _declared("llc_runtime.h") | _declared("llc_cuda.h")
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(_capi.EXPORTED_SYMBOLS)


def test_parse_and_lowering_errors_are_status_codes():
    with pytest.raises(_capi.LlcError) as e:
        _capi.run_pass("module { func.func @main( -> ", "parse")
    assert e.value.code == 1
    bad_op = 'module { func.func @main(%a: tensor<2xf32>) -> tensor<2xf32> attributes {entrance} {\n %0 = "llh.frobnicate"(%a) : (tensor<2xf32>) -> tensor<2xf32>\n return %0 : tensor<2xf32>\n } }'
    with pytest.raises(_capi.LlcError) as e:
        _capi.run_pass(bad_op, "lower")
    assert e.value.code == 2 and "frobnicate" in str(e.value)
    with pytest.raises(_capi.LlcError) as e:
        _capi.compile_text(bad_op.replace("llh.frobnicate", "llh.abs"), mode="training")
    assert e.value.code == 2 and "inference" in str(e.value)


def test_load_without_a_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    text = 'module { func.func @main(%a: tensor<2xf32>) -> tensor<2xf32> attributes {entrance} {\n %0 = "llh.abs"(%a) : (tensor<2xf32>) -> tensor<2xf32>\n return %0 : tensor<2xf32>\n } }'
    path = _capi.compile_text(text)
    lib = _capi.lib()
    exe = ctypes.c_void_p()
    rc = lib.llc_load(path.encode(), 0, ctypes.byref(exe))
    assert rc == 5 and b"no CUDA device" in lib.llc_last_error()
    with pytest.raises(RuntimeError):
        from llcompiler_b200.executor import Torch_ExecutionEngine
        Torch_ExecutionEngine(path)


def test_plan_text_round_trips_through_the_reference_lit_inputs():
    # every LLH module of the reference's own symbol-inference lit file parses and re-prints
    from reference_tree import reference_path
    ref = reference_path("test", "Dialect", "LLH", "symbol_infer", "infer_symbol_shape.mlir")
    if not ref or not os.path.exists(ref):
        pytest.skip("reference tree not present")
    out = _capi.run_pass(open(ref).read(), "parse")
    assert out.count("func.func") >= 20
    assert _capi.run_pass(out, "parse") == out


def test_tensor_buffer_view_get_tool_and_the_package_alias():
    """The rest of the reference's module surface (src/Pybind/Entrance.cpp:71-91, :113): a host Tensor exposes the
    buffer protocol and to_numpy(), executor.get_tool names the in-process tools, and the package imports under the
    reference's name."""
    import numpy as np
    import torch
    from llcompiler_.executor import get_tool
    from llcompiler_.tensor import Tensor
    t = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)[:, ::2]           # a strided host view
    T = Tensor(t.data_ptr(), t.data_ptr(), 4, t.storage_offset(), list(t.shape), list(t.stride()))
    assert np.array_equal(T.to_numpy(), t.numpy()) and np.array_equal(np.asarray(memoryview(T)), t.numpy())
    with pytest.raises(RuntimeError):
        Tensor(0, 0, 4, 0, [1], [1], 0).to_numpy()                               # device memory has no buffer view
    assert "llc_opt" in get_tool("llc-opt")
    with pytest.raises(IndexError):
        get_tool("opt")
    import llcompiler
    from llcompiler.compiler import LLCompiler
    from llcompiler_b200.compiler import LLCompiler as Impl
    assert LLCompiler is Impl and llcompiler.LLCompiler is Impl
