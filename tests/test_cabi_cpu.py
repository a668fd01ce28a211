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
    ref = "/root/reference/test/Dialect/LLH/symbol_infer/infer_symbol_shape.mlir"
    if not os.path.exists(ref):
        pytest.skip("reference tree not present")
    out = _capi.run_pass(open(ref).read(), "parse")
    assert out.count("func.func") >= 20
    assert _capi.run_pass(out, "parse") == out
