"""The LLH-level rewrites behind llc_run_pass on inline text (no reference tree needed): decompose-ops
(src/Dialect/LLH/Transforms/DecomposeOps.cpp:125-144), transform-layout (TransformLayout.cpp:141-198), cse, the folders
(canonicalize, inline) and unload-and-bind-encoding (UnloadAndBindEncoding.cpp).  Each rewritten module is also run
through the lowering and the CPU plan interpreter where it computes something, and compared with eager."""
import re

import torch

from llcompiler_b200 import _capi

BN = '''
func.func @bn(%arg0: tensor<2x3x8x8xf32>, %arg1: tensor<3xf32>, %arg2: tensor<3xf32>, %arg3: tensor<3xf32>, %arg4: tensor<3xf32>) -> (tensor<2x3x8x8xf32>) attributes {entrance} {
  %0 = "llh.batch_norm_inference"(%arg0, %arg1, %arg2, %arg3, %arg4) <{epsilon = 1.000000e-05 : f64, feature_index = 1 : i64, momentum = 1.000000e-01 : f64}> : (tensor<2x3x8x8xf32>, tensor<3xf32>, tensor<3xf32>, tensor<3xf32>, tensor<3xf32>) -> tensor<2x3x8x8xf32>
  return %0 : tensor<2x3x8x8xf32>
}
'''


def _ops(text):
    return re.findall(r'= "(llh\.[a-z_]+)"', text)


def test_decompose_ops_spells_batch_norm_out_in_the_reference_order():
    out = _capi.run_pass(BN, "decompose-ops")
    assert "batch_norm_inference" not in out
    # stddev = sqrt(var + eps); ((x - mean) * scale) / stddev + bias, every per-channel operand reshaped and broadcast
    tail = [o for o in _ops(out) if o in ("llh.sqrt", "llh.sub", "llh.mul", "llh.div", "llh.add")]
    assert tail == ["llh.add", "llh.sqrt", "llh.sub", "llh.mul", "llh.div", "llh.add"]
    assert out.count('"llh.reshape"') == 4 and out.count('"llh.broadcast_to"') == 4 and "tensor<1x3x1x1xf32>" in out
    assert "dense<1.000000e-05> : tensor<1xf32>" in out                      # epsilon in the tensor's element type


def test_decomposed_batch_norm_computes_batch_norm():
    from oracle.plan_interp import PlanInterpreter
    plan = _capi.run_pass(BN, "decompose-ops,lower").split("// -----")[0]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 3, 8, 8, generator=g)
    scale, bias, mean = (torch.randn(3, generator=g) for _ in range(3))
    var = torch.rand(3, generator=g) + 0.5
    got = PlanInterpreter(plan).run([x, scale, bias, mean, var])[0]
    want = torch.nn.functional.batch_norm(x, mean, var, scale, bias, False, 0.1, 1e-5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_transform_layout_moves_a_convolution_to_channel_last():
    text = '''
func.func @conv(%arg0: tensor<2x3x8x8xf32>) -> (tensor<2x4x6x6xf32>) attributes {entrance} {
  %0 = "llh.weight"() <{weight_file = "w.npy"}> : () -> tensor<4x3x3x3xf32>
  %1 = "llh.conv"(%arg0, %0) <{dilation = array<i64: 1, 1>, group = 1 : i64, kernel_shape = array<i64: 3, 3>, layout = #llh.Layout<NCHW>, pad = array<i64: 0, 0, 0, 0>, stride = array<i64: 1, 1>}> : (tensor<2x3x8x8xf32>, tensor<4x3x3x3xf32>) -> tensor<2x4x6x6xf32>
  return %1 : tensor<2x4x6x6xf32>
}
'''
    out = _capi.run_pass(text, "transform-layout")
    assert _ops(out) == ["llh.weight", "llh.transpose", "llh.transpose", "llh.conv", "llh.transpose"]
    assert "layout = #llh.Layout<NHWC>" in out and "weight_layout = #llh.Layout<FHWC>" in out
    assert "perms = array<i64: 0, 2, 3, 1>" in out and "perms = array<i64: 0, 3, 1, 2>" in out
    assert "-> tensor<2x6x6x4xf32>" in out and "return %4 : tensor<2x4x6x6xf32>" in out


CSE = '''
func.func @cse(%arg0: tensor<4x4xf32>) -> (tensor<4x4xf32>) attributes {entrance} {
  %c = "llh.constant"() <{value = 2 : i64}> : () -> i64
  %d = "llh.constant"() <{value = 2 : i64}> : () -> i64
  %0 = "llh.add"(%arg0, %arg0) : (tensor<4x4xf32>, tensor<4x4xf32>) -> tensor<4x4xf32>
  %1 = "llh.add"(%arg0, %arg0) : (tensor<4x4xf32>, tensor<4x4xf32>) -> tensor<4x4xf32>
  %2 = "llh.mul"(%0, %1) : (tensor<4x4xf32>, tensor<4x4xf32>) -> tensor<4x4xf32>
  %a = "llh.add"(%c, %d) : (i64, i64) -> i64
  %3 = "llh.reshape"(%2, %a, %a) : (tensor<4x4xf32>, i64, i64) -> tensor<4x4xf32>
  return %3 : tensor<4x4xf32>
}
'''


def test_cse_merges_equal_operations():
    out = _capi.run_pass(CSE, "cse")
    assert out.count('"llh.constant"') == 1 and out.count('"llh.add"(%arg0, %arg0)') == 1
    assert '"llh.mul"(%1, %1)' in out and '"llh.reshape"(%2, %3, %3)' in out


def test_folders_remove_a_reshape_to_the_same_shape():
    out = _capi.run_pass(CSE, "canonicalize,inline")
    assert "llh.reshape" not in out and "llh.constant" not in out          # 2 + 2 folds, the reshape to 4 x 4 is the identity
    assert out.count('"llh.add"') == 2 and "return %2" in out


def test_unload_and_bind_encoding_moves_encodings_into_bind_ops():
    text = '''
func.func @enc(%arg0: tensor<?x4xf32, #llh.encoding<shapes = @s0, @c4>>) -> (tensor<?x4xf32, #llh.encoding<shapes = @s0, @c4>>) attributes {entrance} {
  %0 = "llh.relu"(%arg0) : (tensor<?x4xf32, #llh.encoding<shapes = @s0, @c4>>) -> tensor<?x4xf32, #llh.encoding<shapes = @s0, @c4>>
  return %0 : tensor<?x4xf32, #llh.encoding<shapes = @s0, @c4>>
}
'''
    out = _capi.run_pass(text, "unload-and-bind-encoding")
    assert out.count('"llh.encoding_bind"') == 2 and out.count("encoding = #llh.encoding<shapes = @s0, @c4>") == 2
    assert "tensor<?x4xf32, #llh.encoding" not in out                       # the types themselves carry none any more


def test_a_pipeline_is_applied_in_order_and_unknown_passes_are_refused():
    out = _capi.run_pass(BN, "decompose-ops,cse")
    assert out.count('"llh.constant"() <{value = 3 : i64}>') == 1          # the repeated extents were merged after the expansion
    try:
        _capi.run_pass(BN, "decompose-ops,no-such-pass")
        assert False
    except _capi.LlcError as e:
        assert "unknown pass" in str(e)
