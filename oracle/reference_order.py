"""CPU oracle, part 3: the reference's own operation order, restated with PyTorch CPU ops.

TEST INFRASTRUCTURE ONLY. Nothing on the product path may import this package.

The plain oracle (oracle/models.py) is PyTorch CPU eager, which is what the reference compares
itself with.  Eager fuses a few operations the reference computes step by step; this module
restates those steps in the reference's order so that the two can be compared, and so that the
places where the reference's arithmetic differs from eager are written down and tested:

  batch-norm inference   ((x - mean) * scale) / sqrt(var + eps) + bias, with eps first cast to the
                         tensor's float type; per-channel operands reshaped and broadcast to the
                         input (src/Dialect/LLH/Transforms/DecomposeOps.cpp:65-74, 125-144)
  softmax                amax -> sub -> exp -> sum -> div, the decomposition of aten._softmax that
                         the reference asks torch for (llcompiler/compiler/torch_compile_config.py:24)
  relu                   max(x, 0) (src/Conversion/LLHToHLO/LLHPreprocessingForHLO.cpp:76-101)
  max-pool               a reduce-window whose initial value is 0, not -inf
                         (src/Conversion/LLHToHLO/LLHToHLO.cpp:313-314): a window whose elements are
                         all negative yields 0.  After a ReLU the two agree exactly, and that is the
                         only place the benchmark models use a max-pool (checked by
                         `max_pools_follow_relu`).

`ReferenceOrder` is a TorchFunctionMode: any eager model run under it computes these four
operations in the reference's order.  Parity status: the restatement follows the cited lines; the
reference itself cannot be run here, so it is pinned only through its agreement with eager (1e-5,
the reference's own tolerance) in tests/test_reference_order_cpu.py.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn.functional as F
from torch.overrides import TorchFunctionMode


def batch_norm_inference(x: torch.Tensor, mean: torch.Tensor, var: torch.Tensor, scale: torch.Tensor | None,
                         bias: torch.Tensor | None, eps: float, feature_index: int = 1) -> torch.Tensor:
    """DecomposeOps.cpp:125-144: stddev = sqrt(var + eps); ((x - mean) * scale) / stddev + bias."""
    shape = [1] * x.dim()
    shape[feature_index] = x.shape[feature_index]
    eps_t = torch.tensor([eps], dtype=torch.float64).to(x.dtype)          # :65-74, eps in the tensor's float type
    stddev = torch.sqrt(var.to(x.dtype) + eps_t)
    ones = torch.ones_like(mean, dtype=x.dtype)
    b = lambda v: v.to(x.dtype).reshape(shape).expand_as(x)               # reshape + broadcast_to, :76-106
    result = x - b(mean)
    result = result * b(scale if scale is not None else ones)
    result = result / b(stddev)
    return result + b(bias if bias is not None else torch.zeros_like(mean, dtype=x.dtype))


def softmax(x: torch.Tensor, dim: int) -> torch.Tensor:
    """torch's decomposition of aten._softmax, the chain the reference imports: amax, sub, exp, sum, div."""
    m = torch.amax(x, dim=dim, keepdim=True)
    e = torch.exp(x - m)
    return e / torch.sum(e, dim=dim, keepdim=True)


def relu(x: torch.Tensor) -> torch.Tensor:
    return torch.maximum(x, torch.zeros((), dtype=x.dtype))


def max_pool2d_zero_init(x: torch.Tensor, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False) -> torch.Tensor:
    """LLHToHLO.cpp:295-339: reduce_window(max) over the padded input with initial value 0; the padding itself is the
    initial value, so the result is max(0, window maximum)."""
    y = F.max_pool2d(x, kernel_size, stride, padding, dilation, ceil_mode)
    return torch.maximum(y, torch.zeros((), dtype=y.dtype))


class ReferenceOrder(TorchFunctionMode):
    """Runs batch-norm inference, softmax, relu and max-pool in the reference's order (see the module text)."""

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is F.batch_norm:
            def bn(input, running_mean, running_var, weight=None, bias=None, training=False, momentum=0.1, eps=1e-5):
                if training or running_mean is None:
                    return None
                return batch_norm_inference(input, running_mean, running_var, weight, bias, eps)
            with torch._C.DisableTorchFunction():
                out = bn(*args, **kwargs)
            if out is not None:
                return out
        elif func in (F.softmax, torch.softmax, torch.Tensor.softmax):
            def sm(input, dim=None, _stacklevel=3, dtype=None):
                return softmax(input if dtype is None else input.to(dtype), dim)
            with torch._C.DisableTorchFunction():
                return sm(*args, **kwargs)
        elif func in (F.relu, torch.relu, torch.Tensor.relu):
            def rl(input, inplace=False):
                return relu(input)
            with torch._C.DisableTorchFunction():
                return rl(*args, **kwargs)
        elif func in (F.max_pool2d, torch.max_pool2d):
            def mp(input, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False, return_indices=False):
                return max_pool2d_zero_init(input, kernel_size, stride, padding, dilation, ceil_mode)
            with torch._C.DisableTorchFunction():
                return mp(*args, **kwargs)
        return func(*args, **kwargs)


def max_pools_follow_relu(model: torch.nn.Module) -> List[str]:
    """Names of the max-pool nodes of `model` whose input is NOT produced by a ReLU (empty = the reference's zero
    initial value cannot show).  Works on the symbolically traced graph."""
    import torch.fx as fx
    gm = fx.symbolic_trace(model)
    mods = dict(gm.named_modules())

    def is_relu(n):
        if n.op == "call_module":
            return isinstance(mods[n.target], torch.nn.ReLU)
        return n.op in ("call_function", "call_method") and getattr(n.target, "__name__", n.target) in ("relu", "relu_")

    def is_pool(n):
        if n.op == "call_module":
            return isinstance(mods[n.target], torch.nn.MaxPool2d)
        return n.op == "call_function" and getattr(n.target, "__name__", "") in ("max_pool2d", "_max_pool2d", "boolean_dispatch")

    bad = []
    for n in gm.graph.nodes:
        if is_pool(n) and not is_relu(n.args[0]):
            bad.append(n.name)
    return bad
