"""torch FX (aten/prims level) -> LLH dialect text.

Mirrors the reference importer's surface: one ``func.func @main`` whose i64
symbol arguments come first and whose tensor arguments carry
``func.input_symbol_<d>`` attributes (llcompiler/importer/fx_translate.py:
197-224, 490-521), parameters become ``llh.weight`` ops that name ``.npy``
files (:409-436), scalars become ``llh.constant`` (llcompiler/dialect/
llh_utility.py:34-58) and every aten/prims node is translated by a function
registered under the op's schema name (:98-113).

Differences that the current torch forces (probed on torch 2.11): dynamo lifts
every parameter to a graph *placeholder*, so the importer is told which
placeholders are static (``TracingContext.fw_metadata.static_input_indices``)
and emits ``llh.weight`` for those; the values are written with ``np.save``
(not ``tensor.tolist()``, which takes minutes at ResNet-50 size) the first time
the compiled function runs, when the real tensors are at hand.
"""
from __future__ import annotations

import operator
import os
import tempfile
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import sympy
import torch
import torch.fx
from torch.fx.passes.shape_prop import TensorMetadata

from ..dialect.llh import (DYNAMIC, Block, Op, TensorType, Value, array_i64, bool_attr, dense_attr, enum_attr,
                           f64_attr, i64_attr, print_module, str_attr)

INT64_MAX = 9223372036854775807

# llcompiler/importer/fx_translate.py:70-77 has no bf16 entry; bf16 is new here.
TORCH_DTYPE_TO_MLIR_TYPE = {
    torch.int64: "i64", torch.int32: "i32", torch.int8: "i8", torch.float16: "f16",
    torch.bfloat16: "bf16", torch.float32: "f32", torch.float64: "f64", torch.bool: "i1",
}

TORCH_FUNCTION_TRANSLATE: Dict[str, Callable] = {}


def translator(*names: str):
    def deco(fn):
        for n in names:
            TORCH_FUNCTION_TRANSLATE[n] = fn
        return fn
    return deco


def target_name(target) -> str:
    if type(target).__name__ == "builtin_function_or_method" or getattr(target, "__module__", "") == "_operator":
        return target.__name__
    if hasattr(target, "name") and callable(target.name):
        return target.name()
    return getattr(target, "__name__", str(target))


class ImportedFunction:
    """Result of one import: the module text plus what the executor needs to call it."""

    def __init__(self) -> None:
        self.text: str = ""
        self.weight_files: List[Tuple[int, str]] = []   # (placeholder position, npy path)
        self.symbol_positions: List[int] = []           # placeholder positions holding SymInts
        self.tensor_positions: List[int] = []           # run-time tensor inputs, in func-arg order
        self.output_dtypes: List[torch.dtype] = []
        self.output_is_tuple: bool = False
        self.num_placeholders: int = 0


class _Ctx:
    def __init__(self, block: Block):
        self.block = block
        self.values: Dict[str, List[Value]] = {}
        self.symbols: Dict[str, Value] = {}


# ---------------------------------------------------------------- type helpers
def _meta(node: torch.fx.Node, index: Optional[int] = None):
    val = node.meta.get("val", None)
    if val is None:
        val = node.meta.get("tensor_meta", None)
    if val is None:
        raise ValueError(f"no value metadata on {node}")
    if isinstance(val, (tuple, list)):
        return val[index if index is not None else 0]
    return val


def tensor_type_of(t) -> TensorType:
    shape = []
    for d in t.shape:
        if isinstance(d, int):
            shape.append(d)
        elif str(d).lstrip("-").isdigit():
            shape.append(int(str(d)))
        else:
            shape.append(DYNAMIC)
    if not shape:                       # rank-0 tensors are emitted as [1] (fx_translate.py:191-194)
        shape = [1]
    return TensorType(shape, TORCH_DTYPE_TO_MLIR_TYPE[t.dtype])


def _sym_expr(ctx: _Ctx, e) -> Value:
    """SymInt / sympy expression -> i64 SSA value (fx_translate.py:116-158)."""
    b = ctx.block
    if isinstance(e, torch.SymInt):
        return _sym_expr(ctx, e.node.expr)
    if isinstance(e, int):
        return b.constant_i64(e)
    if isinstance(e, sympy.Integer):
        return b.constant_i64(int(e))
    if isinstance(e, sympy.Symbol):
        if e.name not in ctx.symbols:
            ctx.symbols[e.name] = b.op("llh.torch_symbolic_int", [], ["i64"],
                                       {"sym_name": str_attr(e.name)}).result
        return ctx.symbols[e.name]
    if isinstance(e, (sympy.Mul, sympy.Add)):
        name = "llh.mul" if isinstance(e, sympy.Mul) else "llh.add"
        acc = _sym_expr(ctx, e.args[0])
        for a in e.args[1:]:
            acc = b.op(name, [acc, _sym_expr(ctx, a)], ["i64"]).result
        return acc
    if isinstance(e, sympy.Pow) and isinstance(e.args[1], sympy.Integer) and int(e.args[1]) > 0:
        base = _sym_expr(ctx, e.args[0])
        acc = base
        for _ in range(int(e.args[1]) - 1):
            acc = b.op("llh.mul", [acc, base], ["i64"]).result
        return acc
    if type(e).__name__ == "FloorDiv":
        return b.op("llh.div", [_sym_expr(ctx, e.args[0]), _sym_expr(ctx, e.args[1])], ["i64"]).result
    raise NotImplementedError(f"symbol expression {e!r} ({type(e)})")


def _dims_of(ctx: _Ctx, fake) -> List[Value]:
    dims = [_sym_expr(ctx, d) for d in fake.shape]
    return dims or [ctx.block.constant_i64(1)]


def _arg(ctx: _Ctx, a, elt: Optional[str] = None) -> Value:
    """FX argument -> SSA value; python scalars become llh.constant (tensor<1xT> when the
    consumer is a tensor op, fx_translate.py:264-335)."""
    if isinstance(a, torch.fx.Node):
        return ctx.values[a.name][0]
    if isinstance(a, bool) and elt is not None:
        return ctx.block.scalar_tensor(a, elt)
    if isinstance(a, (int, float)):
        if elt is not None:
            return ctx.block.scalar_tensor(a, elt)
        return ctx.block.constant_i64(a) if isinstance(a, int) else ctx.block.constant_f32(a)
    raise NotImplementedError(f"argument {a!r}")


def _index_arg(ctx: _Ctx, a) -> Value:
    if isinstance(a, torch.fx.Node):
        return ctx.values[a.name][0]
    return _sym_expr(ctx, a)


def _pair(v) -> List[int]:
    return [v, v] if isinstance(v, int) else list(v)


def _result_type(node, index=None) -> TensorType:
    return tensor_type_of(_meta(node, index))


# ---------------------------------------------------------------- translators
def _binary(name: str):
    def build(ctx: _Ctx, node: torch.fx.Node):
        out = _meta(node)
        if isinstance(out, (torch.SymInt, torch.SymFloat, int)):
            ops = [_index_arg(ctx, node.args[0]), _index_arg(ctx, node.args[1])]
            return ctx.block.op(name, ops, ["i64"])
        rt = tensor_type_of(out)
        ops = []
        for a in node.args[:2]:
            v = _arg(ctx, a, rt.elt)
            if not isinstance(v.type, TensorType):   # SSA scalar -> tensor<1xT> (fx_translate.py:310-324)
                c = ctx.block.op("llh.scalar_cast", [v], [TensorType([1], v.type)]).result
                v = ctx.block.op("llh.convert_to", [c], [TensorType([1], rt.elt)]).result
            ops.append(v)
        # aten::add / aten::sub carry `alpha`: out = a +- alpha * b.  (The reference's translators drop it,
        # fx_op_translate/binary ops; eager parity needs it.)
        alpha = node.kwargs.get("alpha", 1) if name in ("llh.add", "llh.sub") else 1
        if not isinstance(alpha, (int, float)):
            raise NotImplementedError(f"{node.target}: alpha must be a python number, got {alpha!r}")
        if alpha != 1:
            ops[1] = ctx.block.op("llh.mul", [ops[1], ctx.block.scalar_tensor(alpha, rt.elt)], [TensorType(ops[1].type.shape, rt.elt)]).result
        return ctx.block.op(name, ops, [rt])
    return build


translator("aten::add.Tensor", "aten::add.Scalar", "add", "iadd", "prims::add")(_binary("llh.add"))
translator("aten::sub.Tensor", "aten::sub.Scalar", "sub", "prims::sub")(_binary("llh.sub"))
translator("aten::mul.Tensor", "aten::mul.Scalar", "mul", "prims::mul")(_binary("llh.mul"))
translator("aten::div.Tensor", "aten::div.Scalar", "truediv", "floordiv", "prims::div")(_binary("llh.div"))
translator("aten::maximum", "prims::maximum")(_binary("llh.max"))
translator("aten::minimum", "prims::minimum")(_binary("llh.min"))


@translator("aten::rsub.Scalar", "aten::rsub.Tensor")
def _rsub(ctx, node):
    rt = _result_type(node)
    return ctx.block.op("llh.sub", [_arg(ctx, node.args[1], rt.elt), _arg(ctx, node.args[0], rt.elt)], [rt])


def _unary(name: str, props=None):
    def build(ctx, node):
        return ctx.block.op(name, [_arg(ctx, node.args[0])], [_result_type(node)], props)
    return build


for _aten, _llh in (("relu", "relu"), ("abs", "abs"), ("sqrt", "sqrt"), ("rsqrt", "rsqrt"),
                    ("exp", "exp"), ("tanh", "tanh"), ("erf", "erf"), ("sigmoid", "sigmoid"),
                    ("neg", "neg")):
    translator(f"aten::{_aten}", f"prims::{_aten}")(_unary(f"llh.{_llh}"))


@translator("aten::gelu")
def _gelu(ctx, node):
    approx = node.kwargs.get("approximate", "none")
    return ctx.block.op("llh.gelu", [_arg(ctx, node.args[0])], [_result_type(node)],
                        {"approximate": str_attr(approx)})


@translator("aten::reciprocal")
def _reciprocal(ctx, node):
    rt = _result_type(node)
    return ctx.block.op("llh.div", [ctx.block.scalar_tensor(1.0, rt.elt), _arg(ctx, node.args[0])], [rt])


@translator("aten::mm")
def _mm(ctx, node):
    return ctx.block.op("llh.matmul", [_arg(ctx, node.args[0]), _arg(ctx, node.args[1])],
                        [_result_type(node)])


@translator("aten::bmm")
def _bmm(ctx, node):
    return ctx.block.op("llh.batch_matmul", [_arg(ctx, node.args[0]), _arg(ctx, node.args[1])],
                        [_result_type(node)])


@translator("aten::addmm")
def _addmm(ctx, node):
    rt = _result_type(node)
    mm = ctx.block.op("llh.matmul", [_arg(ctx, node.args[1]), _arg(ctx, node.args[2])], [rt]).result
    # out = beta * input + alpha * (mat1 @ mat2)
    beta, alpha = node.kwargs.get("beta", 1), node.kwargs.get("alpha", 1)
    if not isinstance(beta, (int, float)) or not isinstance(alpha, (int, float)):
        raise NotImplementedError("aten::addmm: beta and alpha must be python numbers")
    bias = _arg(ctx, node.args[0])
    if alpha != 1:
        mm = ctx.block.op("llh.mul", [mm, ctx.block.scalar_tensor(alpha, rt.elt)], [rt]).result
    if beta != 1:
        bias = ctx.block.op("llh.mul", [bias, ctx.block.scalar_tensor(beta, rt.elt)], [TensorType(bias.type.shape, rt.elt)]).result
    return ctx.block.op("llh.add", [mm, bias], [rt])


def _transpose(ctx, x: Value, perms: Sequence[int], rt: Optional[TensorType] = None) -> Op:
    if rt is None:
        rt = TensorType([x.type.shape[p] for p in perms], x.type.elt)
    return ctx.block.op("llh.transpose", [x], [rt], {"perms": array_i64(perms)})


@translator("aten::t")
def _t(ctx, node):
    x = _arg(ctx, node.args[0])
    return _transpose(ctx, x, list(reversed(range(x.type.rank))))


@translator("aten::permute")
def _permute(ctx, node):
    x = _arg(ctx, node.args[0])
    perms = [p % x.type.rank for p in node.args[1]]
    return _transpose(ctx, x, perms, _result_type(node))


@translator("aten::transpose.int")
def _transpose_int(ctx, node):
    x = _arg(ctx, node.args[0])
    r = x.type.rank
    perms = list(range(r))
    a, b = node.args[1] % r, node.args[2] % r
    perms[a], perms[b] = perms[b], perms[a]
    return _transpose(ctx, x, perms, _result_type(node))


@translator("aten::view", "aten::reshape", "aten::_unsafe_view")
def _view(ctx, node):
    x = _arg(ctx, node.args[0])
    dims = [_index_arg(ctx, d) for d in node.args[1]]
    return ctx.block.op("llh.reshape", [x] + dims, [_result_type(node)])


@translator("aten::unsqueeze", "aten::squeeze.dim", "aten::squeeze.dims", "prims::squeeze",
            "aten::flatten.using_ints", "prims::collapse_view")
def _reshape_to_result(ctx, node):
    x = _arg(ctx, node.args[0])
    fake = _meta(node)
    return ctx.block.op("llh.reshape", [x] + _dims_of(ctx, fake), [tensor_type_of(fake)])


@translator("prims::broadcast_in_dim")
def _broadcast_in_dim(ctx, node):
    x = _arg(ctx, node.args[0])
    dims = [_index_arg(ctx, d) for d in node.args[1]]
    return ctx.block.op("llh.broadcast_to", [x] + dims, [_result_type(node)],
                        {"cast_dims": array_i64(node.args[2])})


@translator("aten::expand")
def _expand(ctx, node):
    x = _arg(ctx, node.args[0])
    fake = _meta(node)
    rank_in, rank_out = x.type.rank, len(fake.shape)
    return ctx.block.op("llh.broadcast_to", [x] + _dims_of(ctx, fake), [tensor_type_of(fake)],
                        {"cast_dims": array_i64(range(rank_out - rank_in, rank_out))})


def _filled(ctx, node, value):
    """A tensor of the node's shape holding one value: a one-element constant broadcast to the shape, which the lowering
    keeps as a constant of the expression it is used in (llcompiler/importer/fx_op_translate/alloc_ops.py:83-100)."""
    fake = _meta(node)
    rt = tensor_type_of(fake)
    const_op = ctx.block.op("llh.constant", [], [TensorType([1], rt.elt)], {"value": dense_attr(value, TensorType([1], rt.elt))})
    if len(fake.shape) == 0:
        return const_op
    const = const_op.result
    x = ctx.block.op("llh.reshape", [const] + [ctx.block.constant_i64(1)] * len(fake.shape), [TensorType([1] * len(fake.shape), rt.elt)]).result
    return ctx.block.op("llh.broadcast_to", [x] + _dims_of(ctx, fake), [rt], {"cast_dims": array_i64(range(len(fake.shape)))})


@translator("aten::full")
def _full(ctx, node):
    return _filled(ctx, node, node.args[1])


@translator("aten::zeros", "aten::zeros_like", "aten::new_zeros")
def _zeros(ctx, node):
    return _filled(ctx, node, 0)


@translator("aten::ones", "aten::ones_like", "aten::new_ones")
def _ones(ctx, node):
    return _filled(ctx, node, 1)


@translator("aten::full_like")
def _full_like(ctx, node):
    return _filled(ctx, node, node.args[1])


@translator("aten::scalar_tensor")
def _scalar_tensor(ctx, node):
    # llcompiler/importer/fx_op_translate/alloc_ops.py:72-80
    t = TensorType([1], tensor_type_of(_meta(node)).elt)
    return ctx.block.op("llh.constant", [], [t], {"value": dense_attr(node.args[0], t)})


@translator("aten::empty.memory_format", "aten::empty", "aten::empty_like", "aten::new_empty")
def _empty(ctx, node):
    # uninitialised storage of the node's extents (llcompiler/importer/fx_op_translate/alloc_ops.py:46-69)
    fake = _meta(node)
    return ctx.block.op("llh.empty", _dims_of(ctx, fake), [tensor_type_of(fake)])


@translator("aten::cat")
def _cat(ctx, node):
    # llh.cat with the dim as an attribute (llcompiler/importer/fx_op_translate/cat.py:39-57)
    dim = node.kwargs["dim"] if "dim" in node.kwargs else (node.args[1] if len(node.args) > 1 else 0)
    fake = _meta(node)
    if dim < 0:
        dim += len(fake.shape)
    return ctx.block.op("llh.cat", [_arg(ctx, a) for a in node.args[0]], [tensor_type_of(fake)], {"dim": i64_attr(dim)})


@translator("aten::convolution")
def _convolution(ctx, node):
    x, w = _arg(ctx, node.args[0]), _arg(ctx, node.args[1])
    stride, padding, dilation = _pair(node.args[3]), _pair(node.args[4]), _pair(node.args[5])
    if node.args[6]:
        raise NotImplementedError("transposed convolution")
    props = {   # attribute names and pad order as llcompiler/importer/fx_op_translate/conv.py:48-57
        "dilation": array_i64(dilation),
        "pad": array_i64([padding[0], padding[1], padding[0], padding[1]]),
        "group": i64_attr(node.args[8]),
        "kernel_shape": array_i64(w.type.shape[-2:]),
        "stride": array_i64(stride),
    }
    if node.args[2] is not None:
        return ctx.block.op("llh.conv_bias", [x, w, _arg(ctx, node.args[2])], [_result_type(node)], props)
    return ctx.block.op("llh.conv", [x, w], [_result_type(node)], props)


@translator("aten::_native_batch_norm_legit_no_training")
def _bn_inference(ctx, node):
    ops = [_arg(ctx, node.args[i]) for i in range(5)]
    props = {"epsilon": f64_attr(node.args[6]), "momentum": f64_attr(node.args[5]),
             "feature_index": i64_attr(1), "mode": enum_attr("Mode", "inference")}
    return ctx.block.op("llh.batch_norm_inference", ops, [_result_type(node, 0)], props)


@translator("aten::max_pool2d_with_indices", "aten::max_pool2d")
def _max_pool(ctx, node):
    n = len(node.args)
    kernel = _pair(node.args[1])
    stride = _pair(node.args[2]) if n > 2 and node.args[2] else kernel
    padding = _pair(node.args[3]) if n > 3 else [0, 0]
    dilation = _pair(node.args[4]) if n > 4 else [1, 1]
    ceil_mode = node.args[5] if n > 5 else False
    props = {"dilation": array_i64(dilation),
             "pad": array_i64([padding[0], padding[1], padding[0], padding[1]]),
             "kernel_shape": array_i64(kernel), "stride": array_i64(stride),
             "ceil_mode": bool_attr(ceil_mode)}
    return ctx.block.op("llh.max_pool", [_arg(ctx, node.args[0])], [_result_type(node, 0)], props)


@translator("aten::adaptive_avg_pool2d", "aten::_adaptive_avg_pool2d")
def _adaptive_avg_pool(ctx, node):
    return ctx.block.op("llh.adaptive_average_pool", [_arg(ctx, node.args[0])], [_result_type(node)],
                        {"out_size": array_i64(_pair(node.args[1]))})


def _reduce(name: str):
    def build(ctx, node):
        x = _arg(ctx, node.args[0])
        rank = x.type.rank
        axis = node.args[1] if len(node.args) > 1 and node.args[1] is not None else list(range(rank))
        axis = sorted(a % rank for a in (axis if isinstance(axis, (list, tuple)) else [axis]))
        keepdim = node.args[2] if len(node.args) > 2 else False
        fake = _meta(node)
        rt = tensor_type_of(fake)
        if name == "llh.reduce_mean" and rank == 4 and axis == [2, 3]:
            # the global average pool of the ResNets: the op the dialect declares for it
            kept = TensorType(x.type.shape[:2] + [1, 1], x.type.elt)
            pool = ctx.block.op("llh.adaptive_average_pool", [x], [kept], {"out_size": array_i64([1, 1])})
            if keepdim:
                return pool
            return ctx.block.op("llh.reshape", [pool.result] + _dims_of(ctx, fake), [rt])
        props = {"axis": array_i64(axis)}
        if not keepdim:
            return ctx.block.op(name, [x], [rt], props)
        # keepdim is expressed as reduce + reshape (fx_op_translate/reduce_ops.py:68-82)
        red_shape = [d for i, d in enumerate(x.type.shape) if i not in axis]
        red = ctx.block.op(name, [x], [TensorType(red_shape or [1], x.type.elt)], props).result
        return ctx.block.op("llh.reshape", [red] + _dims_of(ctx, fake), [rt])
    return build


translator("aten::amax")(_reduce("llh.reduce_max"))
translator("aten::amin")(_reduce("llh.reduce_min"))
translator("aten::sum.dim_IntList", "prims::sum")(_reduce("llh.reduce_sum"))
translator("aten::mean.dim")(_reduce("llh.reduce_mean"))


@translator("aten::_softmax", "aten::softmax.int")
def _softmax(ctx, node):
    x = _arg(ctx, node.args[0])
    # aten::_softmax(x, dim, half_to_float) / aten::softmax.int(x, dim, dtype): a result type other than the input's
    # would need a cast in front, which this translator does not insert
    extra = node.args[2] if len(node.args) > 2 else node.kwargs.get("dtype", node.kwargs.get("half_to_float"))
    if extra not in (None, False) and _result_type(node).elt != x.type.elt:
        raise NotImplementedError(f"{node.target}: softmax with a result type different from its input's")
    return ctx.block.op("llh.softmax", [x], [_result_type(node)],
                        {"axis": i64_attr(node.args[1] % x.type.rank)})


@translator("aten::native_layer_norm")
def _layer_norm(ctx, node):
    x = _arg(ctx, node.args[0])
    axis = x.type.rank - len(node.args[1])
    ops = [x, _arg(ctx, node.args[2]), _arg(ctx, node.args[3])]
    return ctx.block.op("llh.layer_norm", ops, [_result_type(node, 0)],
                        {"epsilon": f64_attr(node.args[4]), "axis": i64_attr(axis)})


@translator("aten::embedding")
def _embedding(ctx, node):
    return ctx.block.op("llh.embedding", [_arg(ctx, node.args[0]), _arg(ctx, node.args[1])],
                        [_result_type(node)])


@translator("aten::slice.Tensor")
def _slice(ctx, node):
    x = _arg(ctx, node.args[0])
    rank = x.type.rank
    dim = (node.args[1] if len(node.args) > 1 else 0) % rank
    start = node.args[2] if len(node.args) > 2 and node.args[2] is not None else 0
    end = node.args[3] if len(node.args) > 3 and node.args[3] is not None else INT64_MAX
    step = node.args[4] if len(node.args) > 4 else 1
    extent = x.type.shape[dim]
    if extent != DYNAMIC:                # a static extent: python's own normalisation (negative = from the end, clamped)
        if isinstance(start, int):
            start = min(max(start + extent if start < 0 else start, 0), extent)
        if isinstance(end, int) and end < INT64_MAX:
            end = min(max(end + extent if end < 0 else end, 0), extent)
    elif (isinstance(start, int) and start < 0) or (isinstance(end, int) and end < 0):
        raise NotImplementedError("aten::slice.Tensor: negative bounds on a symbolic extent")
    b = ctx.block
    starts, ends, steps = [], [], []
    for i in range(rank):
        if i == dim:
            starts.append(_index_arg(ctx, start))
            ends.append(b.dim(x, i) if isinstance(end, int) and end >= INT64_MAX else _index_arg(ctx, end))
            steps.append(_index_arg(ctx, step))
        else:
            starts.append(b.constant_i64(0))
            ends.append(b.dim(x, i))
            steps.append(b.constant_i64(1))
    return b.op("llh.stride_slice", [x] + starts + ends + steps, [_result_type(node)],
                {"operandSegmentSizes": f"array<i32: 1, {rank}, {rank}, {rank}>"})


@translator("aten::select.int")
def _select(ctx, node):
    x = _arg(ctx, node.args[0])
    dim = node.args[1] % x.type.rank
    if dim != 0:
        raise NotImplementedError("select on a non-leading dim")
    return ctx.block.op("llh.extract", [x, _index_arg(ctx, node.args[2])], [_result_type(node)])


@translator("aten::_to_copy", "prims::convert_element_type", "aten::to.dtype")
def _convert(ctx, node):
    return ctx.block.op("llh.convert_to", [_arg(ctx, node.args[0])], [_result_type(node)])


def _compare(kind: str):
    def build(ctx, node):
        x = _arg(ctx, node.args[0])
        y = _arg(ctx, node.args[1], x.type.elt)
        return ctx.block.op("llh.compare", [x, y], [_result_type(node)], {"kind": enum_attr("Compare", kind)})
    return build


for _k in ("eq", "ne", "ge", "gt", "le", "lt"):
    translator(f"prims::{_k}", f"aten::{_k}.Scalar", f"aten::{_k}.Tensor")(_compare(_k.upper()))


@translator("aten::where.self", "prims::where")
def _where(ctx, node):
    rt = _result_type(node)
    return ctx.block.op("llh.where", [_arg(ctx, node.args[0]), _arg(ctx, node.args[1], rt.elt),
                                      _arg(ctx, node.args[2], rt.elt)], [rt])


@translator("aten::sym_size.int")
def _sym_size(ctx, node):
    return ctx.block.op("llh.dim", [_arg(ctx, node.args[0]), ctx.block.constant_i64(node.args[1])], ["i64"])


@translator("aten::clone", "aten::alias", "aten::detach", "prims::clone", "aten::lift_fresh_copy",
            "aten::contiguous", "aten::dropout", "aten::native_dropout")
def _identity(ctx, node):
    ctx.values[node.name] = ctx.values[node.args[0].name]
    return None


@translator("getitem")
def _getitem(ctx, node):
    ctx.values[node.name] = [ctx.values[node.args[0].name][node.args[1]]]
    return None


# ---------------------------------------------------------------- function build
def is_supported(node: torch.fx.Node) -> bool:
    return node.op != "call_function" or target_name(node.target) in TORCH_FUNCTION_TRANSLATE


def _input_symbol_attrs(fake) -> Dict[str, str]:
    shape = list(fake.shape) or [1]
    attrs = {}
    for i, d in enumerate(shape):
        s = str(d)
        attrs[f"func.input_symbol_{i}"] = str_attr(("c" + s) if s.lstrip("-").isdigit() else s)
    return attrs


def save_weight(path: str, t: torch.Tensor) -> None:
    """Write one parameter as .npy (format v1, little endian — what the reference's
    load-weight pass parses, src/Dialect/LLH/Transforms/LoadWeight.cpp:58-103).  bf16 has no
    numpy dtype: it is stored as its 16-bit pattern (``<u2``) and the ``llh.weight`` result
    type says bf16."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        arr = t.view(torch.int16).numpy().view(np.uint16)
    else:
        arr = t.numpy()
    if arr.ndim == 0:
        arr = arr.reshape(1)
    np.save(path, arr)


def torch_translate_to_mlir_text(gm: torch.fx.GraphModule, static_positions: Sequence[int] = (),
                                 weight_dir: Optional[str] = None) -> ImportedFunction:
    graph = gm.graph
    block = Block()
    ctx = _Ctx(block)
    res = ImportedFunction()
    placeholders = [n for n in graph.nodes if n.op == "placeholder"]
    res.num_placeholders = len(placeholders)
    static = set(static_positions)
    if weight_dir is None:
        weight_dir = tempfile.mkdtemp(prefix="LLcompiler_weight_")
    os.makedirs(weight_dir, exist_ok=True)

    # 1. symbol arguments first (fx_translate.py:501-503)
    for pos, node in enumerate(placeholders):
        val = node.meta.get("val")
        if isinstance(val, torch.SymInt):
            name = str(val)
            v = block.add_arg("i64", {"func.symbol_int": str_attr(("c" + name) if name.isdigit() else name)})
            ctx.values[node.name] = [v]
            ctx.symbols[name] = v
            res.symbol_positions.append(pos)
    # 2. run-time tensor arguments
    for pos, node in enumerate(placeholders):
        val = node.meta.get("val")
        if isinstance(val, torch.Tensor) and pos not in static:
            v = block.add_arg(tensor_type_of(val), _input_symbol_attrs(val))
            ctx.values[node.name] = [v]
            res.tensor_positions.append(pos)
    # 3. parameters -> llh.weight
    for pos, node in enumerate(placeholders):
        val = node.meta.get("val")
        if isinstance(val, torch.Tensor) and pos in static:
            path = os.path.join(weight_dir, f"{node.name}.npy")
            op = block.op("llh.weight", [], [tensor_type_of(val)], {"weight_file": str_attr(path)})
            ctx.values[node.name] = op.results
            res.weight_files.append((pos, path))
    # module-held parameters (older torch / frozen graphs): same llh.weight route (:409-436)
    attr_tensors = {**dict(gm.named_parameters(remove_duplicate=False)),
                    **dict(gm.named_buffers(remove_duplicate=False))}
    for node in graph.nodes:
        if node.op == "get_attr":
            t = attr_tensors.get(node.target)
            if t is None:
                t = getattr(gm, node.target)
            path = os.path.join(weight_dir, f"{node.name}.npy")
            save_weight(path, t)
            op = block.op("llh.weight", [], [tensor_type_of(t)], {"weight_file": str_attr(path)})
            ctx.values[node.name] = op.results
    # 4. call_function nodes in FX order
    for node in graph.nodes:
        if node.op != "call_function":
            continue
        name = target_name(node.target)
        if name not in TORCH_FUNCTION_TRANSLATE:
            raise NotImplementedError(f"no LLH translation for {name}")
        op = TORCH_FUNCTION_TRANSLATE[name](ctx, node)
        if op is not None:
            ctx.values[node.name] = op.results
    # 5. results
    returns: List[Value] = []
    for node in graph.nodes:
        if node.op != "output":
            continue
        outs = node.args[0]
        res.output_is_tuple = isinstance(outs, (list, tuple))
        for a in (outs if res.output_is_tuple else [outs]):
            if a is None:
                continue
            if not isinstance(a, torch.fx.Node):
                raise NotImplementedError(f"output {a!r}")
            returns.append(ctx.values[a.name][0])
            res.output_dtypes.append(_meta(a).dtype)
    res.text = print_module(block, returns)
    return res
