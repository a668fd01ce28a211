"""ONNX graph -> LLH module text.

The reference names ONNX as an entry (llcompiler/importer/importer.py:52-54) but only maps element types and dumps
initialisers (llcompiler/importer/onnx_translate.py:32-92).  This translator covers the operators of the MLP and ResNet
configurations and of a transformer encoder: Gemm, MatMul (plain, rows-folded and batched), Add, Sub, Mul, Div, Relu,
Gelu, Sqrt, Exp, Tanh, Erf, Sigmoid, Neg, Abs, Softmax, LayerNormalization, Transpose, Gather (embedding rows), Conv,
BatchNormalization, MaxPool, GlobalAveragePool, Flatten, Reshape, Identity.  An input extent given as a `dim_param` (or left unknown) becomes a symbol: the argument carries
`func.input_symbol_<d>` like the arguments of the FX route (llcompiler/importer/fx_translate.py:60-75), result types
show `?` there and the compiler's shape inference fills in the expressions.  Initialisers become `llh.weight` ops backed by .npy files, exactly like
the parameters of the FX route; the result is the same ImportedFunction the FX importer returns.
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Optional

import numpy as np
import torch

from ..dialect.llh import DYNAMIC, Block, TensorType, Value, array_i64, bool_attr, enum_attr, f64_attr, i64_attr, print_module, str_attr
from .fx_translate import ImportedFunction
from .onnx_wire import FLOAT, INT64, OnnxGraph, OnnxNode, parse_model

_ELT = {FLOAT: "f32", INT64: "i64"}
_TORCH = {"f32": torch.float32, "i64": torch.int64}
_UNARY = {"Sqrt": "sqrt", "Exp": "exp", "Tanh": "tanh", "Erf": "erf", "Sigmoid": "sigmoid", "Neg": "neg", "Abs": "abs"}


class _Ctx:
    def __init__(self, graph: OnnxGraph, weight_dir: str):
        self.g, self.block, self.weight_dir = graph, Block(), weight_dir
        self.values: Dict[str, Value] = {}
        self.weight_files: List[str] = []

    def get(self, name: str) -> Value:
        if name in self.values:
            return self.values[name]
        if name in self.g.initializers:
            arr = self.g.initializers[name]
            elt = "f32" if arr.dtype == np.float32 else "i64"
            path = os.path.join(self.weight_dir, f"onnx_{len(self.weight_files)}.npy")
            np.save(path, arr.reshape(1) if arr.ndim == 0 else np.ascontiguousarray(arr))
            self.weight_files.append(path)
            t = TensorType(list(arr.shape) or [1], elt)
            v = self.block.op("llh.weight", [], [t], {"weight_file": str_attr(path)}).result
            self.values[name] = v
            return v
        raise KeyError(f"ONNX value '{name}' is used before it is produced")

    def const_ints(self, name: str) -> List[int]:
        if name not in self.g.initializers:
            raise NotImplementedError(f"'{name}' must be a constant initialiser")
        return [int(v) for v in self.g.initializers[name].reshape(-1)]


def _bcast(a: List[int], b: List[int]) -> List[int]:
    out = []
    for i in range(max(len(a), len(b))):
        x = a[len(a) - 1 - i] if i < len(a) else 1
        y = b[len(b) - 1 - i] if i < len(b) else 1
        if DYNAMIC in (x, y):           # a symbolic extent meets 1, itself or a static extent it must equal at run time
            out.append(max(x, y) if max(x, y) > 1 else DYNAMIC)
            continue
        if x != y and 1 not in (x, y):
            raise ValueError(f"shapes {a} and {b} do not broadcast")
        out.append(max(x, y))
    return out[::-1]


def _prod(dims) -> int:
    return DYNAMIC if DYNAMIC in dims else int(np.prod(dims, dtype=np.int64))


def _extent_value(block: Block, x: Value, dims: range):
    """i64 value of the product of x's extents over `dims` (llh.dim for the symbolic ones)."""
    static = int(np.prod([x.type.shape[d] for d in dims if x.type.shape[d] != DYNAMIC], dtype=np.int64))
    acc = None
    for d in dims:
        if x.type.shape[d] == DYNAMIC:
            v = block.dim(x, d)
            acc = v if acc is None else block.op("llh.mul", [acc, v], ["i64"]).result
    if acc is None:
        return block.constant_i64(static)
    return acc if static == 1 else block.op("llh.mul", [acc, block.constant_i64(static)], ["i64"]).result


def _window(n: int, k: int, s: int, pl: int, ph: int, d: int = 1, ceil: bool = False) -> int:
    if n == DYNAMIC:
        return DYNAMIC
    num = n + pl + ph - d * (k - 1) - 1
    return (-(-num // s) if ceil else num // s) + 1


def _pads(attrs, rank: int = 2) -> List[int]:
    p = attrs.get("pads") or [0] * (2 * rank)
    if attrs.get("auto_pad", "NOTSET") not in ("NOTSET", ""):
        raise NotImplementedError("auto_pad")
    return [p[0], p[1], p[2], p[3]]          # ONNX: (top, left, bottom, right) = the LLH order


def _translate(ctx: _Ctx, n: OnnxNode) -> None:
    b, a, op = ctx.block, n.attrs, n.op_type
    x = ctx.get(n.inputs[0]) if n.inputs else None

    def emit(name, operands, shape, props=None, elt=None):
        r = b.op(name, operands, [TensorType(shape, elt or operands[0].type.elt)], props).result
        ctx.values[n.outputs[0]] = r
        return r

    if op in ("Relu", "Identity"):
        if op == "Identity":
            ctx.values[n.outputs[0]] = x
        else:
            emit("llh.relu", [x], x.type.shape)
    elif op in ("Add", "Sub", "Mul", "Div"):
        y = ctx.get(n.inputs[1])
        emit("llh." + op.lower(), [x, y], _bcast(x.type.shape, y.type.shape))
    elif op in _UNARY:
        emit("llh." + _UNARY[op], [x], x.type.shape)
    elif op == "Gelu":
        emit("llh.gelu", [x], x.type.shape, {"approximate": str_attr(a.get("approximate", "none") or "none")})
    elif op == "Softmax":
        emit("llh.softmax", [x], x.type.shape, {"axis": i64_attr(int(a.get("axis", -1)) % x.type.rank)})
    elif op == "LayerNormalization":
        if len(n.inputs) < 3 or not n.inputs[2]:
            raise NotImplementedError("LayerNormalization without a bias")
        emit("llh.layer_norm", [x, ctx.get(n.inputs[1]), ctx.get(n.inputs[2])], x.type.shape,
             {"epsilon": f64_attr(float(a.get("epsilon", 1e-5))), "axis": i64_attr(int(a.get("axis", -1)) % x.type.rank)})
    elif op == "Transpose":
        perm = [int(p) for p in (a.get("perm") or range(x.type.rank - 1, -1, -1))]
        emit("llh.transpose", [x], [x.type.shape[p] for p in perm], {"perms": array_i64(perm)})
    elif op == "Gather":
        ids = ctx.get(n.inputs[1])
        if int(a.get("axis", 0)) != 0 or x.type.rank != 2 or ids.type.elt != "i64":
            raise NotImplementedError("Gather other than rows of a table by int64 indices")
        emit("llh.embedding", [x, ids], ids.type.shape + [x.type.shape[1]], elt=x.type.elt)
    elif op == "MatMul":
        y = ctx.get(n.inputs[1])
        rx, ry = x.type.rank, y.type.rank
        if rx == 2 and ry == 2:
            emit("llh.matmul", [x, y], [x.type.shape[0], y.type.shape[1]])
        elif rx > 2 and ry == 2:              # [..., M, K] x [K, N]: the leading extents fold into the rows
            rows = b.op("llh.reshape", [x, _extent_value(b, x, range(rx - 1)), b.constant_i64(x.type.shape[-1])],
                        [TensorType([_prod(x.type.shape[:-1]), x.type.shape[-1]], x.type.elt)]).result
            mm = b.op("llh.matmul", [rows, y], [TensorType([rows.type.shape[0], y.type.shape[1]], x.type.elt)]).result
            shape = x.type.shape[:-1] + [y.type.shape[1]]
            emit("llh.reshape", [mm] + [b.dim(x, d) if shape[d] == DYNAMIC else b.constant_i64(shape[d]) for d in range(rx - 1)]
                 + [b.constant_i64(shape[-1])], shape)
        elif rx == ry and rx >= 3:            # batched on both sides: fold the leading extents into one batch
            def fold(v):
                if v.type.rank == 3:
                    return v
                return b.op("llh.reshape", [v, _extent_value(b, v, range(v.type.rank - 2)), b.constant_i64(v.type.shape[-2]), b.constant_i64(v.type.shape[-1])],
                            [TensorType([_prod(v.type.shape[:-2])] + v.type.shape[-2:], v.type.elt)]).result
            if DYNAMIC in x.type.shape[-2:] or DYNAMIC in y.type.shape[-2:]:
                raise NotImplementedError("batched MatMul with a symbolic matrix extent")
            fx, fy = fold(x), fold(y)
            bm = b.op("llh.batch_matmul", [fx, fy], [TensorType([fx.type.shape[0], fx.type.shape[1], fy.type.shape[2]], x.type.elt)]).result
            shape = x.type.shape[:-1] + [y.type.shape[-1]]
            if rx == 3:
                ctx.values[n.outputs[0]] = bm
            else:
                emit("llh.reshape", [bm] + [b.dim(x, d) if shape[d] == DYNAMIC else b.constant_i64(shape[d]) for d in range(rx)], shape)
        else:
            raise NotImplementedError(f"MatMul of ranks {rx} and {ry}")
    elif op == "Gemm":
        if a.get("transA", 0) or float(a.get("alpha", 1.0)) != 1.0 or float(a.get("beta", 1.0)) != 1.0:
            raise NotImplementedError("Gemm with transA, alpha or beta")
        w = ctx.get(n.inputs[1])
        if a.get("transB", 0):          # weights stored [N, K], as torch.nn.Linear exports them
            w = b.op("llh.transpose", [w], [TensorType(w.type.shape[::-1], w.type.elt)], {"perms": array_i64([1, 0])}).result
        shape = [x.type.shape[0], w.type.shape[1]]
        mm = b.op("llh.matmul", [x, w], [TensorType(shape, x.type.elt)]).result
        if len(n.inputs) > 2 and n.inputs[2]:
            emit("llh.add", [mm, ctx.get(n.inputs[2])], shape)
        else:
            ctx.values[n.outputs[0]] = mm
    elif op == "Conv":
        w = ctx.get(n.inputs[1])
        if x.type.rank != 4:
            raise NotImplementedError("Conv of rank other than 4")
        stride, dil, pads = a.get("strides") or [1, 1], a.get("dilations") or [1, 1], _pads(a)
        kh, kw = w.type.shape[2], w.type.shape[3]
        shape = [x.type.shape[0], w.type.shape[0], _window(x.type.shape[2], kh, stride[0], pads[0], pads[2], dil[0]),
                 _window(x.type.shape[3], kw, stride[1], pads[1], pads[3], dil[1])]
        props = {"dilation": array_i64(dil), "pad": array_i64(pads), "group": i64_attr(int(a.get("group", 1))),
                 "kernel_shape": array_i64([kh, kw]), "stride": array_i64(stride)}
        if len(n.inputs) > 2 and n.inputs[2]:
            emit("llh.conv_bias", [x, w, ctx.get(n.inputs[2])], shape, props)
        else:
            emit("llh.conv", [x, w], shape, props)
    elif op == "BatchNormalization":
        if int(a.get("training_mode", 0)):
            raise NotImplementedError("BatchNormalization in training mode")
        operands = [x] + [ctx.get(i) for i in n.inputs[1:5]]       # scale, bias, mean, var: the LLH operand order
        emit("llh.batch_norm_inference", operands, x.type.shape,
             {"epsilon": f64_attr(float(a.get("epsilon", 1e-5))), "momentum": f64_attr(float(a.get("momentum", 0.9))),
              "feature_index": i64_attr(1), "mode": enum_attr("Mode", "inference")})
    elif op == "MaxPool":
        k, pads = a["kernel_shape"], _pads(a)
        stride, dil, ceil = a.get("strides") or [1, 1], a.get("dilations") or [1, 1], bool(a.get("ceil_mode", 0))
        shape = x.type.shape[:2] + [_window(x.type.shape[2], k[0], stride[0], pads[0], pads[2], dil[0], ceil),
                                    _window(x.type.shape[3], k[1], stride[1], pads[1], pads[3], dil[1], ceil)]
        emit("llh.max_pool", [x], shape, {"dilation": array_i64(dil), "pad": array_i64(pads), "kernel_shape": array_i64(k),
                                          "stride": array_i64(stride), "ceil_mode": bool_attr(ceil)})
    elif op in ("ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin"):
        # axes: an attribute up to opset 12 (17 for the others), a constant input after that
        axes = a.get("axes")
        if axes is None and len(n.inputs) > 1 and n.inputs[1]:
            axes = ctx.const_ints(n.inputs[1])
        axes = sorted(int(v) % x.type.rank for v in (axes if axes is not None else range(x.type.rank)))
        keep = int(a.get("keepdims", 1))
        red_shape = [d for i, d in enumerate(x.type.shape) if i not in axes]
        name = {"ReduceMean": "llh.reduce_mean", "ReduceSum": "llh.reduce_sum", "ReduceMax": "llh.reduce_max", "ReduceMin": "llh.reduce_min"}[op]
        if not keep:
            emit(name, [x], red_shape or [1], {"axis": array_i64(axes)})
        else:                                   # keepdims = reduce + reshape, as the FX importer writes it
            red = b.op(name, [x], [TensorType(red_shape or [1], x.type.elt)], {"axis": array_i64(axes)}).result
            shape = [1 if i in axes else d for i, d in enumerate(x.type.shape)]
            dims = [b.constant_i64(1) if i in axes else (b.dim(x, i) if d == DYNAMIC else b.constant_i64(d)) for i, d in enumerate(x.type.shape)]
            emit("llh.reshape", [red] + dims, shape)
    elif op == "Pow":
        if n.inputs[1] not in ctx.g.initializers or ctx.g.initializers[n.inputs[1]].size != 1:
            raise NotImplementedError("Pow with an exponent that is not a constant scalar")
        e = float(ctx.g.initializers[n.inputs[1]].reshape(-1)[0])
        emit("llh.pow", [x, b.scalar_tensor(e, x.type.elt)], x.type.shape)
    elif op == "Cast":
        to = {FLOAT: "f32", INT64: "i64", 16: "bf16", 10: "f16", 6: "i32", 9: "i1"}.get(int(a.get("to", FLOAT)))
        if to is None:
            raise NotImplementedError(f"Cast to ONNX element type {a.get('to')}")
        emit("llh.convert_to", [x], x.type.shape, elt=to)
    elif op == "Where":
        y, z = ctx.get(n.inputs[1]), ctx.get(n.inputs[2])
        shape = _bcast(_bcast(x.type.shape, y.type.shape), z.type.shape)
        ctx.values[n.outputs[0]] = b.op("llh.where", [x, y, z], [TensorType(shape, y.type.elt)]).result
    elif op in ("Unsqueeze", "Squeeze"):
        axes = a.get("axes")
        if axes is None and len(n.inputs) > 1 and n.inputs[1]:
            axes = ctx.const_ints(n.inputs[1])
        if op == "Unsqueeze":
            rank = x.type.rank + len(axes)
            axes = sorted(int(v) % rank for v in axes)
            src = iter(range(x.type.rank))
            pairs = [(1, None) if i in axes else (lambda j: (x.type.shape[j], j))(next(src)) for i in range(rank)]
        else:
            axes = sorted(int(v) % x.type.rank for v in axes) if axes is not None else [i for i, d in enumerate(x.type.shape) if d == 1]
            pairs = [(d, i) for i, d in enumerate(x.type.shape) if i not in axes]
        shape = [d for d, _ in pairs] or [1]
        dims = [b.constant_i64(1) if j is None else (b.dim(x, j) if d == DYNAMIC else b.constant_i64(d)) for d, j in pairs] or [b.constant_i64(1)]
        emit("llh.reshape", [x] + dims, shape)
    elif op == "Slice":
        starts, ends = ctx.const_ints(n.inputs[1]), ctx.const_ints(n.inputs[2])
        axes = ctx.const_ints(n.inputs[3]) if len(n.inputs) > 3 and n.inputs[3] else list(range(len(starts)))
        steps = ctx.const_ints(n.inputs[4]) if len(n.inputs) > 4 and n.inputs[4] else [1] * len(starts)
        rank = x.type.rank
        lo, hi, st = [0] * rank, list(x.type.shape), [1] * rank
        for s0, e0, ax, sp in zip(starts, ends, axes, steps):
            ax %= rank
            ext = x.type.shape[ax]
            if ext == DYNAMIC or sp < 1:
                raise NotImplementedError("Slice along a symbolic extent or with a negative step")
            s0 = max(0, min(ext, s0 + ext if s0 < 0 else s0))
            e0 = max(0, min(ext, e0 + ext if e0 < 0 else e0))
            lo[ax], hi[ax], st[ax] = s0, max(s0, e0), sp
        shape = [x.type.shape[i] if x.type.shape[i] == DYNAMIC else -(-(hi[i] - lo[i]) // st[i]) for i in range(rank)]
        ends_v = [b.dim(x, i) if x.type.shape[i] == DYNAMIC else b.constant_i64(hi[i]) for i in range(rank)]
        emit("llh.stride_slice", [x] + [b.constant_i64(v) for v in lo] + ends_v + [b.constant_i64(v) for v in st], shape,
             {"operandSegmentSizes": "array<i32: 1, %d, %d, %d>" % (rank, rank, rank)})
    elif op == "Concat":
        xs = [ctx.get(i) for i in n.inputs]
        axis = int(a.get("axis", 0)) % x.type.rank
        along = [v.type.shape[axis] for v in xs]
        shape = list(x.type.shape)
        shape[axis] = DYNAMIC if DYNAMIC in along else sum(along)
        emit("llh.cat", xs, shape, {"dim": i64_attr(axis)})
    elif op == "GlobalAveragePool":
        emit("llh.adaptive_average_pool", [x], x.type.shape[:2] + [1, 1], {"out_size": array_i64([1, 1])})
    elif op in ("Flatten", "Reshape"):
        rank = x.type.rank
        if op == "Flatten":
            axis = int(a.get("axis", 1)) % (rank + 1)
            shape = [_prod(x.type.shape[:axis]), _prod(x.type.shape[axis:])]
            dims = [_extent_value(b, x, range(0, axis)), _extent_value(b, x, range(axis, rank))]
        else:
            want = ctx.const_ints(n.inputs[1])
            shape = [x.type.shape[i] if d == 0 else (DYNAMIC if d == -1 else d) for i, d in enumerate(want)]
            dims = [b.dim(x, i) if d == 0 and x.type.shape[i] == DYNAMIC else (None if d == -1 else b.constant_i64(shape[i]))
                    for i, d in enumerate(want)]
            if -1 in want:
                at, known = want.index(-1), [s for i, s in enumerate(shape) if want[i] != -1]
                if DYNAMIC not in x.type.shape and DYNAMIC not in known:
                    shape[at] = _prod(x.type.shape) // max(1, _prod(known))
                    dims[at] = b.constant_i64(shape[at])
                else:                       # total extent / product of the named extents, as i64 arithmetic
                    num = _extent_value(b, x, range(rank))
                    den = None
                    for i, v in enumerate(dims):
                        if i != at:
                            den = v if den is None else b.op("llh.mul", [den, v], ["i64"]).result
                    dims[at] = num if den is None else b.op("llh.div", [num, den], ["i64"]).result
        emit("llh.reshape", [x] + dims, shape)
    else:
        raise NotImplementedError(f"no LLH translation for ONNX operator {op}")


def onnx_translate_to_mlir_text(model, weight_dir: Optional[str] = None) -> ImportedFunction:
    """`model` is the bytes of a .onnx file, a path to one, or an onnx.ModelProto (serialised here)."""
    if hasattr(model, "SerializeToString"):
        model = model.SerializeToString()
    elif isinstance(model, (str, os.PathLike)):
        model = open(model, "rb").read()
    graph = parse_model(bytes(model))
    ctx = _Ctx(graph, weight_dir or tempfile.mkdtemp(prefix="LLcompiler_weight_"))
    os.makedirs(ctx.weight_dir, exist_ok=True)
    res = ImportedFunction()
    for pos, v in enumerate(graph.inputs):
        if v.elem_type not in _ELT:
            raise NotImplementedError(f"ONNX input element type {v.elem_type}")
        shape, attrs = [], {}
        for d, ext in enumerate(v.dims or [1]):
            if isinstance(ext, int) and ext > 0:
                shape.append(ext)
                attrs[f"func.input_symbol_{d}"] = str_attr(f"c{ext}")
            else:                           # dim_param, or an extent the exporter left open: one symbol per distinct name
                name = ext if isinstance(ext, str) and ext not in ("", "?") else f"{v.name}_{d}"
                name = "".join(ch if ch.isalnum() else "_" for ch in name)
                shape.append(DYNAMIC)
                attrs[f"func.input_symbol_{d}"] = str_attr(("s_" + name) if name[0].isdigit() or name[0] == "c" else name)
        ctx.values[v.name] = ctx.block.add_arg(TensorType(shape, _ELT[v.elem_type]), attrs)
        res.tensor_positions.append(pos)
    res.num_placeholders = len(graph.inputs)
    for n in graph.nodes:
        _translate(ctx, n)
    returns = [ctx.get(o.name) for o in graph.outputs]
    res.text = print_module(ctx.block, returns)
    res.output_dtypes = [_TORCH[r.type.elt] for r in returns]
    res.output_is_tuple = len(returns) != 1
    return res
