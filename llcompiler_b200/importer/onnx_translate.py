"""ONNX graph -> LLH module text.

The reference names ONNX as an entry (llcompiler/importer/importer.py:52-54) but only maps element types and dumps
initialisers (llcompiler/importer/onnx_translate.py:32-92).  This translator covers the operators of the MLP and ResNet
configurations with static shapes: Gemm, MatMul, Add, Sub, Mul, Div, Relu, Conv, BatchNormalization, MaxPool,
GlobalAveragePool, Flatten, Reshape, Identity.  Initialisers become `llh.weight` ops backed by .npy files, exactly like
the parameters of the FX route; the result is the same ImportedFunction the FX importer returns.
"""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Optional

import numpy as np
import torch

from ..dialect.llh import Block, TensorType, Value, array_i64, bool_attr, enum_attr, f64_attr, i64_attr, print_module, str_attr
from .fx_translate import ImportedFunction
from .onnx_wire import FLOAT, INT64, OnnxGraph, OnnxNode, parse_model

_ELT = {FLOAT: "f32", INT64: "i64"}
_TORCH = {"f32": torch.float32, "i64": torch.int64}


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
        if x != y and 1 not in (x, y):
            raise ValueError(f"shapes {a} and {b} do not broadcast")
        out.append(max(x, y))
    return out[::-1]


def _window(n: int, k: int, s: int, pl: int, ph: int, d: int = 1, ceil: bool = False) -> int:
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
    elif op == "MatMul":
        y = ctx.get(n.inputs[1])
        if x.type.rank != 2 or y.type.rank != 2:
            raise NotImplementedError("MatMul of rank other than 2")
        emit("llh.matmul", [x, y], [x.type.shape[0], y.type.shape[1]])
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
    elif op == "GlobalAveragePool":
        emit("llh.adaptive_average_pool", [x], x.type.shape[:2] + [1, 1], {"out_size": array_i64([1, 1])})
    elif op in ("Flatten", "Reshape"):
        if op == "Flatten":
            axis = int(a.get("axis", 1))
            shape = [int(np.prod(x.type.shape[:axis], dtype=np.int64)), int(np.prod(x.type.shape[axis:], dtype=np.int64))]
        else:
            shape = ctx.const_ints(n.inputs[1])
            total = int(np.prod(x.type.shape, dtype=np.int64))
            shape = [x.type.shape[i] if d == 0 else d for i, d in enumerate(shape)]
            if -1 in shape:
                shape[shape.index(-1)] = total // int(-np.prod(shape, dtype=np.int64))
        emit("llh.reshape", [x] + [b.constant_i64(d) for d in shape], shape)
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
        if any(not isinstance(d, int) or d <= 0 for d in v.dims):
            raise NotImplementedError(f"ONNX input '{v.name}' has symbolic extents {v.dims}; only static shapes are imported")
        if v.elem_type not in _ELT:
            raise NotImplementedError(f"ONNX input element type {v.elem_type}")
        ctx.values[v.name] = ctx.block.add_arg(TensorType(list(v.dims), _ELT[v.elem_type]), {})
        res.tensor_positions.append(pos)
    res.num_placeholders = len(graph.inputs)
    for n in graph.nodes:
        _translate(ctx, n)
    returns = [ctx.get(o.name) for o in graph.outputs]
    res.text = print_module(ctx.block, returns)
    res.output_dtypes = [_TORCH[r.type.elt] for r in returns]
    res.output_is_tuple = len(returns) != 1
    return res
