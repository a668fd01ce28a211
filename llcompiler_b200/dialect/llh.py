"""A dependency-free builder and printer for the LLH dialect's textual form.

The reference builds LLH ops with xDSL IRDL classes
(llcompiler/dialect/llh.py:445-490 lists the 40 ops it registers) and hands
``str(module)`` to the C++ compiler (llcompiler/compiler/compiler.py:132-135).
Only that text crosses the boundary, so this module keeps the same op names,
operand order and attribute names and prints MLIR generic form directly; no
xDSL is involved.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Union

DYNAMIC = -1

# op names of the LLH surface (include/llcompiler/Dialect/LLH/IR/LLHOps.td:64-553),
# plus the ones the five benchmark graphs need that the reference only declares
# or lacks: layer_norm (LLHOps.td:454-463), adaptive_average_pool (:337-339),
# softmax (llcompiler/dialect/llh.py:406-411), gelu, embedding, stride_slice.
LLH_OPS = {
    "torch_symbolic_int", "symbolic_bind", "constant", "weight", "dim", "shape_of",
    "scalar_cast", "convert_to", "empty", "reshape", "broadcast_to", "transpose",
    "extract", "stride_slice", "slice", "cat", "expand", "flatten",
    "add", "sub", "mul", "div", "max", "min", "pow",
    "relu", "abs", "sqrt", "rsqrt", "exp", "gelu", "tanh", "erf", "sigmoid", "neg",
    "drop", "compare", "where",
    "conv", "conv_bias", "matmul", "batch_matmul", "layer_norm", "batch_norm",
    "batch_norm_inference", "max_pool", "adaptive_average_pool",
    "reduce_max", "reduce_min", "reduce_sum", "reduce_mean", "softmax", "embedding",
    "print", "aot",
}


class TensorType:
    def __init__(self, shape: Sequence[int], elt: str):
        self.shape = [int(d) for d in shape]
        self.elt = elt

    @property
    def rank(self) -> int:
        return len(self.shape)

    def __str__(self) -> str:
        dims = "".join(("?" if d == DYNAMIC else str(d)) + "x" for d in self.shape)
        return f"tensor<{dims}{self.elt}>"

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorType) and str(self) == str(other)


Type = Union[TensorType, str]


class Value:
    __slots__ = ("name", "type")

    def __init__(self, name: str, type: Type):
        self.name = name
        self.type = type


# ---- attribute spellings ---------------------------------------------------
def i64_attr(v: int) -> str:
    return f"{int(v)} : i64"


def f64_attr(v: float) -> str:
    return f"{_float_text(v)} : f64"


def f32_attr(v: float) -> str:
    return f"{_float_text(v)} : f32"


def bool_attr(v) -> str:
    return "true" if v else "false"


def str_attr(s: str) -> str:
    return '"' + s.replace("\\", "\\\\").replace('"', '\\"') + '"'


def array_i64(vals: Iterable[int]) -> str:
    vals = [int(v) for v in vals]
    return "array<i64: " + ", ".join(str(v) for v in vals) + ">" if vals else "array<i64>"


def enum_attr(kind: str, value: str) -> str:
    return f"#llh.{kind}<{value}>"


def _float_text(v: float) -> str:
    v = float(v)
    if v != v:
        return "0x7FC00000"
    if v in (float("inf"), float("-inf")):
        return "0x7F800000" if v > 0 else "0xFF800000"
    return format(v, ".6e") if v == float(format(v, ".6e")) else repr(v)


def dense_attr(val, type: TensorType) -> str:
    body = str(int(val)) if type.elt[0] == "i" else _float_text(val)
    if type.elt == "i1":
        body = "true" if val else "false"
    return f"dense<{body}> : {type}"


class Op:
    def __init__(self, name: str, operands: Sequence[Value] = (), result_types: Sequence[Type] = (),
                 props: Optional[Dict[str, str]] = None):
        assert name.startswith("llh.") and name[4:] in LLH_OPS, name
        self.name = name
        self.operands = list(operands)
        self.props = dict(props or {})
        self.result_types = list(result_types)
        self.results: List[Value] = []

    @property
    def result(self) -> Value:
        return self.results[0]


class Block:
    """One function body; values are numbered in creation order like xDSL's printer."""

    def __init__(self) -> None:
        self.ops: List[Op] = []
        self.args: List[Value] = []
        self.arg_attrs: List[Dict[str, str]] = []
        self._n = 0

    def _fresh(self, type: Type) -> Value:
        v = Value(f"%{self._n}", type)
        self._n += 1
        return v

    def add_arg(self, type: Type, attrs: Dict[str, str]) -> Value:
        v = self._fresh(type)
        self.args.append(v)
        self.arg_attrs.append(attrs)
        return v

    def add(self, op: Op) -> Op:
        op.results = [self._fresh(t) for t in op.result_types]
        self.ops.append(op)
        return op

    def op(self, name: str, operands=(), result_types=(), props=None) -> Op:
        return self.add(Op(name, operands, result_types, props))

    # helpers shared by translators (llcompiler/dialect/llh_utility.py:34-86)
    def constant_i64(self, v: int) -> Value:
        return self.op("llh.constant", [], ["i64"], {"value": i64_attr(v)}).result

    def constant_f32(self, v: float) -> Value:
        return self.op("llh.constant", [], ["f32"], {"value": f32_attr(v)}).result

    def scalar_tensor(self, v, elt: str) -> Value:
        t = TensorType([1], elt)
        return self.op("llh.constant", [], [t], {"value": dense_attr(v, t)}).result

    def dim(self, x: Value, i: int) -> Value:
        return self.op("llh.dim", [x, self.constant_i64(i)], ["i64"]).result


def print_module(block: Block, returns: Sequence[Value], func_name: str = "main") -> str:
    """Text of one ``builtin.module`` holding ``func.func @main ... attributes {entrance}``
    (llcompiler/importer/fx_translate.py:517-521)."""
    out: List[str] = ["builtin.module {"]
    args = []
    for v, attrs in zip(block.args, block.arg_attrs):
        a = f"{v.name} : {v.type}"
        if attrs:
            a += " {" + ", ".join(f"{k} = {val}" for k, val in attrs.items()) + "}"
        args.append(a)
    rets = ", ".join(str(v.type) for v in returns)
    rets = f"({rets})" if len(returns) != 1 else rets
    out.append(f"  func.func @{func_name}({', '.join(args)}) -> {rets} attributes {{entrance}} {{")
    for op in block.ops:
        lhs = ", ".join(r.name for r in op.results)
        lhs = lhs + " = " if lhs else ""
        operands = ", ".join(o.name for o in op.operands)
        props = ""
        if op.props:
            props = " <{" + ", ".join(f"{k} = {v}" for k, v in op.props.items()) + "}>"
        in_types = ", ".join(str(o.type) for o in op.operands)
        if len(op.result_types) == 1:
            out_types = str(op.result_types[0])
        else:
            out_types = "(" + ", ".join(str(t) for t in op.result_types) + ")"
        out.append(f'    {lhs}"{op.name}"({operands}){props} : ({in_types}) -> {out_types}')
    if returns:
        out.append("    func.return " + ", ".join(v.name for v in returns) + " : "
                   + ", ".join(str(v.type) for v in returns))
    else:
        out.append("    func.return")
    out.append("  }")
    out.append("}")
    return "\n".join(out) + "\n"
