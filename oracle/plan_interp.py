"""CPU oracle, part 2: an interpreter for kernel plans.

TEST INFRASTRUCTURE ONLY (never imported by the product path).  It executes
the text plan the GPU pipeline emits with plain PyTorch CPU ops, one op per
plan step, so that the *compiler* (parsing, symbolic shapes, stride algebra,
epilogue fusion, buffer reuse) can be checked against eager PyTorch on a
machine without a GPU, and so that each CUDA kernel has a step-level
restatement to be compared with.

Each step follows the reference's lowering of the LLH op(s) it was fused from:
  gemm      llh.matmul / llh.batch_matmul -> stablehlo.dot / dot_general
            (src/Conversion/LLHToHLO/LLHToHLO.cpp:363-382, :485)
  conv      llh.conv -> stablehlo.convolution, NCHW x FCHW (LLHToHLO.cpp:214-270)
            + batch-norm inference as a per-channel affine map
            (src/Dialect/LLH/Transforms/DecomposeOps.cpp:125-144)
  maxpool   llh.max_pool -> stablehlo.reduce_window (LLHToHLO.cpp:295-339); the
            window is initialised with -inf here, the reference uses 0
            (:313-314), which only differs for all-negative windows
  reduce    llh.reduce_* -> stablehlo.reduce (LLHToHLO.cpp:81-171)
  softmax   amax, sub, exp, sum, div (llcompiler/compiler/torch_compile_config.py:24)
  eltwise   llh.add/sub/mul/div/max/... -> stablehlo elementwise (LLHToHLO.cpp:479-490)
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np
import torch
import torch.nn.functional as F

_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "f64": torch.float64,
       "i64": torch.int64, "i32": torch.int32, "i16": torch.int16, "i8": torch.int8, "i1": torch.bool}


def load_npy(path: str, dtype: str) -> torch.Tensor:
    arr = np.load(path)
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dtype == "bf16":
        t = t.view(torch.int16).view(torch.bfloat16) if t.dtype != torch.bfloat16 else t
    return t.reshape(-1)


class PlanInterpreter:
    def __init__(self, text: str, weight_dir: str = ""):
        self.weight_dir = weight_dir       # when set, weight files are looked up there by name first (as llc_load_from does)
        self.options: Dict[str, str] = {}
        self.symbols: List[tuple] = []
        self.buffers: List[dict] = []
        self.inputs: List[dict] = []
        self.outputs: List[dict] = []
        self.steps: List[dict] = []
        self.nsymargs = 0
        for line in text.splitlines():
            tok = line.split()
            if not tok or tok[0] in ("llcplan", "//"):
                continue
            kw = tok[0]
            if kw == "option":
                self.options[tok[1]] = " ".join(tok[2:])
            elif kw == "nsymargs":
                self.nsymargs = int(tok[1])
            elif kw == "symbol":
                self.symbols.append((tok[1], tok[2], [int(x) for x in tok[3:]]))
            elif kw == "buffer":
                b = {"dtype": tok[2], "kind": tok[3], "numel": tok[4], "index": -1, "file": None, "values": None}
                rest = line.split(None, 5)[5] if len(tok) > 5 else ""
                if 'file="' in rest:
                    b["file"] = rest.split('file="')[1].split('"')[0]
                for t in rest.split():
                    if t.startswith("index="):
                        b["index"] = int(t[6:])
                    if t.startswith("values="):
                        b["values"] = [float(x) for x in t[7:].split(",")]
                self.buffers.append(b)
            elif kw in ("input", "output"):
                d = {"buf": int(tok[2]), "dtype": tok[3], "shape": _split(tok[4])}
                (self.inputs if kw == "input" else self.outputs).append(d)
            elif kw in ("step", "init"):
                s = {"init": kw == "init", "kernel": tok[1], "views": {}, "params": {}}
                for t in tok[2:]:
                    eq, co = t.find("="), t.find(":")
                    if eq > 0 and (co < 0 or eq < co) and t[eq + 1] == "b" and "@" in t:
                        s["views"][t[:eq]] = _parse_view(t[eq + 1:])
                    else:
                        s["params"][t[:co]] = t[co + 1:]
                self.steps.append(s)
            else:
                raise ValueError(f"unknown plan line: {line}")
        self._weights: Dict[int, torch.Tensor] = {}

    # ------------------------------------------------------------------ run
    def bind(self, symbols: Sequence[int], inputs: Sequence[torch.Tensor]) -> Dict[str, int]:
        env: Dict[str, int] = {}
        for name, how, pos in self.symbols:
            val = symbols[pos[0]] if how == "arg" else inputs[pos[0]].shape[pos[1]]
            if env.setdefault(name, int(val)) != int(val):
                raise ValueError(f"symbol {name} bound to both {env[name]} and {val}")
        return env

    def run(self, inputs: Sequence[torch.Tensor], symbols: Sequence[int] = ()) -> List[torch.Tensor]:
        env = self.bind(symbols, inputs)
        mem: Dict[int, torch.Tensor] = {}
        for i, b in enumerate(self.buffers):
            n = _ev(b["numel"], env)
            dt = _DT[b["dtype"]]
            if b["kind"] == "input":
                mem[i] = inputs[b["index"]].contiguous().reshape(-1).to(dt)
            elif b["kind"] == "weight":
                if i not in self._weights:
                    path = b["file"]
                    if self.weight_dir:
                        import os
                        cand = os.path.join(self.weight_dir, os.path.basename(path))
                        path = cand if os.path.exists(cand) else path
                    self._weights[i] = load_npy(path, b["dtype"]).to(dt)
                mem[i] = self._weights[i]
            elif b["values"] is not None:
                mem[i] = torch.tensor(b["values"], dtype=torch.float64).to(dt)
            else:
                mem[i] = torch.full((max(n, 1),), float("nan") if dt.is_floating_point else 0, dtype=dt)
        for s in self.steps:
            views = {k: _as_view(mem, v, env) for k, v in s["views"].items()}
            getattr(self, "_k_" + s["kernel"])(views, s["params"])
        outs = []
        for o in self.outputs:
            shape = [_ev(d, env) for d in o["shape"]]
            outs.append(mem[o["buf"]][: math.prod(shape)].reshape(shape))
        return outs

    # ------------------------------------------------------------------ kernels
    @staticmethod
    def _epilogue(acc, v, p):
        acc = acc * float(p.get("alpha", "1"))
        cshape = [1] * acc.dim()
        if "scale" in v:
            acc = acc * v["scale"].float().reshape(-1)
        if "shift" in v:
            acc = acc + v["shift"].float().reshape(-1)
        if "res" in v:
            acc = acc + v["res"].float()
        act = p.get("act", "none")
        if act == "relu":
            acc = torch.relu(acc)
        elif act == "gelu":
            acc = F.gelu(acc)
        return acc

    def _k_gemm(self, v, p):
        a, b = v["a"].float(), v["b"].float()
        acc = torch.matmul(a, b)                      # [b0,b1,M,N], channel = last dim
        v["out"].copy_(self._epilogue(acc, v, p).to(v["out"].dtype))

    def _k_conv(self, v, p):
        x = v["x"].float()                            # logical NCHW
        w = v["w"].float().permute(0, 3, 1, 2)        # [F,KH,KW,C] -> FCHW
        st, pad, dil = _ints(p["stride"]), _ints(p["pad"]), _ints(p["dil"])
        x = F.pad(x, (pad[1], pad[3], pad[0], pad[2]))
        acc = F.conv2d(x, w, None, st, 0, dil)        # NCHW
        acc = acc.permute(0, 2, 3, 1)                 # channel last for the epilogue
        vv = dict(v)
        if "res" in vv:
            vv["res"] = vv["res"].permute(0, 2, 3, 1)
        out = self._epilogue(acc, vv, p).permute(0, 3, 1, 2)
        v["out"].copy_(out.to(v["out"].dtype))

    def _k_maxpool(self, v, p):
        x = v["x"].float()
        k, st, pad, dil = _ints(p["kernel"]), _ints(p["stride"]), _ints(p["pad"]), _ints(p["dil"])
        x = F.pad(x, (pad[1], pad[3], pad[0], pad[2]), value=float("-inf"))
        out = F.max_pool2d(x, k, st, 0, dil)
        oh, ow = v["out"].shape[2], v["out"].shape[3]
        v["out"].copy_(out[:, :, :oh, :ow].to(v["out"].dtype))

    def _k_reduce(self, v, p):
        x = v["x"].float()
        op = p["op"]
        r = {"sum": lambda t: t.sum(1), "mean": lambda t: t.mean(1), "max": lambda t: t.amax(1),
             "min": lambda t: t.amin(1)}[op](x)
        v["out"].copy_(r.to(v["out"].dtype))

    def _k_softmax(self, v, p):
        x = v["x"].float()
        m = x.amax(-1, keepdim=True)
        e = torch.exp(x - m)
        v["out"].copy_((e / e.sum(-1, keepdim=True)).to(v["out"].dtype))

    def _k_attention(self, v, p):
        # q, out [b0,b1,M,D]; k [b0,b1,D,N]; v [b0,b1,N,D]; mask broadcast view [b0,b1,M,N]
        s = torch.matmul(v["q"].float(), v["k"].float()) * float(p.get("scale", "1"))
        if "mask" in v:
            s = s + v["mask"].float()
        v["out"].copy_(torch.matmul(torch.softmax(s, -1), v["v"].float()).to(v["out"].dtype))

    def _k_layernorm(self, v, p):
        x = v["x"].float()
        out = F.layer_norm(x, (x.shape[-1],), v["gamma"].float(), v["beta"].float(), float(p["eps"]))
        v["out"].copy_(out.to(v["out"].dtype))

    def _k_nchw2nhwc(self, v, p):
        # llh.transpose perms [0,2,3,1] around conv (src/Dialect/LLH/Transforms/TransformLayout.cpp:141-198);
        # the output view is logical NCHW over an NHWC buffer, extra channels are zero
        out, x = v["out"], v["x"]
        out.zero_()
        if "wide" in p:                                    # rows widened by a zero halo: image at column `left`
            left = _ints(p["wide"])[0]
            out[:, : x.shape[1], :, left: left + x.shape[3]].copy_(x)
        else:
            out[:, : x.shape[1]].copy_(x)

    def _k_gather(self, v, p):
        v["out"].copy_(v["table"][v["ids"].long()].to(v["out"].dtype))

    def _k_eltwise(self, v, p):
        regs: List[torch.Tensor] = []
        out = v["out"]
        for ins in p["prog"].split(";"):
            if ins.startswith("ld"):
                regs.append(v["in" + ins[2:]].float())
                continue
            if ins.startswith("#"):
                regs.append(torch.tensor(float(ins[1:]), dtype=torch.float32))
                continue
            f = ins.split(",")
            a = [regs[int(i)] for i in f[1:]]
            regs.append(_ELT[f[0]](*a))
        r = regs[-1]
        if not out.dtype.is_floating_point and out.dtype != torch.bool:
            r = torch.trunc(r)
        out.copy_(torch.broadcast_to(r, out.shape).to(out.dtype))


_ELT = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
    "max": torch.maximum, "min": torch.minimum, "pow": torch.pow,
    "relu": torch.relu, "abs": torch.abs, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "exp": torch.exp,
    "gelu": F.gelu, "tanh": torch.tanh, "erf": torch.erf, "sigmoid": torch.sigmoid, "neg": torch.neg,
    "cast": lambda a: a, "trunc": torch.trunc,
    "tf32lo": lambda a: a - (a.contiguous().view(torch.int32) & -8192).view(torch.float32),
    "where": lambda c, a, b: torch.where(c != 0, a, b),
    "eq": lambda a, b: (a == b).float(), "ne": lambda a, b: (a != b).float(), "ge": lambda a, b: (a >= b).float(),
    "gt": lambda a, b: (a > b).float(), "le": lambda a, b: (a <= b).float(), "lt": lambda a, b: (a < b).float(),
}


def _ints(s: str) -> List[int]:
    return [int(x) for x in s.split(",")]


def _split(s: str) -> List[str]:
    out, cur, depth = [], "", 0
    for c in s:
        depth += c == "("
        depth -= c == ")"
        if c == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += c
    if cur:
        out.append(cur)
    return out


def _parse_view(t: str) -> dict:
    at, lb = t.index("@"), t.index("[")
    sc, rb = t.index(";", lb), t.rindex("]")
    return {"buf": int(t[1:at]), "offset": t[at + 1:lb], "shape": _split(t[lb + 1:sc]),
            "strides": _split(t[sc + 1:rb]), "dtype": t[rb + 2:]}


def _ev(text: str, env: Dict[str, int]) -> int:
    return int(eval(text, {"__builtins__": {}}, env))


def _as_view(mem, v, env) -> torch.Tensor:
    shape = [_ev(d, env) for d in v["shape"]]
    strides = [_ev(d, env) for d in v["strides"]]
    base = mem[v["buf"]]
    if _DT[v["dtype"]] != base.dtype:
        raise TypeError(f"view dtype {v['dtype']} does not match buffer dtype {base.dtype}")
    # as_strided takes an offset into the underlying storage, not into `base`
    return torch.as_strided(base, shape, strides, base.storage_offset() + _ev(v["offset"], env))
