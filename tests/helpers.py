"""Shared test plumbing: compile a torch module through the importer and the C-ABI
compiler, then execute either on the CPU plan interpreter (oracle) or on the GPU."""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from llcompiler_b200 import _capi  # noqa: E402
from llcompiler_b200.compiler import LLCompiler  # noqa: E402
from oracle.plan_interp import PlanInterpreter  # noqa: E402


class _InterpEngine:
    def __init__(self, plan_path: str, weight_dir: str = ""):
        self.text = open(plan_path).read()
        self.interp = PlanInterpreter(self.text, weight_dir or "")

    def run(self, *args):
        symbols = [a for a in args if isinstance(a, int)]
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        return self.interp.run(tensors, symbols)


class InterpreterCompiler(LLCompiler):
    """LLCompiler whose plans run on the CPU oracle interpreter (no GPU needed).  Compilation
    still goes through the C ABI (llc_compile)."""

    def _compile_text(self, text: str) -> str:
        return _capi.compile_text(text, mode=self.mode, target=self.target, pipeline=self.pipeline,
                                  global_layout=self.target_layout, precision=self.precision,
                                  log_root=self.log_root or None)

    def _make_engine(self, plan_path: str, weight_dir=None):
        return _InterpEngine(plan_path, weight_dir)


def compile_with(compiler: LLCompiler, model: torch.nn.Module, dynamic: bool = False):
    torch._dynamo.reset()
    return torch.compile(model, backend=compiler, dynamic=dynamic, fullgraph=True)
