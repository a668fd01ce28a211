"""``LLCompiler``: the torch.compile backend, same constructor and call surface as the
reference class (llcompiler/compiler/compiler.py:41-168), targeting the B200 pipeline.

Flow of one compilation (reference flow in parentheses):
  dynamo FX graph -> aot_autograd with LLC_DECOMPOSITIONS (compiler.py:161-166)
  -> importer: FX -> LLH text (compiler.py:128)
  -> llcompiler_.compiler.Compiler().compile_mlir_to_shared_lib(text, options) (compiler.py:132-135)
  -> Torch_ExecutionEngine(path) (compiler.py:136)

What differs: weights.  Current torch hands every parameter to the backend as a graph
input, so the compiled function receives them on each call.  In inference mode they are
frozen the first time the function runs: written once as ``.npy`` next to the plan, named
by the module's ``llh.weight`` ops, uploaded once by ``Execution.load`` and dropped from
the run-time argument list.  Later changes to the parameters are therefore not seen; build
a new compiled model after changing weights.
"""
from __future__ import annotations

import tempfile
from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.fx
from torch._decomp import get_decompositions
from torch._dynamo.backends.common import aot_autograd

from ..importer import ImportedFunction, Importer, save_weight
from .torch_compile_config import LLC_DECOMPOSITIONS, unsupported_nodes


class CompiledFunction:
    """What aot_autograd calls in place of the FX graph: filters the flat argument list into
    symbol values and run-time tensors and forwards to the execution engine."""

    _boxed_call = True

    def __init__(self, imported: ImportedFunction, plan_path: str, engine_factory: Callable[[str], Any]):
        self.imported = imported
        self.plan_path = plan_path
        self._engine_factory = engine_factory
        self.engine = None

    def _freeze(self, args: Sequence[Any]) -> None:
        for pos, path in self.imported.weight_files:
            save_weight(path, args[pos])
        self.engine = self._engine_factory(self.plan_path)

    def __call__(self, args):
        args = list(args)
        if self.engine is None:
            self._freeze(args)
        im = self.imported
        symbols = [int(args[p]) for p in im.symbol_positions]
        tensors = [args[p] for p in im.tensor_positions]
        outs = self.engine.run(*symbols, *tensors)
        if not isinstance(outs, (list, tuple)):
            outs = [outs]
        return tuple(outs) if im.output_is_tuple else outs[0]


class LLCompiler(Importer):
    def __init__(
        self,
        mode: str = "inference",
        target: str = "sm_100a",
        pipeline: str = "cuda",
        index_bit_width: int = 64,
        symbol_infer: bool = True,
        target_layout: str = "NCHW",
        vebose_first_ir: bool = False,
        log_root: str = "",
        log_level: str = "debug",
        log_llvm: bool = True,
        cpu: str = "",
        mtriple: str = "",
        precision: str = "auto",
        device: Optional[int] = None,
        **kwargs,
    ) -> None:
        super().__init__(**kwargs)
        self.vebose_first_ir = vebose_first_ir
        self.pipeline = pipeline
        self.mode = mode
        self.log_root = log_root
        self.log_level = log_level
        self.target = target
        self.target_layout = target_layout
        self.log_llvm = log_llvm
        self.cpu = cpu
        self.mtriple = mtriple
        self.precision = precision
        self.device = device
        self.index_bit_width = index_bit_width
        self.symbol_infer = symbol_infer
        self.compile_count = 0
        self.compiled: List[CompiledFunction] = []

    # -- reference: compiler.py:99-114
    def _gen_compiler_options(self):
        from llcompiler_.compiler import CompileOptions
        o = CompileOptions()
        o.set_log_root(self.log_root if self.log_root == "" else self.log_root + "_" + str(self.compile_count))
        o.set_mode(self.mode)
        o.set_target(self.target)
        o.set_log_level(self.log_level)
        o.set_pipeline(self.pipeline)
        o.set_global_layout(self.target_layout)
        o.set_cpu(self.cpu)
        o.set_mtriple(self.mtriple)
        o.set_precision(self.precision)
        self.compile_count += 1
        return o

    def _compile_text(self, text: str) -> str:
        from llcompiler_.compiler import Compiler
        return Compiler().compile_mlir_to_shared_lib(text, self._gen_compiler_options())

    def _make_engine(self, plan_path: str):
        from ..executor import Torch_ExecutionEngine
        return Torch_ExecutionEngine(plan_path, device=self.device)

    # -- reference: compiler.py:116-138
    def compiler_fx(self, model: torch.fx.GraphModule, inputs: List[torch.Tensor], **kwargs):
        missing = unsupported_nodes(model)
        if missing:
            raise NotImplementedError("no LLH translation for: " + ", ".join(missing))
        static = ()
        if self.mode == "inference":
            ctx = torch._guards.TracingContext.try_get()
            if ctx is not None and getattr(ctx, "fw_metadata", None) is not None:
                static = tuple(ctx.fw_metadata.static_input_indices)
        return self.compiler_fx_submodule(model, static_positions=static)

    def compiler_fx_submodule(self, model: torch.fx.GraphModule, static_positions: Sequence[int] = (), **kwargs):
        weight_dir = tempfile.mkdtemp(prefix="LLcompiler_weight_")
        imported = self.importer(model, static_positions, weight_dir)
        self._mlir_module = imported.text
        if self.vebose_first_ir:
            print(imported.text)
        plan_path = self._compile_text(imported.text)
        fn = CompiledFunction(imported, plan_path, self._make_engine)
        self.compiled.append(fn)
        return fn

    def compile_onnx(self, model):
        """An ONNX model (onnx.ModelProto, the bytes of a .onnx file, or its path) -> a callable that takes the graph's
        inputs in order and returns its outputs.  The reference names this entry (llcompiler/importer/importer.py:52-54)
        but stops at a stub; weights are the model's initialisers, written out as .npy at import."""
        weight_dir = tempfile.mkdtemp(prefix="LLcompiler_weight_")
        imported = self.importer(model, (), weight_dir)
        self._mlir_module = imported.text
        plan_path = self._compile_text(imported.text)
        fn = CompiledFunction(imported, plan_path, self._make_engine)
        self.compiled.append(fn)
        return lambda *tensors: fn(tensors)

    # -- reference: compiler.py:140-168
    def __call__(self, model, inputs: List[torch.Tensor]) -> Any:
        if not isinstance(model, torch.fx.GraphModule):
            raise ValueError("Unsupported")
        if self.mode != "inference":
            raise NotImplementedError("the B200 pipeline compiles inference graphs only")
        return aot_autograd(
            fw_compiler=self.compiler_fx,
            inference_compiler=self.compiler_fx,
            decompositions=get_decompositions(LLC_DECOMPOSITIONS),
        )(model, inputs)
