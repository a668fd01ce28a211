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

import hashlib
import json
import os
import shutil
import tempfile
from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.fx
from torch._decomp import get_decompositions
from torch._dynamo.backends.common import aot_autograd

from ..importer import ImportedFunction, Importer, save_weight
from .torch_compile_config import LLC_DECOMPOSITIONS, unsupported_nodes


def cache_root() -> Optional[str]:
    """Directory of the plan and weight cache: ``LLC_CACHE_DIR``, else ``llcompiler_b200_cache_<uid>`` under the
    temporary directory; ``LLC_CACHE_DIR=off`` (or empty) switches the cache off."""
    env = os.environ.get("LLC_CACHE_DIR")
    if env is not None:
        return None if env.strip().lower() in ("", "off", "0", "none") else env
    return os.path.join(tempfile.gettempdir(), f"llcompiler_b200_cache_{os.getuid()}")


def _tensor_digest(h, t: torch.Tensor) -> None:
    t = t.detach()
    h.update(f"{t.dtype}{tuple(t.shape)}".encode())
    c = t.contiguous().cpu()
    h.update(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")


class CompiledFunction:
    """What aot_autograd calls in place of the FX graph: filters the flat argument list into
    symbol values and run-time tensors and forwards to the execution engine."""

    _boxed_call = True

    def __init__(self, imported: ImportedFunction, plan_path: str, engine_factory: Callable[..., Any], cache_entry: Optional[str] = None):
        self.imported = imported
        self.plan_path = plan_path
        self._engine_factory = engine_factory
        self.cache_entry = cache_entry       # directory of this graph in the cache (None: no cache)
        self.weight_dir: Optional[str] = None
        self.engine = None

    def _freeze(self, args: Sequence[Any]) -> None:
        if self.cache_entry is None:
            for pos, path in self.imported.weight_files:
                save_weight(path, args[pos])
            self.engine = self._engine_factory(self.plan_path)
            return
        # The weights are named by their content: one directory per set of values under the graph's cache entry.  A set
        # that is already there (marker file) is not written again, and the executor finds its uploaded pool beside it.
        h = hashlib.blake2b(digest_size=16)
        for pos, _ in self.imported.weight_files:
            _tensor_digest(h, args[pos])
        def write_set(directory: str) -> None:
            for pos, path in self.imported.weight_files:
                save_weight(os.path.join(directory, os.path.basename(path)), args[pos])

        self.weight_dir = publish_weight_set(self.cache_entry, "v_" + h.hexdigest(), write_set)
        self.engine = self._engine_factory(self.plan_path, self.weight_dir)

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


def publish_weight_set(entry: str, name: str, write_set) -> str:
    """Directory ``entry/name`` holding a complete weight set, written at most once however many processes ask for it at
    the same time (the ranks of a multi-GPU job all compile the same graph).  A writer fills a directory of its own and
    renames it into place, so a reader never sees a file that is still being written; the loser of that race throws its
    copy away.  Returns the directory to load from."""
    final = os.path.join(entry, name)
    marker = os.path.join(final, ".complete")
    if os.path.exists(marker):
        return final
    tmp = tempfile.mkdtemp(prefix=name + ".tmp", dir=entry)
    write_set(tmp)
    open(os.path.join(tmp, ".complete"), "w").close()
    try:
        os.rename(tmp, final)
        return final
    except OSError:
        if os.path.exists(marker):                     # another process published the same set first
            shutil.rmtree(tmp, ignore_errors=True)
            return final
        return tmp                                     # something unfinished sits under that name: keep the private copy


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
        self.cache_hits = 0                  # compilations served from the plan cache
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

    def _make_engine(self, plan_path: str, weight_dir: Optional[str] = None):
        from ..executor import Torch_ExecutionEngine
        return Torch_ExecutionEngine(plan_path, device=self.device, weight_dir=weight_dir)

    # -- the plan and weight cache (the reference derives its artefact's name from a hash of the module text,
    #    src/Compiler/Compiler.cpp:305-309, but rebuilds it and rewrites every weight on each compile)
    def _graph_key(self, model: torch.fx.GraphModule, static_positions: Sequence[int]) -> str:
        """What the plan depends on besides the weights' values: the FX graph, the placeholders' types, which of them are
        frozen, the options, the switches that change the lowering, the values of tensors held by the graph itself, and
        the library build."""
        h = hashlib.blake2b(digest_size=16)
        h.update(str(model.graph).encode())
        for n in model.graph.nodes:
            if n.op == "placeholder":
                v = n.meta.get("val")
                h.update(f"{n.name}:{getattr(v, 'dtype', type(v).__name__)}:{[str(d) for d in getattr(v, 'shape', [])] if hasattr(v, 'shape') else str(v)}".encode())
            elif n.op == "get_attr":
                t = getattr(model, n.target, None)
                if isinstance(t, torch.Tensor):
                    _tensor_digest(h, t)
        opts = (tuple(static_positions), self.mode, self.target, self.pipeline, self.target_layout, self.precision, self.log_root,
                os.environ.get("LLC_FUSE_ATTENTION", ""), os.environ.get("LLC_MERGE_STEM_ROWS", ""), os.environ.get("LLC_FUSE_SIBLING_GEMMS", ""), type(self).__name__)
        h.update(repr(opts).encode())
        from .. import _capi
        st = os.stat(_capi.LIB_PATH)
        h.update(f"{st.st_size}:{st.st_mtime_ns}:{torch.__version__}".encode())
        return h.hexdigest()

    def _compile_cached(self, model, static_positions: Sequence[int], key: Optional[str]) -> CompiledFunction:
        root = cache_root()
        if root is None or key is None:
            weight_dir = tempfile.mkdtemp(prefix="LLcompiler_weight_")
            imported = self.importer(model, static_positions, weight_dir)
            self._mlir_module = imported.text
            if self.vebose_first_ir:
                print(imported.text)
            return CompiledFunction(imported, self._compile_text(imported.text), self._make_engine)
        entry = os.path.join(root, "g_" + key)
        meta_path, plan_path = os.path.join(entry, "imported.json"), os.path.join(entry, "plan.llcplan")
        if os.path.exists(meta_path) and os.path.exists(plan_path):
            # the same graph was compiled before (by this or another process): no import, no lowering
            meta = json.load(open(meta_path))
            imported = ImportedFunction()
            imported.text = meta["text"]
            imported.weight_files = [(int(p), f) for p, f in meta["weight_files"]]
            imported.symbol_positions, imported.tensor_positions = meta["symbol_positions"], meta["tensor_positions"]
            imported.output_is_tuple, imported.num_placeholders = meta["output_is_tuple"], meta["num_placeholders"]
            self.cache_hits += 1
        else:
            os.makedirs(os.path.join(entry, "w"), exist_ok=True)
            imported = self.importer(model, static_positions, os.path.join(entry, "w"))
            tmp_plan = self._compile_text(imported.text)
            shutil.copyfile(tmp_plan, plan_path + f".tmp{os.getpid()}")
            os.replace(plan_path + f".tmp{os.getpid()}", plan_path)
            meta = {"text": imported.text, "weight_files": [[p, f] for p, f in imported.weight_files],
                    "symbol_positions": imported.symbol_positions, "tensor_positions": imported.tensor_positions,
                    "output_is_tuple": imported.output_is_tuple, "num_placeholders": imported.num_placeholders}
            with open(meta_path + f".tmp{os.getpid()}", "w") as f:
                json.dump(meta, f)
            os.replace(meta_path + f".tmp{os.getpid()}", meta_path)
        self._mlir_module = imported.text
        if self.vebose_first_ir:
            print(imported.text)
        return CompiledFunction(imported, plan_path, self._make_engine, cache_entry=entry)

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
        fn = self._compile_cached(model, static_positions, self._graph_key(model, static_positions) if cache_root() else None)
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
