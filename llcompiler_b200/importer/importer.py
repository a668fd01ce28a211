"""Front door of the importer, mirroring llcompiler/importer/importer.py:31-54."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.fx

from .fx_translate import ImportedFunction, torch_translate_to_mlir_text


class Importer:
    def __init__(self, **kwargs) -> None:
        pass

    def importer(self, model, static_positions: Sequence[int] = (), weight_dir: Optional[str] = None) -> ImportedFunction:
        if isinstance(model, torch.fx.GraphModule):
            return self._importer_fx_module(model, static_positions, weight_dir)
        if type(model).__name__ == "ModelProto":
            return self._importer_onnx(model)
        if isinstance(model, torch.nn.Module):
            return self._importer_torch_module(model)
        raise NotImplementedError(f"cannot import {type(model)}")

    def _importer_fx_module(self, model: torch.fx.GraphModule, static_positions=(), weight_dir=None) -> ImportedFunction:
        return torch_translate_to_mlir_text(model, static_positions, weight_dir)

    def _importer_torch_module(self, model: torch.nn.Module):
        raise NotImplementedError("pass the module through torch.compile(model, backend=LLCompiler(...))")

    def _importer_onnx(self, model):
        # the reference's ONNX entry is a stub that raises (llcompiler/importer/mlir_gen.py:82-99)
        raise NotImplementedError("ONNX import is not implemented")
