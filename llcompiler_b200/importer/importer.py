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
        if type(model).__name__ == "ModelProto" or isinstance(model, (bytes, bytearray)) or \
                (isinstance(model, str) and model.endswith(".onnx")):
            return self._importer_onnx(model, weight_dir)
        if isinstance(model, torch.nn.Module):
            return self._importer_torch_module(model)
        raise NotImplementedError(f"cannot import {type(model)}")

    def _importer_fx_module(self, model: torch.fx.GraphModule, static_positions=(), weight_dir=None) -> ImportedFunction:
        return torch_translate_to_mlir_text(model, static_positions, weight_dir)

    def _importer_torch_module(self, model: torch.nn.Module):
        raise NotImplementedError("pass the module through torch.compile(model, backend=LLCompiler(...))")

    def _importer_onnx(self, model, weight_dir=None) -> ImportedFunction:
        # the reference's ONNX entry is a stub (llcompiler/importer/importer.py:52-54); here a ModelProto, the bytes of a
        # .onnx file or its path are decoded without the onnx package (static or named extents, the MLP, ResNet and encoder-layer operator set)
        from .onnx_translate import onnx_translate_to_mlir_text
        return onnx_translate_to_mlir_text(model, weight_dir)
