from .importer import Importer
from .fx_translate import torch_translate_to_mlir_text, ImportedFunction, save_weight

__all__ = ["Importer", "torch_translate_to_mlir_text", "ImportedFunction", "save_weight"]
