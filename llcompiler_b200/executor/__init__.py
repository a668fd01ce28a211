from .engine import ExecutionEngine, Torch_ExecutionEngine

__all__ = ["ExecutionEngine", "Torch_ExecutionEngine"]
