from .torch_compile_config import LLC_DECOMPOSITIONS, LLCOperatorSupport
from .compiler import LLCompiler, CompiledFunction

__all__ = ["LLC_DECOMPOSITIONS", "LLCOperatorSupport", "LLCompiler", "CompiledFunction"]
