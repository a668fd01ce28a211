"""Import alias: the reference's package name (`from llcompiler.compiler import LLCompiler`,
llcompiler/compiler/compiler.py:41 in the reference) served by llcompiler_b200, so that a script written
against the reference runs unchanged.  `llcompiler.compiler`, `llcompiler.executor`, `llcompiler.importer`,
`llcompiler.dialect` and `llcompiler.utility` are the llcompiler_b200 modules of the same name."""
import importlib
import sys

import llcompiler_b200 as _impl

for _name in ("compiler", "executor", "importer", "dialect", "utility"):
    _mod = importlib.import_module(f"llcompiler_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod

from llcompiler_b200.compiler import LLCompiler  # noqa: E402,F401  (the reference's __init__ exports it)
