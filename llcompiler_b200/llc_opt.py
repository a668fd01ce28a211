"""`llc-opt` for the textual LLH surface: runs passes of the C++ compile library over a file and prints the result,
the way the reference's lit files drive its tool (`// RUN: llc-opt --split-input-file --<pass> %s | FileCheck %s`,
test/lit.cfg.py:49-61; tools/llc-opt/llc-opt.cpp:37-60).

    python -m llcompiler_b200.llc_opt --infer-symbol-shape [--split-input-file] file.mlir

Passes (several are applied in the order given, as one pipeline): --parse, --operation-legalization,
--remove-redundant-ops, --fuse-softmax, --infer-symbol-shape, --decompose-ops, --transform-layout, --canonicalize,
--inline, --cse, --symbol-cse, --unload-and-bind-encoding, --lower (the kernel plan).  `-` reads standard input.
"""
from __future__ import annotations

import sys

from . import _capi

PASSES = ("parse", "operation-legalization", "remove-redundant-ops", "fuse-softmax", "infer-symbol-shape", "decompose-ops", "transform-layout",
          "canonicalize", "inline", "cse", "symbol-cse", "unload-and-bind-encoding", "lower")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    split = "--split-input-file" in argv
    names = [a.lstrip("-") for a in argv if a.startswith("--") and a != "--split-input-file"]
    files = [a for a in argv if not a.startswith("--")]
    bad = [n for n in names if n not in PASSES]
    if bad or len(files) != 1:
        sys.stderr.write(__doc__ + (f"\nunknown pass: {bad[0]}\n" if bad else ""))
        return 2
    text = sys.stdin.read() if files[0] == "-" else open(files[0]).read()
    pieces = text.split("// -----") if split else [text]
    outs = []
    for piece in pieces:
        try:
            # the passes run as one pipeline over the parsed module, as llc-opt's do
            cur = _capi.run_pass(piece, ",".join(names or ["parse"])).split("// -----")[0]
            outs.append(cur.rstrip("\n"))
        except _capi.LlcError as e:
            sys.stderr.write(f"error: {e}\n")
            return 1
    sys.stdout.write("\n// -----\n".join(outs) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
