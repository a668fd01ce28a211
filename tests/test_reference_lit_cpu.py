"""The reference's own lit files (`// RUN: llc-opt --<pass> %s | FileCheck %s`, test/lit.cfg.py:49-61) driven
through llc_run_pass and a small FileCheck.  The files are read from the reference tree where it is present
(they are not copied here); the FileCheck itself is tested on inline text either way."""
import glob
import os
import re

import pytest

import filecheck_lite as F
from llcompiler_b200 import _capi
from reference_tree import reference_path

REF = reference_path("test", "Dialect", "LLH") or ""
PASSES = {"--infer-symbol-shape": "infer-symbol-shape", "-infer-symbol-shape": "infer-symbol-shape", "--operation-legalization": "operation-legalization",
          "--remove-redundant-ops": "remove-redundant-ops", "--decompose-ops": "decompose-ops", "--transform-layout": "transform-layout",
          "--canonicalize": "canonicalize", "-canonicalize": "canonicalize", "--inline": "inline", "--cse": "cse",
          "--unload-and-bind-encoding": "unload-and-bind-encoding", "--symbol-cse": "symbol-cse"}
# functions of each file whose CHECK lines hold on this implementation's output (None: all of them)
EXPECTED = {
    "infer_symbol_shape.mlir": None,
    "extra_symbol_infer_shape.mlir": None,
    "canonicalize_symbol.mlir": None,
    "symbol_cse.mlir": None,
    "remove_redundant_ops.mlir": None,      # all of them
    "operation-legalization.mlir": None,
    "decompose_ops.mlir": None,
    "transform_layout.mlir": None,
    "canonicalize.mlir": None,
    "fold.mlir": None,
    "insert_braodcast.mlir": None,
    "reshape_before_braodcast.mlir": None,
    "layout_canonicalize.mlir": None,
    "unload_and_bind_encoding.mlir": None,
    "ops.mlir": None,
}


def test_filecheck_directives():
    text = "func.func @f(%a: i32)\n  %0 = \"x.op\"() : () -> tensor<4xf32, #enc<@c4>>\n  return %0\n"
    src = "// CHECK-LABEL: f\n// CHECK: x.op\n// CHECK-SAME: tensor<4xf32, #enc<@c4>>\n// CHECK-NEXT: return\n// CHECK-NOT: y.op\n"
    assert F.check(text, F.directives(src))[0]
    assert not F.check(text, F.directives("// CHECK: x.op\n// CHECK-SAME: tensor<5xf32"))[0]
    assert not F.check(text, F.directives("// CHECK: return\n// CHECK: x.op"))[0]              # order matters
    assert F.check(text, F.directives("// CHECK: tensor<{{[0-9]+}}xf32"))[0]
    assert not F.check(text, F.directives("// CHECK-NOT: x.op\n// CHECK: return"))[0]
    assert F.directives("// CHECK-ENCODING: abc\n// CHECK: d", "CHECK") == [("PLAIN", "d")]


def _run_file(path):
    src = open(path).read()
    # the passes of the first RUN line, in order (flags that only steer the driver or that MLIR itself provides for
    # printing are left out; a file whose RUN line names no pass is parsed and printed back)
    run = re.findall(r"RUN: llc-opt (.*?)\|", src)
    flags = re.findall(r"(--?[\w-]+)(?:=\"[^\"]*\")?", run[0]) if run else []
    chain = [PASSES[f] for f in flags if f in PASSES]
    unknown = [f for f in flags if f not in PASSES and f not in ("--split-input-file", "--mlir-print-op-generic")]
    name = ",".join(chain) if chain else ("parse" if run and not unknown else None)
    if unknown:
        name = None
    results = {}
    for piece in src.split("// -----"):
        fn = re.search(r"func\.func @(\w+)", piece)
        if not fn or name is None:
            continue
        try:
            out = _capi.run_pass(piece, name)
            ok = F.check(out, F.directives(piece))[0]
        except _capi.LlcError:
            ok = False
        results[fn.group(1)] = results.get(fn.group(1), True) and ok
    return results


@pytest.mark.parametrize("fname", sorted(EXPECTED))
def test_reference_check_lines_hold(fname):
    paths = glob.glob(os.path.join(REF, "**", fname), recursive=True)
    if not paths:
        pytest.skip("reference tree not present")
    results = _run_file(paths[0])
    assert results, "no test functions found"
    want = EXPECTED[fname] if EXPECTED[fname] is not None else set(results)
    failed = sorted(n for n in want if not results.get(n, False))
    assert not failed, f"CHECK lines no longer hold for {failed}"


def test_llc_opt_command_line(tmp_path, capsys):
    from llcompiler_b200 import llc_opt
    f = tmp_path / "t.mlir"
    f.write_text('func.func @t(%arg0: tensor<?x3x?x?xf32>) -> (tensor<*xf32>) attributes {entrance} {\n'
                 '  %0 = "llh.transpose"(%arg0) <{perms = array<i64: 3, 2, 1, 0>}> : (tensor<?x3x?x?xf32>) -> tensor<*xf32>\n'
                 '  return %0: tensor<*xf32>\n}\n// -----\n'
                 'func.func @u(%arg0: tensor<2x2xf32>) -> (tensor<2x2xf32>) attributes {entrance} {\n  return %arg0: tensor<2x2xf32>\n}\n')
    assert llc_opt.main(["--split-input-file", "--infer-symbol-shape", str(f)]) == 0
    out = capsys.readouterr().out
    assert "tensor<?x?x3x?xf32, #llh.encoding<shapes = @s2, @s1, @c3, @s0>>" in out and out.count("// -----") == 1
    assert '"llh.symbolic_int"() <{sym_name = "c3"}>' in out
    assert llc_opt.main(["--no-such-pass", str(f)]) == 2
