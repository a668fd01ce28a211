"""Op-level parity on the GPU against the committed golden vectors: each op family of the
reference's op tests (test/python/ops/*.py) is compiled with LLCompiler, run on the GPU through
the llcompiler_ module, static and dynamic shapes, and compared with tests/golden/op_vectors.pt
(PyTorch CPU eager fp32).  Bit-exact for copy / index / max / relu paths, otherwise the
reference's tolerance rtol = atol = 1e-5 (llcompiler/test_models/utility.py:18-21)."""
import copy
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from helpers import compile_with  # noqa: E402
from llcompiler_b200.compiler import LLCompiler  # noqa: E402
from op_models import OP_CASES, REFERENCE_SHAPE_CASES, build_case, build_reference_shape_case, sample_of  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = torch.load(os.path.join(HERE, "golden", "op_vectors.pt"))
GOLDEN_REF_SHAPES = torch.load(os.path.join(HERE, "golden", "op_vectors_reference_shapes.pt"))


@pytest.mark.parametrize("dynamic", [False, True])
@pytest.mark.parametrize("name", sorted(OP_CASES))
def test_op_on_gpu_matches_golden(name, dynamic):
    model, inputs, exact = build_case(name)
    comp = LLCompiler()
    with torch.no_grad():
        got = compile_with(comp, copy.deepcopy(model).cuda(), dynamic)(*[i.cuda() for i in inputs])
    torch.cuda.synchronize()
    want = GOLDEN["cases"][name]["output"]
    assert comp.compiled[0].engine.executor.last_launch_count() > 0
    got = got.cpu()
    assert got.shape == want.shape
    if exact:
        assert torch.equal(got, want)
    else:
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-5, equal_nan=True)


@pytest.mark.parametrize("name", sorted(REFERENCE_SHAPE_CASES))
def test_op_on_gpu_at_the_reference_shapes(name):
    """The reference's op scripts at their own sizes (3x3x224x224 images, a 10 x 100000 linear layer, ...) through
    importer, lowering and the CUDA kernels: the whole output against PyTorch CPU eager computed here, and its strided
    sample against the committed golden vector; the reference's tolerance rtol = atol = 1e-5, bit-exact where it applies."""
    model, inputs, exact = build_reference_shape_case(name)
    comp = LLCompiler()
    with torch.no_grad():
        want = model(*inputs)
        got = compile_with(comp, copy.deepcopy(model).cuda(), False)(*[i.cuda() for i in inputs])
    torch.cuda.synchronize()
    comp.compiled[0].engine.status()
    assert comp.compiled[0].engine.executor.last_launch_count() > 0
    got = got.cpu()
    g = GOLDEN_REF_SHAPES["cases"][name]
    assert list(got.shape) == g["shape"]
    if exact:
        assert torch.equal(got, want) and torch.equal(sample_of(got), g["sample"])
    else:
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-5, equal_nan=True)
        assert torch.allclose(sample_of(got), g["sample"], rtol=1e-5, atol=1e-5, equal_nan=True)


def test_known_answers_on_gpu():
    import json
    from llcompiler_.compiler import Compiler, CompileOptions
    from llcompiler_b200.executor import Torch_ExecutionEngine
    known = json.load(open(os.path.join(HERE, "golden", "known_answers.json")))
    for name, case in known.items():
        if name.startswith("_"):
            continue
        path = Compiler().compile_mlir_to_shared_lib(case["mlir"], CompileOptions())
        eng = Torch_ExecutionEngine(path)
        out = eng.executor.output_shapes([], [])
        res = torch.empty(out[0][0], dtype=torch.float32, device="cuda")
        eng.executor.run([], eng.trans_to_tensor(res))
        torch.cuda.synchronize()
        assert res.cpu().tolist() == case["expect"], name
