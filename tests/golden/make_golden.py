"""Regenerates tests/golden/op_vectors.pt: for every op case in tests/op_models.py the seeded
inputs' checksum and the PyTorch CPU eager fp32 output.  PyTorch CPU eager is what the
reference compares its compiled results with (llcompiler/test_models/utility.py:18-28), so
these are outputs of the reference's own correctness pin, produced on this machine
(torch version recorded in the file).  tests/golden/op_vectors_reference_shapes.pt holds the same families at the
input shapes the reference's scripts use (3x3x224x224, 10x100000, ...) as a strided sample per output.  Run:  python tests/golden/make_golden.py
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from op_models import OP_CASES, REFERENCE_SHAPE_CASES, build_case, build_reference_shape_case, sample_of  # noqa: E402

out = {"torch": str(torch.__version__), "cases": {}}
torch.set_num_threads(1)
for name in OP_CASES:
    model, inputs, exact = build_case(name)
    with torch.no_grad():
        y = model(*inputs)
    out["cases"][name] = {"output": y.clone(), "input_sum": [float(i.double().sum()) for i in inputs]}
torch.save(out, os.path.join(HERE, "op_vectors.pt"))
print("wrote", len(out["cases"]), "cases")

# the same families at the reference's own input shapes: a strided sample of each output, its shape and its sum
ref = {"torch": str(torch.__version__), "cases": {}}
for name in REFERENCE_SHAPE_CASES:
    model, inputs, exact = build_reference_shape_case(name)
    with torch.no_grad():
        y = model(*inputs)
    ref["cases"][name] = {"sample": sample_of(y), "shape": list(y.shape), "sum": float(y.double().sum()),
                          "input_sum": [float(i.double().sum()) for i in inputs]}
torch.save(ref, os.path.join(HERE, "op_vectors_reference_shapes.pt"))
print("wrote", len(ref["cases"]), "reference-shape cases")
