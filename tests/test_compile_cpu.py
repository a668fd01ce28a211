"""Compiler-only checks that need no GPU: importer -> llc_compile -> kernel plan, with the
plan executed by the CPU oracle interpreter and compared with eager PyTorch (the reference's
own parity pin, llcompiler/test_models/utility.py:18-28)."""
import pytest
import torch

from helpers import InterpreterCompiler, compile_with
from oracle.models import build_model, max_rel_err


def _run(model, inputs, dynamic=False, precision="auto"):
    comp = InterpreterCompiler(precision=precision)
    with torch.no_grad():
        want = model(*inputs)
        got = compile_with(comp, model, dynamic)(*inputs)
    return comp, got, want


def test_mlp_dynamic_batch():
    m = build_model("mlp")
    comp, got, want = _run(m, (torch.randn(64, 784),), dynamic=True)
    assert max_rel_err(got, want) < 1e-5
    plan = comp.compiled[0].engine.text
    assert plan.count("step gemm") == 2 and "step eltwise" not in plan      # bias+relu fused
    # the same plan serves another batch size (symbolic batch)
    x = torch.randn(7, 784)
    with torch.no_grad():
        got7 = comp.compiled[0].engine.run(7, x)[0]
        assert max_rel_err(got7, m(x)) < 1e-5


def test_resnet18_fuses_to_conv_steps():
    m = build_model("resnet18")
    comp, got, want = _run(m, (torch.randn(2, 3, 64, 64),))
    assert max_rel_err(got, want) < 1e-4
    plan = comp.compiled[0].engine.text
    assert plan.count("step conv") == 20 and plan.count("step maxpool") == 1
    assert plan.count("step eltwise") == 0 and plan.count("step nchw2nhwc") == 1   # only the input re-layout


def test_encoder_layer_dynamic_seq():
    m = build_model("encoder")
    comp, got, want = _run(m, (torch.randn(2, 16, 768),), dynamic=True)
    assert max_rel_err(got, want) < 1e-4
    plan = comp.compiled[0].engine.text
    assert plan.count("step softmax") == 1 and plan.count("step layernorm") == 2


def test_bert_two_layers():
    m = build_model("bert", n_layers=2)
    ids = torch.randint(0, 30522, (2, 16))
    mask = torch.ones(2, 16, dtype=torch.int64)
    mask[1, 10:] = 0
    comp, got, want = _run(m, (ids, mask))
    assert max_rel_err(got, want) < 1e-4


def test_resnet18_tensor_core_plan_pads_the_stem():
    # at a tensor-core precision the 3-channel stem is zero-padded to 4 channels (16 bytes)
    m = build_model("resnet18")
    comp, got, want = _run(m, (torch.randn(2, 3, 64, 64),), precision="tf32x3")
    assert max_rel_err(got, want) < 1e-4
    plan = comp.compiled[0].engine.text
    # ... and a filter row (7 taps x 4 channels, padded to 8 x 4) is the channel dim of a 1-wide kernel over the widened copy
    assert "prec:tf32x3" in plan and "w=b104@0[64,7,1,32;" in plan and "wide:3,70" in plan and "pad:3,0,3,0" in plan
    # weights are split into their tf32 high and low parts once, at load time
    assert plan.count(" w_lo=") == 20 and plan.count(" b_lo=") == 1 and plan.count("tf32lo") == 21


def _bert_bf16(monkeypatch, fuse, dynamic=False, seq=16):
    from oracle.models import round_to_bf16_
    monkeypatch.setenv("LLC_FUSE_ATTENTION", "1" if fuse else "0")
    ref = round_to_bf16_(build_model("bert", n_layers=2))
    ids = torch.randint(0, 30522, (2, seq))
    mask = torch.ones(2, seq, dtype=torch.int64)
    mask[1, seq - 5:] = 0
    with torch.no_grad():
        want = ref(ids, mask)
    comp = InterpreterCompiler(precision="auto")
    with torch.no_grad():
        got = compile_with(comp, build_model("bert", n_layers=2).to(torch.bfloat16), dynamic)(ids, mask)
    return comp.compiled[0].engine.text, got.float(), want


def test_bert_bf16_attention_becomes_one_step(monkeypatch):
    # batch_matmul -> scale -> mask -> softmax -> batch_matmul: one attention step per layer that reads the heads in
    # place from the projections' [B, S, H*D] outputs and writes [B, S, H, D] directly
    plan, got, want = _bert_bf16(monkeypatch, fuse=True)
    assert plan.count("step attention") == 2 and plan.count("step softmax") == 0
    # the query, key and value projections of a layer are one GEMM over weights stacked at load time (N = 3 x 768), and
    # the attention step reads its three operands as column ranges of that GEMM's output
    assert plan.count("step gemm") == 8 and plan.count("step eltwise") == 2 and plan.count("[1,1,768,2304;") == 2
    assert plan.count("init eltwise out=") >= 12 and " k=b" in plan and "@768[2,12,64,16;36864,64,1,2304]" in plan
    assert "scale:0.125" in plan and " mask=" in plan
    assert max_rel_err(got, want) < 2e-2


def test_bert_bf16_projections_kept_apart_are_the_same_function(monkeypatch):
    monkeypatch.setenv("LLC_FUSE_SIBLING_GEMMS", "0")
    plan, got, want = _bert_bf16(monkeypatch, fuse=True)
    assert plan.count("step gemm") == 12 and plan.count("2304") == 0
    assert max_rel_err(got, want) < 2e-2


def test_bert_bf16_unfused_attention_is_the_same_function(monkeypatch):
    plan, got, want = _bert_bf16(monkeypatch, fuse=False)
    assert plan.count("step attention") == 0 and plan.count("step softmax") == 2 and plan.count("step gemm") == 14   # query and key projections fuse; the value projection comes after the score GEMM
    assert max_rel_err(got, want) < 2e-2


def test_resnet18_stem_without_row_merging(monkeypatch):
    monkeypatch.setenv("LLC_MERGE_STEM_ROWS", "0")
    m = build_model("resnet18")
    comp, got, want = _run(m, (torch.randn(2, 3, 64, 64),), precision="tf32x3")
    assert max_rel_err(got, want) < 1e-4
    plan = comp.compiled[0].engine.text
    assert "[64,7,7,4;" in plan and "wide:" not in plan


class _Siblings(torch.nn.Module):
    """Linear layers over one activation in the forms the sibling-GEMM fusion has to tell apart."""

    def __init__(self, form):
        super().__init__()
        self.form = form
        self.a, self.b, self.c = (torch.nn.Linear(128, 64) for _ in range(3))
        self.wide = torch.nn.Linear(128, 128)
        self.register_buffer("mix", torch.linspace(-1, 1, 4 * 64).view(4, 64))

    def forward(self, x):
        if self.form == "three":                # two of them read through reshapes before the third is computed: those two fuse
            q, k, v = self.a(x), self.b(x), self.c(x)
            return (q.view(-1, 4, 16) * k.view(-1, 4, 16)).sum(-1) @ self.mix + v
        if self.form == "activation":           # the sums are absorbed as residual epilogues, so each GEMM has a reader of the one before: none fuses
            return self.a(x) + torch.relu(self.b(x)) + self.c(x)
        if self.form == "widths":               # a different width is not a sibling
            return self.a(x).sum(-1, keepdim=True) + self.wide(x)
        if self.form == "flat":                 # a reader that flattens rows and columns cannot be restated: no fusion
            return self.a(x).reshape(4, 128).abs(), self.b(x).abs()
        raise ValueError(self.form)


@pytest.mark.parametrize("form,gemms,fused", [("three", 3, 1), ("activation", 3, 0), ("widths", 2, 0), ("flat", 2, 0)])
def test_sibling_gemms_fuse_only_where_every_reader_can_follow(form, gemms, fused):
    torch.manual_seed(0)
    m = _Siblings(form)
    comp, got, want = _run(m, (torch.randn(8, 128),))
    for g, w in zip(got, want) if isinstance(want, tuple) else [(got, want)]:
        assert max_rel_err(g, w) < 1e-4
    plan = comp.compiled[0].engine.text
    assert plan.count("step gemm") == gemms, plan
    # a fused GEMM reads the stacked weights: a B operand of 2 or 3 x 64 columns with batch strides of its own
    n_fused = sum(1 for line in plan.splitlines() if line.startswith("step gemm") and (";16384,16384,1,128]" in line or ";24576,24576,1,128]" in line))
    assert n_fused == fused, plan


def test_sibling_gemms_that_are_graph_outputs_stay_apart():
    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = torch.nn.Linear(128, 64), torch.nn.Linear(128, 64)

        def forward(self, x):
            return self.a(x), self.b(x)

    torch.manual_seed(0)
    m = Two()
    comp, got, want = _run(m, (torch.randn(8, 128),))
    assert max_rel_err(got[0], want[0]) < 1e-4 and max_rel_err(got[1], want[1]) < 1e-4
