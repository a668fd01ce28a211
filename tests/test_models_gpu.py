"""End-to-end parity on the GPU: the benchmark models go through
torch.compile(backend=LLCompiler) -> importer -> llcompiler_.Compiler -> Execution, and the
result is compared with the CPU oracle (PyTorch CPU fp32 eager on the same seeded model and
inputs).  Tolerances are the ones the benchmark definition states: 1e-4 relative for fp32
paths, 2e-2 relative for bf16 paths (against the fp32 oracle on bf16-rounded parameters)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from helpers import compile_with  # noqa: E402
from llcompiler_b200.compiler import LLCompiler  # noqa: E402
from oracle.models import CONFIGS, assert_parity, build_model, max_rel_err, round_to_bf16_  # noqa: E402


def _gpu_run(model, inputs, dynamic=False, precision="auto", device_inputs=True):
    comp = LLCompiler(precision=precision)
    if device_inputs:
        model = copy.deepcopy(model).cuda()
    fn = compile_with(comp, model, dynamic)
    args = [i.cuda() if device_inputs else i for i in inputs]
    with torch.no_grad():
        out = fn(*args)
    torch.cuda.synchronize()
    return comp, fn, out


def test_mlp_symbolic_batch_device_and_host_tensors():
    m = build_model("mlp")
    x = CONFIGS["mlp"].make_inputs()[0]
    with torch.no_grad():
        want = m(x)
    comp, fn, out = _gpu_run(m, (x,), dynamic=True)
    assert out.is_cuda
    assert_parity(out, want, 1e-4, "mlp fp32")
    eng = comp.compiled[0].engine
    assert eng.executor.last_launch_count() == 2          # two fused GEMM launches, nothing else
    for b in (1, 7, 65, 1024):                             # same plan, other batch sizes
        xb = torch.randn(b, 784, generator=torch.Generator().manual_seed(b))
        with torch.no_grad():
            got = eng.run(b, xb.cuda())[0]
            assert max_rel_err(got, m(xb)) < 1e-4
    # host tensors in, host tensors out (the reference's calling convention)
    with torch.no_grad():
        got = eng.run(64, x)[0]
    assert not got.is_cuda and max_rel_err(got, want) < 1e-4


def test_resnet18_fp32():
    m = build_model("resnet18")
    x = CONFIGS["resnet18"].make_inputs(batch=8)[0]
    with torch.no_grad():
        want = m(x)
    comp, fn, out = _gpu_run(m, (x,))
    assert_parity(out, want, 1e-4, "resnet18 fp32")
    assert comp.compiled[0].engine.executor.last_launch_count() == 24


@pytest.mark.parametrize("seq", [128, 512])
def test_encoder_layer_symbolic_seq(seq):
    m = build_model("encoder")
    x = CONFIGS["encoder"].make_inputs(batch=8, seq=seq)[0]
    with torch.no_grad():
        want = m(x)
    comp, fn, out = _gpu_run(m, (x,), dynamic=True)
    assert_parity(out, want, 1e-4, f"encoder fp32 S={seq}")   # fp32 FMA path; the TF32 path states 2e-2


def test_resnet50_bf16():
    m = round_to_bf16_(build_model("resnet50"))
    x = CONFIGS["resnet50"].make_inputs(batch=4)[0].to(torch.bfloat16)
    with torch.no_grad():
        want = m(x.float())
    mb = build_model("resnet50").to(torch.bfloat16)
    comp, fn, out = _gpu_run(mb, (x,))
    assert out.dtype == torch.bfloat16
    assert_parity(out.float(), want, 2e-2, "resnet50 bf16")


def test_bert_bf16_two_layers_with_mask():
    m = round_to_bf16_(build_model("bert", n_layers=2))
    ids, mask = CONFIGS["bert"].make_inputs(batch=4, seq=384)
    mask = mask.clone()
    mask[1, 300:] = 0
    with torch.no_grad():
        want = m(ids, mask)
    mb = build_model("bert", n_layers=2).to(torch.bfloat16)
    comp, fn, out = _gpu_run(mb, (ids, mask))
    assert_parity(out.float(), want, 2e-2, "bert bf16, 2 layers, masked")


def test_bert_fp32_two_layers():
    m = build_model("bert", n_layers=2)
    ids, mask = CONFIGS["bert"].make_inputs(batch=2, seq=64)
    with torch.no_grad():
        want = m(ids, mask)
    comp, fn, out = _gpu_run(m, (ids, mask))
    assert_parity(out, want, 1e-4, "bert fp32, 2 layers")


def test_wrong_inputs_raise():
    m = build_model("mlp")
    x = torch.randn(4, 784)
    comp, fn, out = _gpu_run(m, (x,), dynamic=True)
    eng = comp.compiled[0].engine
    with pytest.raises(RuntimeError):
        eng.run(4, torch.randn(4, 783).cuda())             # wrong static extent
    with pytest.raises(RuntimeError):
        eng.run(5, torch.randn(4, 784).cuda())             # symbol value contradicts the tensor
    with pytest.raises(RuntimeError):
        eng.run(4, torch.randn(4, 784, dtype=torch.float64).cuda())
    assert max_rel_err(eng.run(4, x.cuda())[0], m(x)) < 1e-4   # the handle stays usable


def test_resnet18_fp32_on_tensor_cores_tf32x3():
    # three-pass TF32 keeps the fp32 configuration inside its 1e-4 tolerance on tensor cores
    m = build_model("resnet18")
    x = CONFIGS["resnet18"].make_inputs(batch=8)[0]
    with torch.no_grad():
        want = m(x)
    comp, fn, out = _gpu_run(m, (x,), precision="tf32x3")
    assert_parity(out, want, 1e-4, "resnet18 tf32x3")


@pytest.mark.parametrize("seq", [128, 512])
def test_encoder_layer_tf32(seq):
    m = build_model("encoder")
    x = CONFIGS["encoder"].make_inputs(batch=8, seq=seq)[0]
    with torch.no_grad():
        want = m(x)
    comp, fn, out = _gpu_run(m, (x,), dynamic=True, precision="tf32")
    assert_parity(out, want, 2e-2, f"encoder tf32 S={seq}")   # the tolerance stated for TF32 paths


def test_host_results_are_page_locked_and_never_aliased():
    m = build_model("mlp")
    x = torch.randn(16, 784)
    comp, fn, out = _gpu_run(m, (x,), dynamic=True)
    eng = comp.compiled[0].engine
    a = eng.run(16, x)[0]                       # host tensors in, host tensor out
    assert a.is_pinned() and not a.is_cuda
    keep = a.clone()
    b = eng.run(16, x * 2)[0]                   # `a` is still referenced: the engine must not hand its buffer out again
    assert b.data_ptr() != a.data_ptr() and torch.equal(a, keep)
    view = b[:4]
    ptr_b = b.data_ptr()
    del b                                       # a view keeps the storage alive: still no reuse
    c = eng.run(16, x * 3)[0]
    assert c.data_ptr() != ptr_b and torch.equal(view, eng.run(16, x * 2)[0][:4])
    ptr_a = a.data_ptr()
    del a, keep
    d = eng.run(16, x)[0]                       # nothing refers to the first buffer any more: it is reused
    assert d.data_ptr() in (ptr_a, ptr_b) or d.is_pinned()
    with torch.no_grad():
        assert max_rel_err(d, m(x)) < 1e-5


@pytest.mark.parametrize("name,batch,precision,bf16,tol", [("resnet18", 32, "tf32x3", False, 1e-4), ("resnet50", 256, "auto", True, 2e-2),
                                                            ("bert", 256, "auto", True, 2e-2)])
def test_full_size_batch_sharding_is_invisible(name, batch, precision, bf16, tol):
    # At the benchmark's own sizes the CPU oracle takes minutes, so the check is a property that holds at any size: every
    # sample is independent (inference-mode batch norm, per-sequence attention), so the full batch must equal its two halves
    # run separately - which is also what batch-sharding over GPUs relies on.  Tile widths and split-K differ between the
    # two batch sizes, so equality is to the configuration's tolerance, not bitwise.
    kw = {"n_layers": 12} if name == "bert" else {}
    m = build_model(name, **kw)
    if bf16:
        m = m.to(torch.bfloat16)
    inputs = CONFIGS[name].make_inputs(batch=batch) if name != "bert" else CONFIGS[name].make_inputs(batch=batch, seq=384)
    if bf16:
        inputs = [i.to(torch.bfloat16) if i.is_floating_point() else i for i in inputs]
    comp = LLCompiler(precision=precision)
    fn = compile_with(comp, copy.deepcopy(m).cuda(), False)         # static shapes: the half batch compiles to a plan of its own
    with torch.no_grad():
        full = fn(*[i.cuda() for i in inputs]).float()
        half = batch // 2
        parts = [fn(*[i[k * half:(k + 1) * half].cuda() for i in inputs]).float() for k in range(2)]
    torch.cuda.synchronize()
    assert full.shape[0] == batch and torch.isfinite(full).all()
    assert max_rel_err(torch.cat(parts), full) < tol
    comp.compiled[0].engine.status()
    # eight samples spread over the full batch (first, last, one in every eighth) against the CPU oracle: they were
    # computed with the tile plan of the full batch, which the small-batch tests above never see
    ref = round_to_bf16_(build_model(name, **kw)) if bf16 else build_model(name, **kw)
    pick = torch.tensor(sorted({0, batch - 1} | {(k * batch) // 8 + k for k in range(1, 7)}))
    with torch.no_grad():
        want = ref(*[(i[pick].float() if i.is_floating_point() else i[pick]) for i in inputs])
    lowp = None
    if bf16:        # PyTorch's own bf16 run of the same samples: the yardstick for what bf16 storage alone costs
        with torch.no_grad():
            lowp = copy.deepcopy(m).cuda()(*[i[pick].cuda() for i in inputs]).float().cpu()
    assert_parity(full[pick.cuda()].cpu(), want, tol, f"{name} full batch {batch}, samples {pick.tolist()}", lowp_eager=lowp)


def test_onnx_entry_on_the_gpu():
    import numpy as np
    from llcompiler_b200.importer import onnx_wire as W
    rng = np.random.default_rng(0)
    w1, b1 = (rng.standard_normal((512, 784)) * 0.05).astype(np.float32), rng.standard_normal(512).astype(np.float32)
    w2, b2 = (rng.standard_normal((10, 512)) * 0.05).astype(np.float32), rng.standard_normal(10).astype(np.float32)
    data = W.build_model([("Gemm", ["x", "w1", "b1"], ["h"], {"transB": 1}), ("Relu", ["h"], ["r"], {}), ("Gemm", ["r", "w2", "b2"], ["y"], {"transB": 1})],
                         {"w1": w1, "b1": b1, "w2": w2, "b2": b2}, [("x", [64, 784])], [("y", [64, 10])])
    fn = LLCompiler().compile_onnx(data)
    x = torch.randn(64, 784)
    t = torch.from_numpy
    want = torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(x, t(w1), t(b1))), t(w2), t(b2))
    assert max_rel_err(fn(x.cuda()).cpu(), want) < 1e-4
    # the same graph with a named batch extent: one plan, any batch
    data = W.build_model([("Gemm", ["x", "w1", "b1"], ["h"], {"transB": 1}), ("Relu", ["h"], ["r"], {}), ("Gemm", ["r", "w2", "b2"], ["y"], {"transB": 1})],
                         {"w1": w1, "b1": b1, "w2": w2, "b2": b2}, [("x", ["N", 784])], [("y", ["N", 10])])
    comp = LLCompiler()
    fn = comp.compile_onnx(data)
    for rows in (64, 3, 257):
        assert max_rel_err(fn(x[:rows].cuda() if rows <= 64 else x.repeat(5, 1)[:rows].cuda()).cpu(), (want if rows <= 64 else want.repeat(5, 1))[:rows]) < 1e-4
    assert len(comp.compiled) == 1


def test_empty_and_single_sample_batches_through_the_engine():
    # the symbolic batch may be 0 (an empty shard when a batch does not divide over the ranks) or 1
    m = build_model("mlp")
    comp, fn, out = _gpu_run(m, (torch.randn(8, 784),), dynamic=True)
    eng = comp.compiled[0].engine
    got0 = eng.run(0, torch.empty(0, 784).cuda())[0]
    assert tuple(got0.shape) == (0, 10)
    x1 = torch.randn(1, 784)
    with torch.no_grad():
        assert max_rel_err(eng.run(1, x1.cuda())[0], m(x1)) < 1e-4
    host0 = eng.run(0, torch.empty(0, 784))[0]            # host tensors too
    assert tuple(host0.shape) == (0, 10) and not host0.is_cuda


@pytest.mark.parametrize("name,precision,tol", [("mlp", "auto", 1e-4), ("encoder", "auto", 1e-4), ("resnet18", "tf32x3", 1e-4)])
def test_repeated_device_calls_replay_a_graph_with_identical_results(name, precision, tol):
    """A caller that keeps coming back with the same device pointers is served by one graph launch from its second
    call on; every replay has to give the bits of the first, step-by-step, run - also on a side stream, with
    other inputs in the same buffer, and after a call of another batch size in between."""
    m = build_model(name)
    dynamic = CONFIGS[name].dynamic
    inputs = CONFIGS[name].make_inputs(batch=8)
    with torch.no_grad():
        want = m(*inputs)
    comp, fn, first = _gpu_run(m, inputs, dynamic=dynamic, precision=precision)
    assert max_rel_err(first, want) < tol
    eng = comp.compiled[0].engine
    launches = eng.executor.last_launch_count()
    args = [i.cuda() for i in inputs]
    with torch.no_grad():
        for _ in range(8):                                # outputs are allocated per call: the addresses cycle
            out = fn(*args)
            assert eng.executor.last_launch_count() == launches
            assert torch.equal(out, first)
        if dynamic:                                       # another binding of the same plan in between
            other = fn(*[a[:4].contiguous() for a in args])
            assert max_rel_err(other, want[:4]) < tol
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(5):
                assert torch.equal(fn(*args), first)
        side.synchronize()
        # same buffers, new contents: a replay reads what is there now
        fresh = [torch.randn_like(a) if a.is_floating_point() else a for a in args]
        want2 = m(*[f.cpu() for f in fresh])
        first = None
        for a, f in zip(args, fresh):
            a.copy_(f)
        for _ in range(4):
            out2 = fn(*args)
        assert max_rel_err(out2, want2) < tol


def test_mlp_fp32_on_tensor_cores_tf32x3():
    m = build_model("mlp")
    for batch in (64, 1000):
        x = CONFIGS["mlp"].make_inputs(batch=batch)[0]
        with torch.no_grad():
            want = m(x)
        comp, fn, out = _gpu_run(m, (x,), dynamic=True, precision="tf32x3")
        assert max_rel_err(out, want) < 1e-4
        assert comp.compiled[0].engine.executor.last_launch_count() == 2


def test_out_of_range_embedding_ids_are_an_error_of_the_call():
    """The gather kernel writes zeros for an id outside its table and counts it; the executor reads that count
    wherever it waits for its results, so the call fails instead of returning a wrong batch, and the handle stays usable."""
    m = build_model("bert", n_layers=1)
    ids, mask = CONFIGS["bert"].make_inputs(batch=2, seq=64)
    with torch.no_grad():
        want = m(ids, mask)
    comp, fn, out = _gpu_run(m, (ids, mask))
    eng = comp.compiled[0].engine
    assert eng.status() == [0, 0, 0]
    bad = ids.clone()
    bad[1, 7] = 30522                                     # one past the last row of the table
    with pytest.raises(RuntimeError, match="embedding indices"):
        eng.run(bad, mask)                                # host tensors: the call waits and checks
    eng.run(bad.cuda(), mask.cuda())                      # device tensors: the call only enqueues ...
    with pytest.raises(RuntimeError, match="embedding indices"):
        eng.status()                                      # ... and the caller asks after its synchronisation
    assert eng.status() == [0, 0, 0]                      # reading clears
    assert_parity(eng.run(ids, mask)[0], want, 1e-4, "bert after a refused call")


def test_one_plan_on_two_devices_in_one_process():
    """The dynamic shared-memory opt-in of the tensor-core kernels is kept per device: a second executor on another GPU
    of the same process must launch them too, and the caller's current device must be left alone."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m = round_to_bf16_(build_model("bert", n_layers=1))
    ids, mask = CONFIGS["bert"].make_inputs(batch=2, seq=128)
    with torch.no_grad():
        want = m(ids, mask)
    mb = build_model("bert", n_layers=1).to(torch.bfloat16)
    outs = []
    for d in (0, 1):
        comp = LLCompiler(device=d)
        fn = compile_with(comp, copy.deepcopy(mb).to(f"cuda:{d}"), False)
        with torch.no_grad():
            outs.append(fn(ids.to(f"cuda:{d}"), mask.to(f"cuda:{d}")))
        torch.cuda.synchronize(d)
        comp.compiled[0].engine.status()
        assert torch.cuda.current_device() == 0
        assert_parity(outs[-1].float(), want, 2e-2, f"bert bf16 on cuda:{d}")
    assert torch.equal(outs[0].cpu(), outs[1].cpu())


def test_cached_plan_and_weight_pool_give_identical_results(tmp_path, monkeypatch):
    """Second compilation of the same model with the same weights: the plan comes from the cache (no import, no lowering)
    and the executor uploads the saved weight pool instead of reading the .npy files and running the load-time kernels
    (filter re-layout, folded batch norm, the low-order parts of the tf32x3 weights); the results are the same bits."""
    monkeypatch.setenv("LLC_CACHE_DIR", str(tmp_path))
    m = build_model("resnet18")
    x = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(1))
    outs, comps = [], []
    for _ in range(2):
        comp = LLCompiler(precision="tf32x3")
        with torch.no_grad():
            outs.append(compile_with(comp, copy.deepcopy(m).cuda(), False)(x.cuda()))
        torch.cuda.synchronize()
        comps.append(comp)
    first, second = (c.compiled[0].engine.executor for c in comps)
    assert comps[0].cache_hits == 0 and not first.loaded_from_pool()
    assert comps[1].cache_hits == 1 and second.loaded_from_pool()
    assert torch.equal(outs[0], outs[1])
    with torch.no_grad():
        assert_parity(outs[1], m(x), 1e-4, "resnet18 from the cache")


@pytest.mark.gpu
def test_pipelined_runner_returns_every_batch_in_order():
    """Five different batches through BatchShardedRunner.pipelined (two in flight, results copied back on a stream of
    their own) equal the same batches run one at a time."""
    from llcompiler_b200.executor import BatchShardedRunner
    model = build_model("mlp")
    comp = LLCompiler(device=0)
    torch._dynamo.reset()
    fn = torch.compile(model, backend=comp, dynamic=False, fullgraph=True)
    g = torch.Generator().manual_seed(7)
    batches = [(torch.randn(64, 784, generator=g).pin_memory(),) for _ in range(5)]
    with torch.no_grad():
        fn(batches[0][0])                       # host tensors, as the reference's engine takes them
    eng = comp.compiled[0].engine
    runner = BatchShardedRunner(lambda *a: eng.run(*a), device=torch.device("cuda", 0))
    want = [eng.run(b[0])[0].clone() for b in batches]
    got = [o.clone() for o in runner.pipelined(iter(batches), depth=2)]
    assert len(got) == 5 and all(not o.is_cuda for o in got)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    got3 = [o.clone() for o in runner.pipelined(iter(batches), depth=3)]
    assert all(torch.equal(a, b) for a, b in zip(got3, want))
    eng.status()
