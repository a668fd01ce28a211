"""The reference-order restatement (oracle/reference_order.py) against the plain eager oracle.

Both oracles must agree within the reference's own tolerance (rtol = atol = 1e-5,
llcompiler/test_models/utility.py:18-21) on the reference's op shapes and on the benchmark models;
the one place they are known to differ -- a max-pool window with only negative values, where the
reference's zero initial value shows -- is pinned here too, together with the check that no
benchmark model feeds a max-pool anything but a ReLU output."""
import pytest
import torch

from op_models import build_reference_shape_case
from oracle.models import CONFIGS, build_model
from oracle.reference_order import ReferenceOrder, batch_norm_inference, max_pool2d_zero_init, max_pools_follow_relu, softmax


@pytest.mark.parametrize("name", ["batch_norm_2d_inference", "batch_norm_1d_inference", "relu"])
def test_reference_order_agrees_with_eager_on_the_reference_op_shapes(name):
    model, inputs, exact = build_reference_shape_case(name)
    with torch.no_grad():
        want = model(*inputs)
        with ReferenceOrder():
            got = model(*inputs)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_batch_norm_order_and_epsilon_type():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3, 3, 224, 224, generator=g)
    mean, var = torch.randn(3, generator=g), torch.rand(3, generator=g) + 0.5
    scale, bias = torch.randn(3, generator=g), torch.randn(3, generator=g)
    want = torch.nn.functional.batch_norm(x, mean, var, scale, bias, False, 0.1, 1e-5)
    got = batch_norm_inference(x, mean, var, scale, bias, 1e-5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    # the written order, literally
    lit = ((x - mean[None, :, None, None]) * scale[None, :, None, None]) / torch.sqrt(var + torch.tensor(1e-5))[None, :, None, None] + bias[None, :, None, None]
    assert torch.equal(got, lit)


def test_softmax_chain():
    x = torch.randn(4, 12, 128, 128, generator=torch.Generator().manual_seed(4)) * 3
    assert torch.allclose(softmax(x, -1), torch.softmax(x, -1), rtol=1e-5, atol=1e-6)


def test_zero_initialised_max_pool_differs_only_on_all_negative_windows():
    x = torch.randn(2, 3, 32, 32, generator=torch.Generator().manual_seed(5))
    eager = torch.nn.functional.max_pool2d(x, 3, 2, 1)
    ref = max_pool2d_zero_init(x, 3, 2, 1)
    assert torch.equal(ref, eager.clamp_min(0))
    assert (eager < 0).any() and not torch.equal(ref, eager)          # raw activations: the zero initial value shows
    xr = torch.relu(x)
    assert torch.equal(max_pool2d_zero_init(xr, 3, 2, 1), torch.nn.functional.max_pool2d(xr, 3, 2, 1))   # after a ReLU it cannot


@pytest.mark.parametrize("name", ["resnet18", "resnet50"])
def test_max_pool_only_follows_relu_in_the_benchmark_models(name):
    assert max_pools_follow_relu(build_model(name)) == []


def test_the_check_itself_sees_a_pool_without_relu():
    m = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3), torch.nn.MaxPool2d(2))
    assert max_pools_follow_relu(m) != []


@pytest.mark.parametrize("name,kw,batch", [("resnet18", {}, 2), ("encoder", {"seq": 128}, 2), ("mlp", {}, 8)])
def test_models_in_reference_order_agree_with_eager(name, kw, batch):
    m = build_model(name)
    inputs = CONFIGS[name].make_inputs(batch=batch, **kw)
    with torch.no_grad():
        want = m(*inputs)
        with ReferenceOrder():
            got = m(*inputs)
    scale = float(want.abs().max())
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5 * max(scale, 1.0))
