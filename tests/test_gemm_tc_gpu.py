"""Tensor-core GEMM (tcgen05 + TMA) parity through the C ABI.  bf16 operands multiply exactly
and accumulate in fp32, so with fp32 output the result must agree with the fp32 CPU oracle on
the same bf16-rounded inputs to 1e-4 relative (any descriptor or swizzle mistake is O(1)).
fp32 operands: 5e-5 at precision tf32x3 (three-pass split; what remains is the tensor core's
truncating fp32 accumulation, which grows with K), 2e-3 at single-pass tf32.  After every
case the kernels' health word must read 0 (no bounded wait gave up)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

import gpu_ops as G  # noqa: E402
from llcompiler_b200 import _capi as C  # noqa: E402
from oracle.models import max_rel_err  # noqa: E402


@pytest.fixture(autouse=True)
def _small_problems_stay_on_the_tensor_cores(monkeypatch):
    # by default fp32 problems below 2^25 multiply-adds go to the FMA kernel; these tests are about the tensor-core one
    monkeypatch.setenv("LLC_TC_MIN_MACS_LOG2", "18")

DEV = "cuda"


def _rand(*shape, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g).to(dtype)


def _healthy():
    assert C.lib().llc_cuda_status() == 0


SHAPES = [(128, 128, 64), (64, 64, 64), (256, 256, 512), (300, 200, 136), (1024, 768, 768), (130, 70, 72),
          (98, 1000, 2048), (4096, 64, 576), (1, 512, 1024), (257, 129, 8)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_bf16_fp32_out(m, n, k):
    a, w = _rand(m, k, dtype=torch.bfloat16), _rand(n, k, dtype=torch.bfloat16, seed=1)
    bias, res = _rand(n, seed=2), _rand(m, n, seed=3)
    want = F.gelu(a.float() @ w.float().t() * 0.25 + bias + res)
    out = torch.full((1, 1, m, n), float("nan"), device=DEV)
    G.gemm(a.to(DEV)[None, None], w.to(DEV).t()[None, None], out, shift=bias.to(DEV), res=res.to(DEV)[None, None],
           alpha=0.25, act="gelu", prec="bf16")
    assert max_rel_err(out[0, 0], want) < 1e-4
    _healthy()


@pytest.mark.parametrize("m,n,k", [(256, 256, 512), (300, 200, 136), (130, 70, 72)])
def test_bf16_bf16_out_scale_relu(m, n, k):
    a, w = _rand(m, k, dtype=torch.bfloat16), _rand(n, k, dtype=torch.bfloat16, seed=1)
    scale, shift = _rand(n, seed=2).abs() + 0.5, _rand(n, seed=3)
    res = _rand(m, n, dtype=torch.bfloat16, seed=4)
    want = torch.relu(a.float() @ w.float().t() * scale + shift + res.float())
    out = torch.empty(1, 1, m, n, device=DEV, dtype=torch.bfloat16)
    G.gemm(a.to(DEV)[None, None], w.to(DEV).t()[None, None], out, scale=scale.to(DEV), shift=shift.to(DEV),
           res=res.to(DEV)[None, None], act="relu", prec="bf16")
    assert max_rel_err(out[0, 0].float(), want) < 2e-2
    _healthy()


@pytest.mark.parametrize("prec,tol", [("tf32x3", 5e-5), ("tf32", 2e-3)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (256, 256, 512), (300, 200, 136), (64, 512, 784), (1024, 768, 3072), (100, 10, 512)])
def test_fp32_on_tensor_cores(m, n, k, prec, tol):
    a, w, bias = _rand(m, k), _rand(n, k, seed=1), _rand(n, seed=2)
    want = torch.relu((a.double() @ w.double().t()).float() + bias)
    out = torch.full((1, 1, m, n), float("nan"), device=DEV)
    G.gemm(a.to(DEV)[None, None], w.to(DEV).t()[None, None], out, shift=bias.to(DEV), act="relu", prec=prec)
    assert max_rel_err(out[0, 0], want) < tol
    _healthy()


def test_bf16_batched_strided_heads_with_mask():
    Bn, S, H, D = 2, 384, 12, 64
    q, k = _rand(Bn, S, H * D, dtype=torch.bfloat16), _rand(Bn, S, H * D, dtype=torch.bfloat16, seed=1)
    mask = _rand(Bn, 1, 1, S, seed=2)
    qh, kh = q.float().view(Bn, S, H, D).permute(0, 2, 1, 3), k.float().view(Bn, S, H, D).permute(0, 2, 1, 3)
    want = qh @ kh.transpose(-1, -2) / 8.0 + mask
    Q = q.to(DEV).view(Bn, S, H, D).permute(0, 2, 1, 3)
    K = k.to(DEV).view(Bn, S, H, D).permute(0, 2, 3, 1)
    out = torch.full((Bn, H, S, S), float("nan"), device=DEV)
    G.gemm(Q, K, out, res=mask.to(DEV).expand(Bn, H, S, S), alpha=0.125, prec="bf16")
    assert max_rel_err(out, want) < 1e-4
    _healthy()


def test_bf16_shared_weights_across_batch():
    # B operand broadcast over the batch dims (stride 0)
    a, w = _rand(3, 2, 200, 128, dtype=torch.bfloat16), _rand(96, 128, dtype=torch.bfloat16, seed=1)
    want = a.float() @ w.float().t()
    out = torch.full((3, 2, 200, 96), float("nan"), device=DEV)
    G.gemm(a.to(DEV), w.to(DEV).t()[None, None].expand(3, 2, 128, 96), out, prec="bf16")
    assert max_rel_err(out, want) < 1e-4
    _healthy()


CONV_TC = [
    # n, c, h, w, f, k, stride, pad, dil   (ResNet layer shapes at a small batch, plus ragged ones)
    (4, 64, 56, 56, 64, 3, 1, 1, 1), (4, 64, 56, 56, 256, 1, 1, 0, 1), (4, 128, 28, 28, 256, 1, 2, 0, 1),
    (4, 256, 14, 14, 256, 3, 1, 1, 1), (2, 512, 7, 7, 512, 3, 1, 1, 1), (3, 64, 15, 13, 128, 3, 2, 1, 1),
    (1, 8, 9, 17, 24, 3, 1, 2, 2), (2, 16, 30, 30, 40, 5, 1, 2, 1), (2, 64, 112, 112, 64, 7, 2, 3, 1),
    # channel counts the im2col TMA load takes (128-byte K blocks inside one tap): dilation, stride with a remainder, asymmetric extents
    (1, 64, 9, 17, 32, 3, 1, 2, 2), (2, 32, 14, 14, 64, 3, 2, 1, 1), (5, 128, 10, 6, 72, 3, 1, 0, 1), (2, 64, 20, 11, 64, 5, 3, 2, 1),
]


def _conv_case(case, dtype, prec, tol):
    n, c, h, w, f, k, s, p, d = case
    x, wt = _rand(n, c, h, w, dtype=dtype), (_rand(f, c, k, k, seed=1) * 0.1).to(dtype)
    scale, shift = _rand(f, seed=2).abs() + 0.5, _rand(f, seed=3)
    y = F.conv2d(x.double(), wt.double(), None, s, p, d).float()
    res = _rand(*y.shape, dtype=dtype, seed=4)
    want = torch.relu(y * scale.view(1, -1, 1, 1) + shift.view(1, -1, 1, 1) + res.float())
    X = x.to(DEV).permute(0, 2, 3, 1).contiguous()
    W = wt.to(DEV).permute(0, 2, 3, 1).contiguous()
    R = res.to(DEV).permute(0, 2, 3, 1).contiguous()
    out = torch.full((n, y.shape[2], y.shape[3], f), float("nan"), device=DEV, dtype=torch.float32)
    G.conv2d(X, W, out, (s, s), (p, p), (d, d), scale=scale.to(DEV), shift=shift.to(DEV), res=R, act="relu", prec=prec)
    assert max_rel_err(out.permute(0, 3, 1, 2), want) < tol
    _healthy()


@pytest.mark.parametrize("case", CONV_TC)
def test_conv_bf16_tensor_cores(case):
    _conv_case(case, torch.bfloat16, "bf16", 1e-4)       # fp32 output: exact products, fp32 accumulation


@pytest.mark.parametrize("prec,tol", [("tf32x3", 5e-5), ("tf32", 2e-3)])
@pytest.mark.parametrize("case", CONV_TC)
def test_conv_fp32_on_tensor_cores(case, prec, tol):
    _conv_case(case, torch.float32, prec, tol)


@pytest.mark.parametrize("prec,dtype,tol", [("bf16", torch.bfloat16, 1e-4), ("tf32x3", torch.float32, 5e-5), ("tf32", torch.float32, 2e-3)])
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 128, 512), (300, 200, 136), (384, 64, 384), (1000, 72, 264)])
def test_b_operand_stored_k_by_n(m, n, k, prec, dtype, tol):
    # B given as [K, N] row-major (unit stride along n): the MN-major tensor-core operand
    a, b = _rand(m, k, dtype=dtype), _rand(k, n, dtype=dtype, seed=1)
    want = (a.double() @ b.double()).float()
    out = torch.full((1, 1, m, n), float("nan"), device=DEV)
    G.gemm(a.to(DEV)[None, None], b.to(DEV)[None, None], out, prec=prec)
    assert max_rel_err(out[0, 0], want) < tol
    _healthy()


def test_bf16_attention_pv_strided_heads():
    # P [B,H,S,S] times V read in place from [B,S,H*D] storage (unit stride along the head dim)
    Bn, S, H, D = 2, 384, 12, 64
    pmat = torch.softmax(_rand(Bn, H, S, S), -1).to(torch.bfloat16)
    v = _rand(Bn, S, H * D, dtype=torch.bfloat16, seed=3)
    want = pmat.float() @ v.float().view(Bn, S, H, D).permute(0, 2, 1, 3)
    out = torch.full((Bn, H, S, D), float("nan"), device=DEV)
    G.gemm(pmat.to(DEV), v.to(DEV).view(Bn, S, H, D).permute(0, 2, 1, 3), out, prec="bf16")
    assert max_rel_err(out, want) < 1e-4
    _healthy()


def _tf32_lo(t):
    return t - (t.contiguous().view(torch.int32) & -8192).view(torch.float32)


def test_tf32x3_presplit_weight_operand():
    # the low-order part of a constant B (and of convolution weights) may be handed in instead of being derived from
    # every tile: same result to the last bit (the kernel computes the same values itself otherwise)
    m, n, k = 300, 200, 520
    a, w = _rand(m, k).to(DEV), _rand(n, k, seed=1).to(DEV)
    o1 = torch.empty(1, 1, m, n, device=DEV); o2 = torch.empty_like(o1)
    G.gemm(a[None, None], w.t()[None, None], o1, prec="tf32x3")
    G.gemm(a[None, None], w.t()[None, None], o2, prec="tf32x3", b_lo=_tf32_lo(w).t()[None, None])
    assert torch.equal(o1, o2)
    want = (a.double() @ w.double().t()).float()
    assert max_rel_err(o2[0, 0], want) < 5e-5
    x = _rand(2, 30, 30, 64).to(DEV); wt = (_rand(72, 3, 3, 64, seed=1) * 0.1).to(DEV)
    c1 = torch.empty(2, 30, 30, 72, device=DEV); c2 = torch.empty_like(c1)
    G.conv2d(x, wt, c1, (1, 1), (1, 1), prec="tf32x3")
    G.conv2d(x, wt, c2, (1, 1), (1, 1), prec="tf32x3", w_lo=_tf32_lo(wt))
    assert torch.equal(c1, c2)
    _healthy()


@pytest.mark.parametrize("dtype,prec,c_pad,tol", [(torch.float32, "tf32x3", 4, 5e-5), (torch.float32, "tf32", 4, 2e-3), (torch.bfloat16, "bf16", 8, 1e-4)])
@pytest.mark.parametrize("n,h,w,f,k,s,pad", [(4, 224, 224, 64, 7, 2, 3), (2, 37, 29, 32, 5, 1, 2), (3, 16, 40, 24, 3, 2, 0)])
def test_stem_rows_as_channels_over_a_widened_copy(dtype, prec, c_pad, tol, n, h, w, f, k, s, pad):
    # 3-channel NCHW input -> channel-last copy with zero halo columns; the convolution then reads eight pixels (one filter
    # row, zero-padded to eight taps) as the channels of a kernel one pixel wide, through an overlapping strided view
    x = _rand(n, 3, h, w, dtype=dtype)
    wt = (_rand(f, 3, k, k, seed=1) * 0.1).to(dtype)
    shift = _rand(f, seed=2)
    want = torch.relu(F.conv2d(x.double(), wt.double(), None, s, pad).float() + shift.view(1, -1, 1, 1))
    oh, ow = want.shape[2], want.shape[3]
    w_total = max(pad + w, (ow - 1) * s + 8)
    wide = torch.full((n, h, w_total, c_pad), float("nan"), device=DEV, dtype=dtype)
    G.nchw_to_nhwc_wide(x.to(DEV), wide, c_pad, pad, w_total)
    ref_wide = torch.zeros(n, h, w_total, c_pad, dtype=dtype)
    ref_wide[:, :, pad: pad + w, :3] = x.permute(0, 2, 3, 1)
    assert torch.equal(wide.cpu(), ref_wide)                       # a copy: bit-exact
    wm = torch.zeros(f, k, 8, c_pad, dtype=dtype)
    wm[:, :, :k, :3] = wt.permute(0, 2, 3, 1)
    wm = wm.reshape(f, k, 1, 8 * c_pad).contiguous().to(DEV)
    out = torch.full((n, oh, ow, f), float("nan"), device=DEV, dtype=torch.float32)
    merged_w = (ow - 1) * s + 1
    G.conv2d(wide, wm, out, (s, s), (pad, 0), shift=shift.to(DEV), act="relu", prec=prec,
             x_strides=(h * w_total * c_pad, w_total * c_pad, c_pad), x_shape=(n, h, merged_w, 8 * c_pad))
    assert max_rel_err(out.permute(0, 3, 1, 2), want) < tol
    _healthy()


@pytest.mark.parametrize("dtype,prec,tol", [(torch.bfloat16, "bf16", 1e-4), (torch.float32, "tf32x3", 5e-5), (torch.float32, "tf32", 2e-3)])
def test_split_k_meets_in_the_workspace(dtype, prec, tol, monkeypatch):
    # few output tiles and a long K loop: with a workspace the K loop is cut into slices that run on otherwise idle SMs
    # (forced here; left to itself the library splits only where a slice stays long enough to pay for the meeting)
    monkeypatch.setenv("LLC_TC_SPLITK", "2")
    ws = torch.zeros(16 << 20, dtype=torch.uint8, device=DEV)
    m, n, k = 300, 256, 4096
    a, w = _rand(m, k, dtype=dtype).to(DEV), _rand(n, k, seed=1, dtype=dtype).to(DEV)
    shift = _rand(n, seed=2).to(DEV)
    res = _rand(m, n, seed=3).to(DEV)
    want = torch.relu((a.double() @ w.double().t()).float().cpu() + shift.cpu() + res.cpu())
    for _ in range(2):                                  # twice: the counters must be back at zero after a launch
        out = torch.full((1, 1, m, n), float("nan"), device=DEV)
        G.gemm(a[None, None], w.t()[None, None], out, shift=shift, res=res[None, None], act="relu", prec=prec, workspace=ws)
        assert max_rel_err(out[0, 0], want) < tol
    assert int(ws[:4096].max()) == 0
    # ResNet layer4 at a small batch: 13 x 4 tiles of 128 x 128, 144 K blocks
    x = _rand(32, 7, 7, 512, dtype=dtype).to(DEV); wt = (_rand(512, 3, 3, 512, seed=1) * 0.05).to(dtype).to(DEV)
    y = F.conv2d(x.permute(0, 3, 1, 2).double().cpu(), wt.permute(0, 3, 1, 2).double().cpu(), None, 1, 1).float()
    out = torch.full((32, 7, 7, 512), float("nan"), device=DEV)
    G.conv2d(x, wt, out, (1, 1), (1, 1), prec=prec, workspace=ws)
    assert max_rel_err(out.permute(0, 3, 1, 2), y) < tol
    assert int(ws[:4096].max()) == 0
    _healthy()


def test_small_fp32_problems_take_the_fma_kernel_by_default(monkeypatch):
    """Below 2^25 multiply-adds the tensor-core kernel's fixed cost loses: the call is served with plain fp32 FMAs, so its
    result carries no TF32 rounding at all, whatever precision was asked for."""
    monkeypatch.delenv("LLC_TC_MIN_MACS_LOG2")
    torch.manual_seed(0)
    a, b = torch.randn(1, 1, 32, 512, device="cuda"), torch.randn(1, 1, 1000, 512, device="cuda")
    want = (a.double() @ b.double().transpose(2, 3)).float()
    out = torch.empty(1, 1, 32, 1000, device="cuda")
    G.gemm(a, b.transpose(2, 3), out, prec="tf32")
    torch.cuda.synchronize()
    assert max_rel_err(out, want) < 2e-6                  # a single-pass TF32 product of K=512 is off by about 1e-4
    monkeypatch.setenv("LLC_TC_MIN_MACS_LOG2", "18")
    G.gemm(a, b.transpose(2, 3), out, prec="tf32")
    torch.cuda.synchronize()
    assert 2e-6 < max_rel_err(out, want) < 2e-3


@pytest.mark.parametrize("prec,in_dtype", [("tf32", torch.float32), ("bf16", torch.bfloat16)])
def test_fp32_output_gelu_epilogue_is_erf_gelu_to_1e6(prec, in_dtype):
    """With fp32 output the tensor-core epilogue computes GELU with a polynomial erf (one exp, one reciprocal, five
    FMAs).  The activation is isolated here: the same GEMM runs once without and once with the activation, and the
    activated result is compared with the erf GELU (float64) of the kernel's own un-activated result, so that what is
    measured is the activation's error alone: 1e-6 relative to the largest value, and 2e-6 absolute on every element."""
    m, n, k = 512, 384, 256
    a, w = (_rand(m, k) * 0.25).to(in_dtype), _rand(n, k, seed=1).to(in_dtype)
    bias = _rand(n, seed=2)
    A, B = a.to(DEV)[None, None], w.to(DEV).t()[None, None]
    pre = torch.empty(1, 1, m, n, device=DEV)
    act = torch.empty(1, 1, m, n, device=DEV)
    G.gemm(A, B, pre, shift=bias.to(DEV), prec=prec)
    G.gemm(A, B, act, shift=bias.to(DEV), act="gelu", prec=prec)
    torch.cuda.synchronize()
    x = pre[0, 0].double().cpu()
    want = 0.5 * x * (1.0 + torch.erf(x / 2.0 ** 0.5))
    assert x.abs().max() > 4                              # both tails of the activation are exercised
    assert max_rel_err(act[0, 0], want) < 1e-6
    assert float((act[0, 0].double().cpu() - want).abs().max()) < 2e-6
    _healthy()
