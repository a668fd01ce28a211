"""Kernel-level parity on the GPU: every kernel family is called through the C ABI
(include/llc_cuda.h) and compared with the CPU oracle (PyTorch CPU fp32 on the same seeded
inputs).  Tolerances: bit-exact for copies, gathers, max pooling and ReLU-only paths; 1e-5
relative (the reference's own allclose tolerance, llcompiler/test_models/utility.py:18-21)
for fp32 arithmetic; 2e-2 relative for bf16 storage.  Shapes cover the reference's op tests
(test/python/ops/*.py) plus ragged tails, unit extents and strided/batched operands."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

import gpu_ops as G  # noqa: E402
from oracle.models import max_rel_err  # noqa: E402

DEV = "cuda"


def _rand(*shape, dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("m,n,k", [(64, 512, 784), (64, 10, 512), (1, 1, 1), (7, 5, 3), (129, 65, 33), (3, 3, 3),
                                   (10, 100, 1000), (256, 256, 256), (1000, 1000, 20), (130, 260, 4)])
@pytest.mark.parametrize("b_kmajor", [True, False])
def test_gemm_fp32(m, n, k, b_kmajor):
    a = _rand(m, k)
    w = _rand(n, k, seed=1) if b_kmajor else _rand(k, n, seed=1)
    bias = _rand(n, seed=2)
    res = _rand(m, n, seed=3)
    want = torch.relu(a @ (w.t() if b_kmajor else w) * 0.5 + bias + res)
    A = a.to(DEV)[None, None]
    W = w.to(DEV)
    B = (W.t() if b_kmajor else W)[None, None]
    out = torch.empty(1, 1, m, n, device=DEV)
    G.gemm(A, B, out, shift=bias.to(DEV), res=res.to(DEV)[None, None], alpha=0.5, act="relu")
    assert max_rel_err(out[0, 0], want) < 1e-5


def test_gemm_linear_k100000():
    # the reference's Linear op test runs K = 100000 (test/python/ops/linear.py)
    a, w = _rand(10, 100000), _rand(10, 100000, seed=1)
    out = torch.empty(1, 1, 10, 10, device=DEV)
    G.gemm(a.to(DEV)[None, None], w.to(DEV).t()[None, None], out)
    assert max_rel_err(out[0, 0], (a.double() @ w.double().t()).float()) < 1e-5


def test_gemm_batched_strided_heads():
    # attention-style operands: [B,S,H,D] storage read as [B,H,S,D] without a copy
    Bn, S, H, D = 2, 48, 12, 64
    q, k = _rand(Bn, S, H * D), _rand(Bn, S, H * D, seed=1)
    mask = _rand(Bn, 1, 1, S, seed=2)
    qh, kh = q.view(Bn, S, H, D).permute(0, 2, 1, 3), k.view(Bn, S, H, D).permute(0, 2, 1, 3)
    want = qh @ kh.transpose(-1, -2) / 8.0 + mask
    Q = q.to(DEV).view(Bn, S, H, D).permute(0, 2, 1, 3)
    K = k.to(DEV).view(Bn, S, H, D).permute(0, 2, 3, 1)         # [B,H,D,S]: k stride 1
    out = torch.empty(Bn, H, S, S, device=DEV)
    G.gemm(Q, K, out, res=mask.to(DEV).expand(Bn, H, S, S), alpha=0.125)
    assert max_rel_err(out, want) < 1e-5
    # P @ V with V read n-major
    p, v = torch.softmax(want, -1), _rand(Bn, S, H * D, seed=3)
    vh = v.view(Bn, S, H, D).permute(0, 2, 1, 3)
    out2 = torch.empty(Bn, H, S, D, device=DEV)
    G.gemm(p.to(DEV), v.to(DEV).view(Bn, S, H, D).permute(0, 2, 1, 3), out2)
    assert max_rel_err(out2, p @ vh) < 1e-5


@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (100, 72, 40), (5, 3, 7)])
def test_gemm_bf16(m, n, k):
    a, w, bias = _rand(m, k, dtype=torch.bfloat16), _rand(n, k, dtype=torch.bfloat16, seed=1), _rand(n, seed=2)
    want = F.gelu(a.float() @ w.float().t() + bias)
    out = torch.empty(1, 1, m, n, device=DEV, dtype=torch.bfloat16)
    G.gemm(a.to(DEV)[None, None], w.to(DEV).t()[None, None], out, shift=bias.to(DEV), act="gelu", prec="bf16")
    assert max_rel_err(out[0, 0].float(), want) < 2e-2


CONV_CASES = [
    # n, c, h, w, f, k, stride, pad, dil
    (3, 3, 32, 32, 3, 5, 1, 2, 1),       # the reference's conv op test (5x5, pad 2, 3->3), smaller image
    (2, 3, 37, 41, 64, 7, 2, 3, 1),      # ResNet stem shape family, ragged image
    (2, 64, 14, 14, 64, 3, 1, 1, 1),
    (2, 64, 15, 13, 128, 3, 2, 1, 1),
    (2, 64, 14, 14, 128, 1, 2, 0, 1),    # 1x1 stride-2 downsample
    (1, 8, 9, 17, 12, 3, 1, 2, 2),       # dilation
    (1, 4, 1, 1, 4, 1, 1, 0, 1),
    (2, 20, 10, 10, 6, 3, 1, 1, 1),      # channels not a multiple of 16
]


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2d(case, dtype):
    n, c, h, w, f, k, s, p, d = case
    x, wt = _rand(n, c, h, w, dtype=dtype), (_rand(f, c, k, k, seed=1) * 0.2).to(dtype)
    scale, shift = _rand(f, seed=2).abs() + 0.5, _rand(f, seed=3)
    y = F.conv2d(x.float(), wt.float(), None, s, p, d)
    res = _rand(*y.shape, dtype=dtype, seed=4)
    want = torch.relu(y * scale.view(1, -1, 1, 1) + shift.view(1, -1, 1, 1) + res.float())
    X = x.to(DEV).permute(0, 2, 3, 1).contiguous()
    W = wt.to(DEV).permute(0, 2, 3, 1).contiguous()
    R = res.to(DEV).permute(0, 2, 3, 1).contiguous()
    out = torch.empty(n, y.shape[2], y.shape[3], f, device=DEV, dtype=dtype)
    G.conv2d(X, W, out, (s, s), (p, p), (d, d), scale=scale.to(DEV), shift=shift.to(DEV), res=R, act="relu",
             prec="fp32" if dtype == torch.float32 else "bf16")
    got = out.permute(0, 3, 1, 2).float()
    assert max_rel_err(got, want) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("shape,k,s,p,d", [((2, 64, 112, 112), 3, 2, 1, 1), ((3, 3, 30, 30), 5, 1, 2, 2),
                                           ((2, 7, 9, 17), 3, 2, 1, 1), ((1, 4, 1, 1), 1, 1, 0, 1),
                                           ((2, 16, 9, 17), 3, 2, 1, 1), ((1, 8, 2, 2), 3, 2, 1, 1), ((2, 24, 10, 12), 3, 2, 0, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_maxpool_bit_exact(shape, k, s, p, d, dtype):
    x = _rand(*shape, dtype=dtype)
    want = F.max_pool2d(x.float(), k, s, p, d).to(dtype)
    X = x.to(DEV).permute(0, 2, 3, 1).contiguous()
    out = torch.empty(shape[0], want.shape[2], want.shape[3], shape[1], device=DEV, dtype=dtype)
    G.maxpool2d(X, out, (k, k), (s, s), (p, p), (d, d))
    assert torch.equal(out.permute(0, 3, 1, 2).cpu(), want)


@pytest.mark.parametrize("outer,r,inner", [(64, 49, 512), (1536, 49, 1), (3, 1000, 1), (1, 1, 1), (5, 7, 3)])
@pytest.mark.parametrize("op", ["sum", "max", "min", "mean"])
def test_reduce(outer, r, inner, op):
    x = _rand(outer, r, inner)
    want = {"sum": x.sum(1), "max": x.amax(1), "min": x.amin(1), "mean": x.mean(1)}[op]
    out = torch.empty(outer, inner, device=DEV)
    G.reduce(x.to(DEV), out, op)
    if op in ("max", "min"):
        assert torch.equal(out.cpu(), want)
    else:
        assert max_rel_err(out, want) < 1e-5


@pytest.mark.parametrize("rows,length", [(96 * 128, 128), (96 * 8, 512), (17, 384), (5, 1000), (3, 7), (2, 2048), (1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax(rows, length, dtype):
    x = (_rand(rows, length) * 3).to(dtype)
    want = torch.softmax(x.float(), -1)
    out = torch.empty(rows, length, device=DEV, dtype=dtype)
    G.softmax(x.to(DEV), out)
    assert max_rel_err(out.float(), want) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert torch.allclose(out.float().sum(-1).cpu(), torch.ones(rows), atol=2e-2 if dtype == torch.bfloat16 else 1e-5)


# (20011 rows: more rows than resident warps, so every warp walks several rows; 2048 and 1024: the widest register-held rows)
@pytest.mark.parametrize("rows,d", [(1024, 768), (33, 768), (7, 100), (3, 3000), (1, 4), (20011, 768), (300, 2048), (64, 1024), (50, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm(rows, d, dtype):
    x, g, b = (_rand(rows, d) * 2 + 0.3).to(dtype), (_rand(d, seed=1) + 1).to(dtype), _rand(d, seed=2).to(dtype)
    want = F.layer_norm(x.float(), (d,), g.float(), b.float(), 1e-5)
    out = torch.empty(rows, d, device=DEV, dtype=dtype)
    G.layernorm(x.to(DEV), g.to(DEV), b.to(DEV), out, 1e-5)
    assert max_rel_err(out.float(), want) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_gather_bit_exact_and_bad_ids():
    table = _rand(1000, 768)
    ids = torch.randint(0, 1000, (4 * 33,), generator=torch.Generator().manual_seed(3))
    out = torch.empty(ids.numel(), 768, device=DEV)
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    G.gather(table.to(DEV), ids.to(DEV), out, bad)
    assert torch.equal(out.cpu(), table[ids]) and int(bad.item()) == 0
    ids2 = ids.clone()
    ids2[5], ids2[9] = -1, 1000
    G.gather(table.to(DEV), ids2.to(DEV), out, bad)
    assert int(bad.item()) == 2 and torch.count_nonzero(out[5]).item() == 0
    tb = table.to(torch.bfloat16)
    outb = torch.empty(ids.numel(), 768, device=DEV, dtype=torch.bfloat16)
    G.gather(tb.to(DEV), ids.to(DEV), outb)
    assert torch.equal(outb.cpu(), tb[ids])


def test_eltwise_programs():
    x, y = _rand(3, 3, 24, 20), _rand(3, 3, 24, 20, seed=1)
    X, Y = x.to(DEV), y.to(DEV)
    out = torch.empty_like(X)
    for prog, want in [("ld0;ld1;add,0,1", x + y), ("ld0;ld1;sub,0,1", x - y), ("ld0;ld1;mul,0,1", x * y),
                       ("ld0;ld1;div,0,1", x / y), ("ld0;abs,0", x.abs()), ("ld0;abs,0;sqrt,1", x.abs().sqrt()),
                       ("ld0;relu,0", torch.relu(x)), ("ld0;ld1;ge,0,1;ld0;ld1;where,2,3,4", torch.where(x >= y, x, y)),
                       ("ld0;#3;add,0,1;ld0;add,2,3", x + 3 + x), ("ld0;exp,0", x.exp()), ("ld0;gelu,0", F.gelu(x))]:
        G.eltwise(out, [X, Y], prog)
        exact = prog.split(";")[-1].split(",")[0] in ("add", "sub", "mul", "abs", "relu", "where")
        err = max_rel_err(out, want)
        assert (err == 0.0) if exact else (err < 1e-5), (prog, err)


def test_eltwise_broadcast_and_layout_copy():
    # per-channel broadcast (batch-norm form) on NCHW data and an NCHW -> NHWC re-layout: copies are bit-exact
    x, s = _rand(2, 5, 7, 9), _rand(5, seed=1)
    X, S = x.to(DEV), s.to(DEV)
    out = torch.empty_like(X)
    G.eltwise(out, [X, S.view(1, 5, 1, 1).expand(2, 5, 7, 9)], "ld0;ld1;mul,0,1")
    assert torch.equal(out.cpu(), x * s.view(1, 5, 1, 1))
    nhwc = torch.empty(2, 7, 9, 5, device=DEV)
    G.eltwise(nhwc.permute(0, 3, 1, 2), [X], "ld0")
    assert torch.equal(nhwc.cpu(), x.permute(0, 2, 3, 1).contiguous())
    big = _rand(4, 8, 16, 32)
    nhwc2 = torch.empty(4, 16, 32, 8, device=DEV, dtype=torch.bfloat16)
    G.eltwise(nhwc2.permute(0, 3, 1, 2), [big.to(DEV)], "ld0")
    assert torch.equal(nhwc2.cpu(), big.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous())
    ids = torch.arange(24).view(2, 12)
    f = torch.empty(2, 12, device=DEV)
    G.eltwise(f, [ids.to(DEV)], "#1;ld0;cast,1;sub,0,2")
    assert torch.equal(f.cpu(), 1.0 - ids.float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_eltwise_short_programs_on_wide_rows(dtype):
    """Short programs on rows of whole 16-byte vectors take the eight-elements-per-thread kernel: a row broadcast over the
    batch (the embedding sum), a residual add with a strided operand, a cast, a copy between layouts whose inner dim stays
    dense, a scalar broadcast along the rows, a where.  Bit-exact against the same arithmetic in torch."""
    x = _rand(6, 40, 64).to(dtype)
    row = _rand(40, 64, seed=1).to(dtype)
    X, R = x.to(DEV), row.to(DEV)
    out = torch.empty_like(X)
    G.eltwise(out, [X, R.unsqueeze(0).expand(6, 40, 64)], "ld0;ld1;add,0,1")
    assert torch.equal(out.cpu(), (x.float() + row.float()).to(dtype))
    big = _rand(6, 40, 128, seed=2).to(dtype).to(DEV)
    G.eltwise(out, [X, big[:, :, 64:]], "ld0;ld1;sub,0,1")                 # second operand: every other 64-wide half
    assert torch.equal(out.cpu(), (x.float() - big[:, :, 64:].float().cpu()).to(dtype))
    other = torch.bfloat16 if dtype == torch.float32 else torch.float32
    cast = torch.empty(6, 40, 64, device=DEV, dtype=other)
    G.eltwise(cast, [X], "ld0")
    assert torch.equal(cast.cpu(), x.to(other))
    swapped = torch.empty(40, 6, 64, device=DEV, dtype=dtype)
    G.eltwise(swapped.permute(1, 0, 2), [X], "ld0;relu,0")
    assert torch.equal(swapped.cpu(), torch.relu(x).permute(1, 0, 2).contiguous())
    col = _rand(6, 40, 1, seed=3).to(dtype).to(DEV)
    G.eltwise(out, [X, col.expand(6, 40, 64)], "ld0;ld1;mul,0,1")
    assert torch.equal(out.cpu(), (x.float() * col.float().cpu()).to(dtype))
    G.eltwise(out, [X, R.unsqueeze(0).expand(6, 40, 64)], "ld0;ld1;gt,0,1;where,2,0,1")
    assert torch.equal(out.cpu(), torch.where(x > row, x, row.expand(6, 40, 64)))


def test_argument_errors_are_reported():
    from llcompiler_b200 import _capi as C
    a = torch.empty(1, 1, 4, 4, device=DEV)
    with pytest.raises(C.LlcError):
        G.eltwise(a, [a], "ld0;frobnicate,0")
    with pytest.raises(C.LlcError):
        G.eltwise(a, [a], "ld3")
    bt = torch.empty(1, 1, 4, 4, device=DEV)[:, :, ::2, ::2]      # neither stride is 1
    with pytest.raises(C.LlcError):
        G.gemm(a[:, :, :2, :2], bt, torch.empty(1, 1, 2, 2, device=DEV))


@pytest.mark.parametrize("m,n,k", [(64, 512, 784), (64, 10, 512), (7, 100, 4096), (130, 70, 1000)])
def test_gemm_fp32_split_k_matches_single_pass(m, n, k):
    # few output tiles and a long K: the FMA kernel spreads K over idle SMs when given scratch
    a, w, bias = _rand(m, k), _rand(n, k, seed=1), _rand(n, seed=2)
    want = torch.relu((a.double() @ w.double().t()).float() + bias)
    ws = torch.zeros(16 << 20, dtype=torch.uint8, device=DEV)
    A, B = a.to(DEV)[None, None], w.to(DEV).t()[None, None]
    for _ in range(2):                                   # twice: the tile counters must be back at zero
        out = torch.full((1, 1, m, n), float("nan"), device=DEV)
        G.gemm(A, B, out, shift=bias.to(DEV), act="relu", workspace=ws)
        assert max_rel_err(out[0, 0], want) < 1e-5
    assert int(ws[:4096].sum().item()) == 0
    ref = torch.empty(1, 1, m, n, device=DEV)
    G.gemm(A, B, ref, shift=bias.to(DEV), act="relu")
    assert max_rel_err(out[0, 0], ref[0, 0].cpu()) < 1e-5


@pytest.mark.parametrize("n,c,h,w,cp", [(2, 3, 37, 41, 4), (2, 3, 37, 41, 8), (3, 3, 16, 16, 3), (2, 64, 14, 14, 64), (1, 70, 9, 5, 72)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_nchw_to_nhwc_bit_exact_with_zero_padding(n, c, h, w, cp, dtype):
    import ctypes
    from ctypes import c_void_p
    from llcompiler_b200 import _capi as C
    x = _rand(n, c, h, w, dtype=dtype)
    out = torch.full((n, h, w, cp), float("nan"), device=DEV, dtype=dtype)
    f = C.lib().llc_cuda_nchw_to_nhwc
    f.argtypes = [c_void_p, c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, c_void_p]
    X = x.to(DEV)
    C.check(f(X.data_ptr(), out.data_ptr(), 4 if dtype == torch.float32 else 8, n, c, h * w, cp, torch.cuda.current_stream().cuda_stream))
    want = torch.zeros(n, h, w, cp, dtype=dtype)
    want[..., :c] = x.permute(0, 2, 3, 1)
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("n,c,h,w,left,total", [(2, 3, 12, 224, 3, 232), (3, 3, 9, 40, 3, 46), (2, 3, 7, 41, 3, 48), (1, 2, 5, 16, 0, 16), (5, 3, 3, 8, 2, 11)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_nchw_to_nhwc_wide_bit_exact_with_zero_columns(n, c, h, w, left, total, dtype):
    # rows that start on a 4-element boundary take the vector kernel, the others (w = 41) the row kernel
    cp = 4 if dtype == torch.float32 else 8
    x = _rand(n, c, h, w, dtype=dtype)
    out = torch.full((n, h, total, cp), float("nan"), device=DEV, dtype=dtype)
    G.nchw_to_nhwc_wide(x.to(DEV), out, cp, left, total)
    want = torch.zeros(n, h, total, cp, dtype=dtype)
    want[:, :, left:left + w, :c] = x.permute(0, 2, 3, 1)
    assert torch.equal(out.cpu(), want)


def test_empty_problems_launch_nothing_and_succeed():
    # extents of zero (an empty batch) are legal everywhere: the entry points return 0 without touching memory
    f32, bf = torch.float32, torch.bfloat16
    e = lambda *s, dtype=f32: torch.empty(*s, device=DEV, dtype=dtype)
    G.gemm(e(1, 1, 0, 64), e(1, 1, 64, 32), e(1, 1, 0, 32))
    G.gemm(e(0, 2, 8, 64, dtype=bf), e(0, 2, 64, 32, dtype=bf), e(0, 2, 8, 32, dtype=bf), prec="bf16")
    G.conv2d(e(0, 8, 8, 16), e(4, 3, 3, 16), e(0, 8, 8, 4), (1, 1), (1, 1))
    G.maxpool2d(e(0, 8, 8, 4), e(0, 4, 4, 4), (2, 2), (2, 2), (0, 0))
    G.softmax(e(0, 128), e(0, 128))
    G.layernorm(e(0, 64), e(64), e(64), e(0, 64), 1e-5)
    G.reduce(e(0, 7, 3), e(0, 3), "sum")
    G.attention(e(1, 2, 0, 64, dtype=bf), e(1, 2, 16, 64, dtype=bf), e(1, 2, 16, 64, dtype=bf), e(1, 2, 0, 64, dtype=bf))
    torch.cuda.synchronize()
    from llcompiler_b200 import _capi as C
    assert C.lib().llc_cuda_status() == 0


@pytest.mark.parametrize("nbytes,ndst,offset", [(16 * 1000, 3, 0), (16 * 4096 + 7, 2, 160), (5, 1, 16), (151 * 1024 * 1024 // 8, 8, 0)])
def test_push_rows_copies_into_every_destination(nbytes, ndst, offset):
    # the gather kernel with all destinations on this GPU: every destination gets the bytes at the offset, nothing else moves
    import ctypes
    from llcompiler_b200 import _capi as C
    src = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=DEV)
    dsts = [torch.full((offset + nbytes + 32,), 7, dtype=torch.uint8, device=DEV) for _ in range(ndst)]
    ptrs = (ctypes.c_void_p * ndst)(*[d.data_ptr() for d in dsts])
    C.check(C.lib().llc_cuda_push_rows(src.data_ptr(), ptrs, ndst, offset, nbytes, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    for d in dsts:
        assert torch.equal(d[offset:offset + nbytes], src)
        assert bool((d[:offset] == 7).all()) and bool((d[offset + nbytes:] == 7).all())
