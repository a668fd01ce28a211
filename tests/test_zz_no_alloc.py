"""The GEMM entry point that allocates nothing (llc_cuda_gemm_static_scratch).

It exists for callers that cannot allocate device memory at call time -- a process whose own
pool already owns the whole GPU, a loop that cannot take the synchronisation an allocation
implies -- and keeps its split-K scratch in a 1 MiB array that is part of the library.  The
test calls it through the C ABI twice in a row (the second call finds the first call's contents
in the shared array) and compares each result with llc_cuda_gemm on the same operands, at the
1e-5 relative tolerance the fp32 kernel tests use; it also checks that an over-sized split is
refused.  The file name sorts last so that a run stopping at the first failure has already run
every other test."""
import ctypes
from ctypes import byref, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

import gpu_ops as G  # noqa: E402
from llcompiler_b200 import _capi as C  # noqa: E402
from oracle.models import max_rel_err  # noqa: E402

DEV = "cuda"


_DT = {torch.float32: 4, torch.bfloat16: 8}


def _params(a, b, out, shift, act):
    p = C.LlcGemmParams()
    p.a, p.b, p.out, p.shift = c_void_p(a.data_ptr()), c_void_p(b.data_ptr()), c_void_p(out.data_ptr()), c_void_p(shift.data_ptr())
    p.in_dtype, p.out_dtype, p.res_dtype = _DT[a.dtype], _DT[out.dtype], 4
    p.precision = C.PREC["fp32"]
    p.b0, p.b1, p.m, p.n, p.k = out.shape[0], out.shape[1], out.shape[2], out.shape[3], a.shape[3]
    p.a_s0, p.a_s1, p.a_sm = a.stride(0), a.stride(1), a.stride(2)
    p.b_s0, p.b_s1, p.b_sk, p.b_sn = b.stride(0), b.stride(1), b.stride(2), b.stride(3)
    p.o_s0, p.o_s1, p.o_sm = out.stride(0), out.stride(1), out.stride(2)
    p.alpha, p.act = 1.0, C.ACT[act]
    return p


# (b0, b1, m, n, k, dtype): shapes whose reduction is split over the built-in scratch (few tiles, k >= 512), one that is
# not split, bf16 operands, and a batched call whose slices and batch entries share the grid's third dimension
CASES = [(1, 1, 64, 512, 784, torch.float32), (1, 1, 64, 10, 512, torch.float32), (1, 1, 200, 300, 64, torch.float32),
         (1, 1, 64, 128, 1024, torch.bfloat16), (2, 3, 48, 40, 640, torch.float32)]


@pytest.mark.parametrize("b0,b1,m,n,k,dtype", CASES)
def test_static_scratch_gemm_matches_the_allocating_entry_point(b0, b1, m, n, k, dtype):
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(b0, b1, m, k, generator=g).to(dtype)
    w = torch.randn(b0, b1, n, k, generator=g).to(dtype)
    bias = torch.randn(n, generator=g)
    A, B, S = a.to(DEV), w.to(DEV).transpose(2, 3), bias.to(DEV)
    # the CPU oracle: float64 accumulation over the (rounded) operands
    want = torch.relu((a.double() @ w.double().transpose(2, 3)).float() + bias)
    tol = 1e-5 if dtype == torch.float32 else 1e-2          # bf16 results are rounded to bf16 on the way out
    ws = torch.zeros(4 << 20, dtype=torch.uint8, device=DEV)
    ref = torch.empty(b0, b1, m, n, device=DEV, dtype=dtype)
    G.gemm(A, B, ref, shift=S, act="relu", workspace=ws)         # existing entry point, split over caller scratch
    assert max_rel_err(ref.float(), want) < tol
    fn = C.lib().llc_cuda_gemm_static_scratch
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):                                           # two calls in a row share the array
        out = torch.full((b0, b1, m, n), float("nan"), device=DEV, dtype=dtype)
        p = _params(A, B, out, S, "relu")
        C.check(fn(byref(p), stream))
        torch.cuda.synchronize()
        assert max_rel_err(out.float(), ref.float().cpu()) < 1e-5      # same kernel, same split: the two entry points agree
        assert max_rel_err(out.float(), want) < tol                    # and the static-scratch result itself matches the oracle


def test_static_scratch_gemm_refuses_a_split_that_does_not_fit():
    # 37 output tiles x 4 K slices x 16 KiB per partial tile is more than the 1 MiB array
    m, n, k = 64 * 37, 64, 16384
    A = torch.zeros(1, 1, m, k, device=DEV)
    B = torch.zeros(n, k, device=DEV).t()[None, None]
    out = torch.empty(1, 1, m, n, device=DEV)
    p = _params(A, B, out, torch.zeros(n, device=DEV), "none")
    rc = C.lib().llc_cuda_gemm_static_scratch(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 3
    assert b"built-in array" in C.lib().llc_last_error()
