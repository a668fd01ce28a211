"""ctypes wrappers that call the kernel library through its C ABI on torch CUDA tensors
(torch only provides the device memory and the stream)."""
from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p

import torch

from llcompiler_b200 import _capi as C

_DT = {torch.float32: 4, torch.bfloat16: 8, torch.int64: 3, torch.int32: 2, torch.bool: 6, torch.float16: 7,
       torch.float64: 5, torch.int8: 0, torch.int16: 1}


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def gemm(a, b, out, scale=None, shift=None, res=None, alpha=1.0, act="none", prec="fp32", workspace=None, b_lo=None):
    """a [b0,b1,M,K] (k stride 1), b [b0,b1,K,N] (k or n stride 1), out [b0,b1,M,N] views."""
    p = C.LlcGemmParams()
    p.a, p.b, p.out, p.scale, p.shift, p.res = _p(a), _p(b), _p(out), _p(scale), _p(shift), _p(res)
    p.in_dtype, p.out_dtype = _DT[a.dtype], _DT[out.dtype]
    p.res_dtype = _DT[res.dtype] if res is not None else 4
    p.precision = C.PREC[prec]
    p.b0, p.b1, p.m, p.n, p.k = out.shape[0], out.shape[1], out.shape[2], out.shape[3], a.shape[3]
    p.a_s0, p.a_s1, p.a_sm = a.stride(0), a.stride(1), a.stride(2)
    p.b_s0, p.b_s1, p.b_sk, p.b_sn = b.stride(0), b.stride(1), b.stride(2), b.stride(3)
    p.o_s0, p.o_s1, p.o_sm = out.stride(0), out.stride(1), out.stride(2)
    if res is not None:
        p.r_s0, p.r_s1, p.r_sm, p.r_sn = res.stride(0), res.stride(1), res.stride(2), res.stride(3)
    p.alpha, p.act = alpha, C.ACT[act]
    if workspace is not None:
        p.workspace, p.workspace_bytes = _p(workspace), workspace.numel() * workspace.element_size()
    p.b_lo = _p(b_lo)
    C.check(C.lib().llc_cuda_gemm(byref(p), _stream()))


def attention(q, k, v, out, mask=None, scale=1.0):
    """q [b0,b1,M,D], k and v [b0,b1,N,D], out [b0,b1,M,D] views with unit stride along D; mask broadcastable
    [b0,b1,M,N] view (stride 0 where it broadcasts) with unit stride along N."""
    p = C.LlcAttentionParams()
    p.q, p.k, p.v, p.mask, p.out = _p(q), _p(k), _p(v), _p(mask), _p(out)
    p.dtype = _DT[q.dtype]
    p.mask_dtype = _DT[mask.dtype] if mask is not None else 4
    p.b0, p.b1, p.m, p.d, p.n = q.shape[0], q.shape[1], q.shape[2], q.shape[3], k.shape[2]
    p.q_s0, p.q_s1, p.q_sm = q.stride(0), q.stride(1), q.stride(2)
    p.k_s0, p.k_s1, p.k_sn = k.stride(0), k.stride(1), k.stride(2)
    p.v_s0, p.v_s1, p.v_sn = v.stride(0), v.stride(1), v.stride(2)
    p.o_s0, p.o_s1, p.o_sm = out.stride(0), out.stride(1), out.stride(2)
    if mask is not None:
        p.mask_s0, p.mask_s1, p.mask_sm = mask.stride(0), mask.stride(1), mask.stride(2)
    p.scale = scale
    C.check(C.lib().llc_cuda_attention(byref(p), _stream()))


def conv2d(x_nhwc, w_fhwc, out_nhwc, stride, pad, dil=(1, 1), scale=None, shift=None, res=None, alpha=1.0,
           act="none", prec="fp32", w_lo=None, x_strides=None, x_shape=None, workspace=None):
    p = C.LlcConvParams()
    p.x, p.w, p.out, p.scale, p.shift, p.res = _p(x_nhwc), _p(w_fhwc), _p(out_nhwc), _p(scale), _p(shift), _p(res)
    p.in_dtype, p.out_dtype = _DT[x_nhwc.dtype], _DT[out_nhwc.dtype]
    p.res_dtype = _DT[res.dtype] if res is not None else 4
    p.precision = C.PREC[prec]
    p.n, p.h, p.w_in, p.c = x_nhwc.shape
    p.f, p.kh, p.kw = w_fhwc.shape[0], w_fhwc.shape[1], w_fhwc.shape[2]
    p.oh, p.ow = out_nhwc.shape[1], out_nhwc.shape[2]
    p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.dil_h, p.dil_w = stride[0], stride[1], pad[0], pad[1], dil[0], dil[1]
    p.alpha, p.act = alpha, C.ACT[act]
    p.w_lo = _p(w_lo)
    if workspace is not None:
        p.workspace, p.workspace_bytes = _p(workspace), workspace.numel() * workspace.element_size()
    if x_strides is not None:        # (n, h, w) element strides of an explicit, possibly overlapping, view; x_shape = (n, h, w, c)
        p.x_sn, p.x_sh, p.x_sw = x_strides
        p.n, p.h, p.w_in, p.c = x_shape
    C.check(C.lib().llc_cuda_conv2d(byref(p), _stream()))


def maxpool2d(x_nhwc, out_nhwc, k, stride, pad, dil=(1, 1)):
    p = C.LlcPoolParams()
    p.x, p.out = _p(x_nhwc), _p(out_nhwc)
    p.in_dtype, p.out_dtype = _DT[x_nhwc.dtype], _DT[out_nhwc.dtype]
    p.n, p.h, p.w, p.c = x_nhwc.shape
    p.oh, p.ow = out_nhwc.shape[1], out_nhwc.shape[2]
    p.kh, p.kw, p.stride_h, p.stride_w, p.pad_h, p.pad_w, p.dil_h, p.dil_w = k[0], k[1], stride[0], stride[1], pad[0], pad[1], dil[0], dil[1]
    C.check(C.lib().llc_cuda_maxpool2d(byref(p), _stream()))


def reduce(x3, out2, op):
    code = {"sum": 0, "max": 1, "min": 2, "mean": 3}[op]
    f = C.lib().llc_cuda_reduce
    f.argtypes = [c_void_p, c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, c_void_p]
    C.check(f(_p(x3), _p(out2), _DT[x3.dtype], _DT[out2.dtype], x3.shape[0], x3.shape[1], x3.shape[2], code, _stream()))


def softmax(x2, out2):
    f = C.lib().llc_cuda_softmax
    f.argtypes = [c_void_p, c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, c_void_p]
    C.check(f(_p(x2), _p(out2), _DT[x2.dtype], _DT[out2.dtype], x2.shape[0], x2.shape[1], _stream()))


def layernorm(x2, gamma, beta, out2, eps):
    f = C.lib().llc_cuda_layernorm
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_float, c_void_p]
    C.check(f(_p(x2), _p(gamma), _p(beta), _p(out2), _DT[x2.dtype], _DT[gamma.dtype], _DT[out2.dtype], x2.shape[0], x2.shape[1], eps, _stream()))


def gather(table, ids, out, bad=None):
    f = C.lib().llc_cuda_gather
    f.argtypes = [c_void_p, c_void_p, c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, c_void_p, c_void_p]
    C.check(f(_p(table), _p(ids), _p(out), _DT[table.dtype], _DT[out.dtype], out.shape[0], out.shape[1], table.shape[0], _p(bad), _stream()))


def eltwise(out, inputs, prog):
    """out and inputs are (possibly strided / broadcast) views of the same logical shape."""
    p = C.LlcEltwiseParams()
    p.out, p.out_dtype, p.rank = _p(out), _DT[out.dtype], out.dim()
    for d in range(out.dim()):
        p.shape[d] = out.shape[d]
        p.out_strides[d] = out.stride(d)
    p.n_in = len(inputs)
    for k, t in enumerate(inputs):
        p.inputs[k].data = _p(t)
        p.inputs[k].dtype = _DT[t.dtype]
        for d in range(t.dim()):
            p.inputs[k].strides[d] = t.stride(d)
    p.prog = prog.encode()
    C.check(C.lib().llc_cuda_eltwise(byref(p), _stream()))


def nchw_to_nhwc_wide(x_nchw, out, c_pad, w_left, w_total):
    n, c, h, w = x_nchw.shape
    f = C.lib().llc_cuda_nchw_to_nhwc_wide
    f.argtypes = [c_void_p, c_void_p, ctypes.c_int32] + [ctypes.c_int64] * 7 + [c_void_p]
    C.check(f(_p(x_nchw), _p(out), _DT[x_nchw.dtype], n, c, h, w, c_pad, w_left, w_total, _stream()))
