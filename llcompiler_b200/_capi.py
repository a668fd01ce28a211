"""ctypes view of the C ABI in include/llc_runtime.h and include/llc_cuda.h.

The product path goes through the ``llcompiler_`` extension module; this thin
layer exists for the tests (which must call kernels through the C ABI) and for
tools that only need the compile side.  It never falls back to anything: a
missing library is an ImportError with the build command in it.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path
from typing import Optional, Sequence

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libllc_cuda.so"


class LlcTensor(Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("device", c_int32), ("rank", c_int32),
                ("sizes", POINTER(c_int64)), ("strides", POINTER(c_int64))]


class LlcOptions(Structure):
    _fields_ = [(n, c_char_p) for n in ("mode", "target", "pipeline", "global_layout", "log_root",
                                        "log_level", "cpu", "mtriple", "precision")]


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing; build it with `python -m llcompiler_b200.build`")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.llc_last_error.restype = c_char_p
        _lib.llc_version.restype = c_char_p
        _lib.llc_compile.argtypes = [c_char_p, POINTER(LlcOptions), c_char_p, c_size_t]
        _lib.llc_run_pass.argtypes = [c_char_p, c_char_p, POINTER(LlcOptions), POINTER(c_char_p)]
        _lib.llc_cuda_push_rows.argtypes = [ctypes.c_void_p, POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    return _lib


class LlcError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[llc status {code}] {message}")
        self.code = code


def check(code: int) -> None:
    if code != 0:
        raise LlcError(code, lib().llc_last_error().decode("utf-8", "replace"))


def make_options(**kw) -> LlcOptions:
    o = LlcOptions()
    for k, v in kw.items():
        if v is not None:
            setattr(o, k, str(v).encode())
    return o


def run_pass(text: str, pass_name: str, **options) -> str:
    out = c_char_p()
    o = make_options(**options)
    check(lib().llc_run_pass(text.encode(), pass_name.encode(), byref(o), byref(out)))
    return out.value.decode()


def compile_text(text: str, **options) -> str:
    buf = ctypes.create_string_buffer(1024)
    o = make_options(**options)
    check(lib().llc_compile(text.encode(), byref(o), buf, len(buf)))
    return buf.value.decode()


def tensor_desc(ptr: int, dtype_code: int, device: int, sizes: Sequence[int], strides: Sequence[int]):
    """Returns (LlcTensor, keepalive) for caller-owned memory."""
    n = len(sizes)
    s = (c_int64 * max(n, 1))(*sizes)
    st = (c_int64 * max(n, 1))(*strides)
    t = LlcTensor(c_void_p(ptr), dtype_code, device, n, ctypes.cast(s, POINTER(c_int64)), ctypes.cast(st, POINTER(c_int64)))
    return t, (s, st)


# ---- kernel library (include/llc_cuda.h) -----------------------------------------------
from ctypes import c_float  # noqa: E402

LLC_DTYPE = {"int8": 0, "int16": 1, "int32": 2, "int64": 3, "float32": 4, "float64": 5, "bool": 6,
             "float16": 7, "bfloat16": 8}
ACT = {"none": 0, "relu": 1, "gelu": 2}
PREC = {"fp32": 0, "tf32": 1, "tf32x3": 2, "bf16": 3}


class LlcGemmParams(Structure):
    _fields_ = [("a", c_void_p), ("b", c_void_p), ("out", c_void_p), ("scale", c_void_p), ("shift", c_void_p),
                ("res", c_void_p), ("in_dtype", c_int32), ("out_dtype", c_int32), ("res_dtype", c_int32),
                ("precision", c_int32)] + [(n, c_int64) for n in (
                    "m", "n", "k", "b0", "b1", "a_s0", "a_s1", "a_sm", "b_s0", "b_s1", "b_sk", "b_sn",
                    "o_s0", "o_s1", "o_sm", "r_s0", "r_s1", "r_sm", "r_sn")] + [("alpha", c_float), ("act", c_int32),
                                                                               ("workspace", c_void_p), ("workspace_bytes", c_int64), ("b_lo", c_void_p)]


class LlcConvParams(Structure):
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("out", c_void_p), ("scale", c_void_p), ("shift", c_void_p),
                ("res", c_void_p), ("in_dtype", c_int32), ("out_dtype", c_int32), ("res_dtype", c_int32),
                ("precision", c_int32)] + [(n, c_int64) for n in ("n", "h", "w_in", "c", "f", "kh", "kw", "oh", "ow")] + \
               [(n, c_int32) for n in ("stride_h", "stride_w", "pad_h", "pad_w", "dil_h", "dil_w")] + \
               [("alpha", c_float), ("act", c_int32), ("w_lo", c_void_p), ("x_sn", c_int64), ("x_sh", c_int64), ("x_sw", c_int64), ("workspace", c_void_p), ("workspace_bytes", c_int64)]


class LlcAttentionParams(Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("mask", c_void_p), ("out", c_void_p),
                ("dtype", c_int32), ("mask_dtype", c_int32)] + [(n, c_int64) for n in (
                    "b0", "b1", "m", "n", "d", "q_s0", "q_s1", "q_sm", "k_s0", "k_s1", "k_sn", "v_s0", "v_s1", "v_sn",
                    "o_s0", "o_s1", "o_sm", "mask_s0", "mask_s1", "mask_sm")] + [("scale", c_float)]


class LlcPoolParams(Structure):
    _fields_ = [("x", c_void_p), ("out", c_void_p), ("in_dtype", c_int32), ("out_dtype", c_int32)] + \
               [(n, c_int64) for n in ("n", "h", "w", "c", "oh", "ow")] + \
               [(n, c_int32) for n in ("kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w", "dil_h", "dil_w")]


class LlcEltwiseOperand(Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("strides", c_int64 * 6)]


class LlcEltwiseParams(Structure):
    _fields_ = [("out", c_void_p), ("out_dtype", c_int32), ("rank", c_int32), ("shape", c_int64 * 6),
                ("out_strides", c_int64 * 6), ("n_in", c_int32), ("inputs", LlcEltwiseOperand * 8), ("prog", c_char_p)]


EXPORTED_SYMBOLS = [
    "llc_compile", "llc_run_pass", "llc_load", "llc_load_from", "llc_loaded_from_pool", "llc_num_inputs", "llc_num_outputs", "llc_num_symbols",
    "llc_output_shape", "llc_run", "llc_profile", "llc_status", "llc_last_launch_count", "llc_arena_bytes", "llc_free", "llc_last_error",
    "llc_version", "llc_cuda_gemm", "llc_cuda_conv2d", "llc_cuda_maxpool2d", "llc_cuda_reduce",
    "llc_cuda_softmax", "llc_cuda_layernorm", "llc_cuda_gather", "llc_cuda_eltwise", "llc_cuda_status", "llc_cuda_nchw_to_nhwc", "llc_cuda_gemm_static_scratch", "llc_cuda_attention", "llc_cuda_nchw_to_nhwc_wide",
    "llc_cuda_push_rows",
]
