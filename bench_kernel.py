"""Runs one kernel case through the C ABI a few times and prints its CUDA-event time: the small, single-kernel
command that profiler captures are taken on, and the per-kernel timing tool behind the tables in profiles/.

  python bench_kernel.py conv  N C H W F K STRIDE PAD PREC [REPS] [res]
  python bench_kernel.py gemm  M N K PREC [REPS] [plain|bias|gelu|res]
  python bench_kernel.py attention  BATCH HEADS SEQ [REPS]      (bf16, head size 64, row mask)
  python bench_kernel.py layernorm  ROWS D DTYPE [REPS]
  python bench_kernel.py softmax    ROWS LEN DTYPE [REPS]
  python bench_kernel.py maxpool    N C H W DTYPE [REPS]        (3x3, stride 2, pad 1, NHWC)
  python bench_kernel.py gather     ROWS D VOCAB DTYPE [REPS]
  python bench_kernel.py eltwise    ROWS D DTYPE [REPS]         (out = a + b[broadcast row])
  python bench_kernel.py nchw2nhwc  N C H W DTYPE [REPS]        (input re-layout with channel padding and halo)
  python bench_kernel.py push       BYTES NDST [REPS]           (the gather's multi-destination copy, destinations on this GPU)
PREC: bf16 | tf32 | tf32x3 | fp32      DTYPE: bf16 | f32
Every repetition is timed with CUDA events on the launching stream after an L2 flush (a 256 MB write); the line
printed is the median: `<kind> ... ms <t> TFLOP/s <x> GB/s <y> status <word>` with the algorithmic FLOPs and bytes.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "tests"))
sys.path.insert(0, HERE)
import gpu_ops as G  # noqa: E402
from llcompiler_b200 import _capi as C  # noqa: E402

_FLUSH = None


def timed(fn, reps):
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        _FLUSH.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    ms.sort()
    return ms[len(ms) // 2]


def report(label, ms, flops, nbytes):
    print(f"{label}: ms {ms:.4f} TFLOP/s {flops / ms / 1e9:.1f} GB/s {nbytes / ms / 1e6:.1f} status {C.lib().llc_cuda_status()}")


def _dt(name):
    return torch.bfloat16 if name in ("bf16", "bfloat16") else torch.float32


def main(argv):
    kind = argv[0]
    if kind == "conv":
        n, c, h, w, f, k, s, p = (int(a) for a in argv[1:9])
        prec = argv[9]
        reps = int(argv[10]) if len(argv) > 10 else 3
        with_res = len(argv) > 11 and argv[11] == "res"
        dt = torch.bfloat16 if prec == "bf16" else torch.float32
        oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        g = torch.Generator(device="cuda").manual_seed(0)
        x = torch.randn(n, h, w, c, device="cuda", generator=g).to(dt)
        wt = torch.randn(f, k, k, c, device="cuda", generator=g).to(dt)
        out = torch.empty(n, oh, ow, f, device="cuda", dtype=dt)
        res = torch.randn(n, oh, ow, f, device="cuda", generator=g).to(dt) if with_res else None
        shift = torch.zeros(f, device="cuda")
        ws = torch.zeros(16 << 20, dtype=torch.uint8, device="cuda")
        # weights arrive pre-split at precision tf32x3, as the runtime hands them over
        w_lo = (wt - (wt.view(torch.int32) & -8192).view(torch.float32)) if prec == "tf32x3" else None
        ms = timed(lambda: G.conv2d(x, wt, out, (s, s), (p, p), shift=shift, res=res, act="relu", prec=prec, w_lo=w_lo, workspace=ws), reps)
        eb = x.element_size()
        report(" ".join(argv), ms, 2.0 * n * oh * ow * f * k * k * c, (x.numel() + wt.numel() + out.numel() * (2 if with_res else 1)) * eb)
    elif kind == "gemm":
        m, n, k = (int(a) for a in argv[1:4])
        prec = argv[4]
        reps = int(argv[5]) if len(argv) > 5 else 3
        epi = argv[6] if len(argv) > 6 else "plain"
        dt = torch.bfloat16 if prec == "bf16" else torch.float32
        a = torch.randn(m, k, device="cuda").to(dt)
        b = torch.randn(n, k, device="cuda").to(dt)
        out = torch.empty(1, 1, m, n, device="cuda", dtype=dt)
        bias = torch.randn(n, device="cuda") if epi != "plain" else None
        res = torch.randn(1, 1, m, n, device="cuda").to(dt) if epi == "res" else None
        ws = torch.zeros(16 << 20, dtype=torch.uint8, device="cuda")
        ms = timed(lambda: G.gemm(a[None, None], b.t()[None, None], out, shift=bias, res=res, act="gelu" if epi == "gelu" else "none", prec=prec, workspace=ws), reps)
        report(" ".join(argv), ms, 2.0 * m * n * k, (m * k + n * k + m * n * (2 if epi == "res" else 1)) * a.element_size())
    elif kind == "attention":
        b, h, sq = (int(a) for a in argv[1:4])
        reps = int(argv[4]) if len(argv) > 4 else 3
        q, k, v = (torch.randn(b, sq, h * 64, device="cuda").to(torch.bfloat16) for _ in range(3))
        out = torch.empty_like(q)
        mask = torch.zeros(b, 1, 1, sq, device="cuda").expand(b, h, sq, sq)
        heads = lambda t: t.view(b, sq, h, 64).permute(0, 2, 1, 3)
        ms = timed(lambda: G.attention(heads(q), heads(k), heads(v), heads(out), mask=mask, scale=0.125), reps)
        report(" ".join(argv), ms, 4.0 * b * h * sq * sq * 64, 4 * q.numel() * 2)
    elif kind == "layernorm":
        rows, d = int(argv[1]), int(argv[2])
        dt = _dt(argv[3]); reps = int(argv[4]) if len(argv) > 4 else 5
        x = torch.randn(rows, d, device="cuda").to(dt)
        gm, bt = torch.randn(d, device="cuda").to(dt), torch.randn(d, device="cuda").to(dt)
        out = torch.empty_like(x)
        ms = timed(lambda: G.layernorm(x, gm, bt, out, 1e-5), reps)
        report(" ".join(argv), ms, 0.0, 2 * x.numel() * x.element_size())
    elif kind == "softmax":
        rows, ln = int(argv[1]), int(argv[2])
        dt = _dt(argv[3]); reps = int(argv[4]) if len(argv) > 4 else 5
        x = torch.randn(rows, ln, device="cuda").to(dt)
        out = torch.empty_like(x)
        ms = timed(lambda: G.softmax(x, out), reps)
        report(" ".join(argv), ms, 0.0, 2 * x.numel() * x.element_size())
    elif kind == "maxpool":
        n, c, h, w = (int(a) for a in argv[1:5])
        dt = _dt(argv[5]); reps = int(argv[6]) if len(argv) > 6 else 5
        x = torch.randn(n, h, w, c, device="cuda").to(dt)
        oh, ow = (h + 2 - 3) // 2 + 1, (w + 2 - 3) // 2 + 1
        out = torch.empty(n, oh, ow, c, device="cuda", dtype=dt)
        ms = timed(lambda: G.maxpool2d(x, out, (3, 3), (2, 2), (1, 1)), reps)
        report(" ".join(argv), ms, 0.0, (x.numel() + out.numel()) * x.element_size())
    elif kind == "gather":
        rows, d, vocab = (int(a) for a in argv[1:4])
        dt = _dt(argv[4]); reps = int(argv[5]) if len(argv) > 5 else 5
        table = torch.randn(vocab, d, device="cuda").to(dt)
        ids = torch.randint(0, vocab, (rows,), device="cuda")
        out = torch.empty(rows, d, device="cuda", dtype=dt)
        ms = timed(lambda: G.gather(table, ids, out), reps)
        report(" ".join(argv), ms, 0.0, 2 * out.numel() * out.element_size() + ids.numel() * 8)
    elif kind == "eltwise":
        rows, d = int(argv[1]), int(argv[2])
        dt = _dt(argv[3]); reps = int(argv[4]) if len(argv) > 4 else 5
        a = torch.randn(rows, d, device="cuda").to(dt)
        b = torch.randn(1, d, device="cuda").to(dt).expand(rows, d)
        out = torch.empty_like(a)
        ms = timed(lambda: G.eltwise(out, [a, b], "ld0;ld1;add,0,1"), reps)
        report(" ".join(argv), ms, 0.0, 2 * a.numel() * a.element_size())
    elif kind == "nchw2nhwc":
        n, c, h, w = (int(a) for a in argv[1:5])
        dt = _dt(argv[5]); reps = int(argv[6]) if len(argv) > 6 else 5
        cpad = 16 // (2 if dt == torch.bfloat16 else 4)
        x = torch.randn(n, c, h, w, device="cuda").to(dt)
        out = torch.empty(n, h, w + 8, cpad, device="cuda", dtype=dt)
        ms = timed(lambda: G.nchw_to_nhwc_wide(x, out, cpad, 3, w + 8), reps)
        report(" ".join(argv), ms, 0.0, (x.numel() + out.numel()) * x.element_size())
    elif kind == "push":
        import ctypes
        nbytes, ndst = int(argv[1]), int(argv[2])
        reps = int(argv[3]) if len(argv) > 3 else 7
        src = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda")
        dsts = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(ndst)]
        ptrs = (ctypes.c_void_p * ndst)(*[d.data_ptr() for d in dsts])
        st = torch.cuda.current_stream().cuda_stream
        ms = timed(lambda: C.check(C.lib().llc_cuda_push_rows(src.data_ptr(), ptrs, ndst, 0, nbytes, st)), reps)
        assert all(torch.equal(d, src) for d in dsts)
        report(" ".join(argv), ms, 0.0, (1 + ndst) * nbytes)
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1:])
