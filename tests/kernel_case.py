"""Runs one kernel case through the C ABI a few times (no checks): the small, single-kernel
command that profiler captures are taken on.

  python tests/kernel_case.py conv  N C H W F K STRIDE PAD PREC [REPS]
  python tests/kernel_case.py gemm  M N K PREC [REPS]
  python tests/kernel_case.py attention  BATCH HEADS SEQ [REPS]      (bf16, head size 64, row mask)
PREC: bf16 | tf32 | tf32x3 | fp32
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import gpu_ops as G  # noqa: E402


def main(argv):
    kind = argv[0]
    if kind == "conv":
        n, c, h, w, f, k, s, p = (int(a) for a in argv[1:9])
        prec = argv[9]
        reps = int(argv[10]) if len(argv) > 10 else 3
        dt = torch.bfloat16 if prec == "bf16" else torch.float32
        oh, ow = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        g = torch.Generator(device="cuda").manual_seed(0)
        x = torch.randn(n, h, w, c, device="cuda", generator=g).to(dt)
        wt = torch.randn(f, k, k, c, device="cuda", generator=g).to(dt)
        out = torch.empty(n, oh, ow, f, device="cuda", dtype=dt)
        shift = torch.zeros(f, device="cuda")
        # weights arrive pre-split at precision tf32x3, as the runtime hands them over
        w_lo = (wt - (wt.view(torch.int32) & -8192).view(torch.float32)) if prec == "tf32x3" else None
        for _ in range(reps):
            G.conv2d(x, wt, out, (s, s), (p, p), shift=shift, act="relu", prec=prec, w_lo=w_lo)
    elif kind == "gemm":
        m, n, k = (int(a) for a in argv[1:4])
        prec = argv[4]
        reps = int(argv[5]) if len(argv) > 5 else 3
        dt = torch.bfloat16 if prec == "bf16" else torch.float32
        a = torch.randn(m, k, device="cuda").to(dt)
        b = torch.randn(n, k, device="cuda").to(dt)
        out = torch.empty(1, 1, m, n, device="cuda", dtype=dt)
        for _ in range(reps):
            G.gemm(a[None, None], b.t()[None, None], out, prec=prec)
    elif kind == "attention":
        b, h, sq = (int(a) for a in argv[1:4])
        reps = int(argv[4]) if len(argv) > 4 else 3
        q, k, v = (torch.randn(b, sq, h * 64, device="cuda").to(torch.bfloat16) for _ in range(3))
        out = torch.empty_like(q)
        mask = torch.zeros(b, 1, 1, sq, device="cuda").expand(b, h, sq, sq)
        heads = lambda t: t.view(b, sq, h, 64).permute(0, 2, 1, 3)
        for _ in range(reps):
            G.attention(heads(q), heads(k), heads(v), heads(out), mask=mask, scale=0.125)
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1:])
