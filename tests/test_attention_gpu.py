"""Fused attention kernel (llc_cuda_attention) against a float64 PyTorch restatement, through the C ABI."""
import math

import pytest
import torch

from oracle.models import max_rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


def _reference(q, k, v, mask, scale):
    s = q.double() @ k.double().transpose(-1, -2) * scale
    if mask is not None:
        s = s + mask.double()
    return (torch.softmax(s, -1) @ v.double()).float()


@pytest.fixture(params=["default", "blockwise"])
def kernel_choice(request, monkeypatch):
    """Up to 384 keys the entry point takes its two-pass kernel, above that the blockwise one; the second run sends
    every shape to the blockwise kernel."""
    if request.param == "blockwise":
        monkeypatch.setenv("LLC_ATTENTION_BLOCKS", "1")
    return request.param


CASES = [
    # b0, b1 (heads), M, N, mask kind
    (2, 12, 384, 384, "row"), (1, 3, 128, 128, None), (2, 2, 100, 200, "row"), (1, 2, 300, 72, "full"),
    (3, 1, 17, 384, None), (1, 4, 256, 64, "row"), (2, 3, 130, 330, "full"),
    # four key blocks (the largest resident K / V), an odd tail, and enough tiles that every CTA walks several
    (2, 2, 512, 512, "row"), (1, 3, 200, 450, "full"), (1, 1, 128, 512, None), (16, 12, 384, 384, "row"),
]


@pytest.mark.parametrize("b0,b1,m,n,mask_kind", CASES)
def test_attention_heads_read_in_place(b0, b1, m, n, mask_kind, kernel_choice):
    import gpu_ops as G
    from llcompiler_b200 import _capi as C
    d = 64
    # the projections' outputs [B, S, H*D]: heads are strided views, nothing is copied
    q = _rand(b0, m, b1 * d, dtype=torch.bfloat16).to(DEV)
    k = _rand(b0, n, b1 * d, seed=1, dtype=torch.bfloat16).to(DEV)
    v = _rand(b0, n, b1 * d, seed=2, dtype=torch.bfloat16).to(DEV)
    heads = lambda t, rows: t.view(b0, rows, b1, d).permute(0, 2, 1, 3)
    mask = None
    if mask_kind == "row":
        mask = (_rand(b0, 1, 1, n, seed=3) * 2).to(DEV).expand(b0, b1, m, n)
    elif mask_kind == "full":
        mask = (_rand(b0, 1, m, n, seed=3) * 2).to(DEV).expand(b0, b1, m, n)
    out = torch.full((b0, m, b1 * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    G.attention(heads(q, m), heads(k, n), heads(v, n), heads(out, m), mask=mask, scale=scale)
    torch.cuda.synchronize()
    want = _reference(heads(q, m), heads(k, n), heads(v, n), mask, scale)
    # probabilities and the output are rounded to bf16: 2^-8 relative each
    assert max_rel_err(heads(out, m).float(), want) < 1.5e-2
    assert C.lib().llc_cuda_status() == 0


def test_attention_masked_out_keys_get_no_weight(kernel_choice):
    import gpu_ops as G
    b0, b1, m, n, d = 1, 2, 64, 256, 64
    q, k, v = (_rand(b0, b1, r, d, seed=i, dtype=torch.bfloat16).to(DEV) for i, r in enumerate((m, n, n)))
    mask = torch.zeros(b0, 1, 1, n, device=DEV)
    mask[..., 100:] = float("-inf")
    out = torch.empty(b0, b1, m, d, device=DEV, dtype=torch.bfloat16)
    G.attention(q, k, v, out, mask=mask.expand(b0, b1, m, n), scale=0.125)
    want = _reference(q[:, :, :, :], k[:, :, :100], v[:, :, :100], None, 0.125)
    assert max_rel_err(out.float(), want) < 1.5e-2


@pytest.mark.parametrize("n", [256, 384, 512])
def test_attention_running_maximum_moves_between_key_blocks(n, kernel_choice):
    """The keys are taken in blocks of 128 with a running maximum that only follows a block's maximum in steps larger
    than 2^8: scores that grow from block to block (by far more than that), that shrink, and that stay level all have to
    come out the same as the two-pass softmax; so do rows whose first block is masked out entirely."""
    import gpu_ops as G
    from llcompiler_b200 import _capi as C
    b0, b1, m, d = 2, 3, 256, 64
    q = _rand(b0, b1, m, d, dtype=torch.bfloat16)
    k = _rand(b0, b1, n, d, seed=1, dtype=torch.bfloat16)
    v = _rand(b0, b1, n, d, seed=2, dtype=torch.bfloat16)
    ramp = torch.linspace(0.0, 6.0, n).view(1, 1, n, 1)                  # later keys score much higher ...
    k_up = (k.float() * (0.2 + ramp)).to(torch.bfloat16)
    k_down = (k.float() * (6.2 - ramp)).to(torch.bfloat16)               # ... or much lower
    for kk in (k_up, k_down, k):
        for masked_head in (False, True):
            mask = torch.zeros(b0, 1, 1, n)
            if masked_head:
                mask[..., :128] = float("-inf")                          # the whole first block of keys
                mask[1, ..., :130] = float("-inf")
            out = torch.full((b0, b1, m, d), float("nan"), device=DEV, dtype=torch.bfloat16)
            G.attention(q.to(DEV), kk.to(DEV), v.to(DEV), out, mask=mask.to(DEV).expand(b0, b1, m, n), scale=1.0)
            torch.cuda.synchronize()
            want = _reference(q, kk, v, mask, 1.0)
            assert max_rel_err(out.float(), want) < 1.5e-2
            assert C.lib().llc_cuda_status() == 0


def test_attention_rejects_what_it_cannot_run():
    import gpu_ops as G
    from llcompiler_b200 import _capi as C
    q = torch.zeros(1, 1, 128, 32, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(C.LlcError):
        G.attention(q, q, q, torch.empty_like(q))                      # head size 32
    q = torch.zeros(1, 1, 640, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(C.LlcError):
        G.attention(q, q, q, torch.empty_like(q))                      # 640 keys: more than stay resident
