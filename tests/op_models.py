"""Small modules that exercise one LLH op family each, mirroring what the reference's own op
tests run (test/python/ops/*.py with llcompiler/test_models/ops/*.py): same op parameters
(conv 5x5 pad 2 applied twice, max-pool (5,1,2,dilation 2) twice, batch-norm inference applied
four times, three bias-free Linear layers, x @ x^T, x[1] + x[-2] + x[0], ...), smaller images so
that the CPU oracle runs in seconds."""
import torch
import torch.nn as nn


class Abs(nn.Module):
    def forward(self, x):
        return torch.abs(x)


class Add(nn.Module):
    def forward(self, x):
        x = x + x
        return x + 3


class Sub(nn.Module):
    def forward(self, x):
        return (x - 2) - x * 0.5


class Mul(nn.Module):
    def forward(self, x):
        return x * x * 2


class Div(nn.Module):
    def forward(self, x):
        return (x / 2) / (x * x + 1.0)


class Relu(nn.Module):
    def forward(self, x):
        return torch.relu(x)


class Sqrt(nn.Module):
    def forward(self, x):
        return torch.sqrt(torch.abs(x))


class ElementaryArithmetic(nn.Module):
    def forward(self, x):
        y = x + x
        y = y - 3
        y = y * x
        return y / 2


class Conv2D(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 3, kernel_size=5, stride=1, padding=2, bias=False)

    def forward(self, x):
        return self.conv(self.conv(x))


class MaxPool2D(nn.Module):
    def __init__(self):
        super().__init__()
        self.pool = nn.MaxPool2d(5, 1, 2, 2)

    def forward(self, x):
        return self.pool(self.pool(x))


class BatchNorm2DInference(nn.Module):
    def __init__(self):
        super().__init__()
        self.bn = nn.BatchNorm2d(3)
        with torch.no_grad():
            self.bn.running_mean.copy_(torch.tensor([0.1, -0.2, 0.3]))
            self.bn.running_var.copy_(torch.tensor([1.5, 0.7, 1.1]))
            self.bn.weight.copy_(torch.tensor([1.2, 0.8, 1.0]))
            self.bn.bias.copy_(torch.tensor([0.0, 0.1, -0.1]))

    def forward(self, x):
        for _ in range(4):
            x = self.bn(x)
        return x


class BatchNorm1DInference(nn.Module):
    def __init__(self):
        super().__init__()
        self.bn = nn.BatchNorm1d(3)

    def forward(self, x):
        for _ in range(4):
            x = self.bn(x)
        return x


class Linear(nn.Module):
    def __init__(self, k=10000):
        super().__init__()
        self.l1, self.l2, self.l3 = nn.Linear(k, 10, bias=False), nn.Linear(10, 100, bias=False), nn.Linear(100, 10, bias=False)

    def forward(self, x):
        return self.l3(self.l2(self.l1(x)))


class Matmul(nn.Module):
    def forward(self, x):
        return torch.matmul(x, x.transpose(-2, -1))


class BatchMatmul(nn.Module):
    def forward(self, x):
        return torch.bmm(x, x.transpose(-2, -1))


class Broadcast(nn.Module):
    def forward(self, x):
        x1 = x + x.reshape(1, x.shape[0], x.shape[1])
        x2 = x + x.reshape(x.shape[0], 1, x.shape[1])
        return x1 + x2


class Extract(nn.Module):
    def forward(self, x):
        return x[1] + x[-2] + x[0]


class Slice(nn.Module):
    def forward(self, x):
        return x[0:3] + x[3:6]


class Unsqueeze(nn.Module):
    def forward(self, x):
        return x.unsqueeze(1) + x.unsqueeze(1)


class Where(nn.Module):
    def forward(self, pre, x, y):
        return x.where(pre, y) + y


class ReduceMax(nn.Module):
    def forward(self, x):
        x2 = x.amax(x.dim() - 2, keepdim=False)
        x1 = x.amax(x.dim() - 2, keepdim=True).squeeze(x.dim() - 2)
        return (x1 + x2).amax(-1, keepdim=True)


class ReduceSum(nn.Module):
    def forward(self, x):
        x2 = x.sum(x.dim() - 2, keepdim=False)
        x1 = x.sum(x.dim() - 2, keepdim=True).squeeze(x.dim() - 2)
        return (x1 + x2).sum(-1, keepdim=True)


class Softmax(nn.Module):
    def forward(self, x):
        return torch.softmax(x * 0.5, dim=-1)


class LayerNormGelu(nn.Module):
    def __init__(self):
        super().__init__()
        self.ln = nn.LayerNorm(48)

    def forward(self, x):
        return torch.nn.functional.gelu(self.ln(x))


class AddAlpha(nn.Module):
    def forward(self, x):
        return torch.sub(torch.add(x, x * x, alpha=2), x, alpha=0.5)


class AddmmBetaAlpha(nn.Module):
    def __init__(self):
        super().__init__()
        self.w = nn.Parameter(torch.randn(24, 16))
        self.b = nn.Parameter(torch.randn(16))

    def forward(self, x):
        return torch.addmm(self.b, x, self.w, beta=0.5, alpha=2.0)


class SliceClamped(nn.Module):
    def forward(self, x):
        return x[:, 2:100] + x[:, -3:]           # an end past the extent is clamped, a negative start counts from the end


class CatAlongDims(nn.Module):
    def forward(self, x):
        a = torch.cat([x, torch.relu(x), x * 2.0], dim=1)        # a view, a lazy expression and another one, along a middle dim
        b = torch.cat((a, a[..., :5]), dim=-1)                  # along the last dim, ragged extents
        return torch.cat([b, b], 0)


class Allocations(nn.Module):
    def forward(self, x):
        d = x.device
        z = torch.zeros(3, 24, 20, device=d)
        o = torch.ones_like(x)
        f = torch.full((24, 20), 0.5, device=d)
        e = torch.empty(3, 3, 24, 20, device=d)                  # uninitialised: only its shape may matter
        return (x + z) * o + f + torch.zeros_like(e) + torch.scalar_tensor(2.0, device=d)


def _g(seed):
    return torch.Generator().manual_seed(seed)


# name -> (module factory, input factory, bit_exact)
OP_CASES = {
    "abs": (Abs, lambda: (torch.randn(3, 3, 24, 20, generator=_g(1)),), True),
    "add": (Add, lambda: (torch.randn(3, 3, 24, 20, generator=_g(2)),), True),
    "sub": (Sub, lambda: (torch.randn(3, 3, 24, 20, generator=_g(3)),), False),
    "mul": (Mul, lambda: (torch.randn(3, 3, 24, 20, generator=_g(4)),), True),
    "div": (Div, lambda: (torch.randn(3, 3, 100, generator=_g(5)),), False),
    "relu": (Relu, lambda: (torch.randn(3, 3, 24, 20, generator=_g(6)),), True),
    "sqrt": (Sqrt, lambda: (torch.randn(3, 3, 24, 20, generator=_g(7)),), False),
    "elementary_arithmetic": (ElementaryArithmetic, lambda: (torch.randn(3, 3, 24, 20, generator=_g(8)),), False),
    "conv2d_nchw_fchw": (Conv2D, lambda: (torch.randn(3, 3, 28, 24, generator=_g(9)),), False),
    "max_pool_2d": (MaxPool2D, lambda: (torch.randn(3, 3, 28, 24, generator=_g(10)),), True),
    "batch_norm_2d_inference": (BatchNorm2DInference, lambda: (torch.randn(3, 3, 24, 20, generator=_g(11)),), False),
    "batch_norm_1d_inference": (BatchNorm1DInference, lambda: (torch.randn(3, 3, 224, generator=_g(12)),), False),
    "linear": (Linear, lambda: (torch.randn(10, 10000, generator=_g(13)),), False),
    "matmul": (Matmul, lambda: (torch.randn(3, 3, generator=_g(14)),), False),
    "batch_matmul": (BatchMatmul, lambda: (torch.randn(3, 24, 12, generator=_g(15)),), False),
    "broadcast": (Broadcast, lambda: (torch.randn(24, 12, generator=_g(16)),), False),
    "extract": (Extract, lambda: (torch.randn(6, 5, 7, generator=_g(17)),), False),
    "slice": (Slice, lambda: (torch.randn(6, 5, 7, generator=_g(18)),), True),
    "unsqueeze": (Unsqueeze, lambda: (torch.randn(3, 3, 24, generator=_g(19)),), True),
    "where": (Where, lambda: (torch.randn(100, 24, generator=_g(20)) > 0, torch.randn(100, 24, generator=_g(21)),
                              torch.randn(100, 24, generator=_g(22))), True),
    "reduce_max": (ReduceMax, lambda: (torch.randn(3, 3, 24, 20, generator=_g(23)),), True),
    "reduce_sum": (ReduceSum, lambda: (torch.randn(3, 3, 24, 20, generator=_g(24)),), False),
    "softmax": (Softmax, lambda: (torch.randn(4, 6, 40, generator=_g(25)),), False),
    "add_sub_alpha": (AddAlpha, lambda: (torch.randn(3, 3, 24, 20, generator=_g(27)),), False),
    "addmm_beta_alpha": (AddmmBetaAlpha, lambda: (torch.randn(10, 24, generator=_g(28)),), False),
    "slice_clamped": (SliceClamped, lambda: (torch.randn(6, 5, 7, generator=_g(29)),), True),
    "layer_norm_gelu": (LayerNormGelu, lambda: (torch.randn(4, 6, 48, generator=_g(26)),), False),
    "cat": (CatAlongDims, lambda: (torch.randn(3, 4, 6, 7, generator=_g(30)),), True),
    "allocations": (Allocations, lambda: (torch.randn(3, 3, 24, 20, generator=_g(31)),), False),
}


# The same op families at the reference's own input shapes (test/python/ops/*.py: 3x3x224x224 images,
# batch_matmul 3x224x112, broadcast 224x112, linear 10 x 100000 through three bias-free layers, where 1000x224 with an
# all-true predicate).  Their outputs are too large to commit whole: the golden file keeps a strided sample and a sum.
REFERENCE_SHAPE_CASES = {
    "abs": (Abs, lambda: (torch.randn(3, 3, 224, 224, generator=_g(101)),), True),
    "add": (Add, lambda: (torch.randn(3, 3, 224, 224, generator=_g(102)),), True),
    "sub": (Sub, lambda: (torch.randn(3, 3, 224, 224, generator=_g(103)),), False),
    "mul": (Mul, lambda: (torch.randn(3, 3, 224, 224, generator=_g(104)),), True),
    "div": (Div, lambda: (torch.randn(3, 3, 100, generator=_g(105)),), False),
    "relu": (Relu, lambda: (torch.randn(3, 3, 224, 224, generator=_g(106)),), True),
    "sqrt": (Sqrt, lambda: (torch.randn(3, 3, 224, 224, generator=_g(107)),), False),
    "conv2d_nchw_fchw": (Conv2D, lambda: (torch.randn(3, 3, 224, 224, generator=_g(109)),), False),
    "max_pool_2d": (MaxPool2D, lambda: (torch.randn(3, 3, 224, 224, generator=_g(110)),), True),
    "batch_norm_2d_inference": (BatchNorm2DInference, lambda: (torch.randn(3, 3, 224, 224, generator=_g(111)),), False),
    "batch_norm_1d_inference": (BatchNorm1DInference, lambda: (torch.randn(3, 3, 224, generator=_g(112)),), False),
    "linear": (lambda: Linear(100000), lambda: (torch.randn(10, 100000, generator=_g(113)),), False),
    "matmul": (Matmul, lambda: (torch.randn(3, 3, generator=_g(114)),), False),
    "batch_matmul": (BatchMatmul, lambda: (torch.randn(3, 224, 112, generator=_g(115)),), False),
    "broadcast": (Broadcast, lambda: (torch.randn(224, 112, generator=_g(116)),), False),
    "extract": (Extract, lambda: (torch.randn(3, 3, 224, 224, generator=_g(117)),), False),
    "unsqueeze": (Unsqueeze, lambda: (torch.randn(3, 3, 224, 224, generator=_g(119)),), True),
    "where": (Where, lambda: (torch.ones(1000, 224, dtype=torch.bool), torch.randn(1000, 224, generator=_g(121)),
                              torch.randn(1000, 224, generator=_g(122))), True),
    "reduce_max": (ReduceMax, lambda: (torch.randn(3, 3, 224, 224, generator=_g(123)),), True),
    "reduce_sum": (ReduceSum, lambda: (torch.randn(3, 3, 224, 224, generator=_g(124)),), False),
}
SAMPLE_LIMIT = 2048


def sample_of(t):
    """The strided sample of an output that the golden file keeps for the reference-shape cases."""
    flat = t.reshape(-1)
    step = max(1, flat.numel() // SAMPLE_LIMIT)
    return flat[::step][:SAMPLE_LIMIT].clone()


def build_reference_shape_case(name):
    torch.manual_seed(0)
    factory, inputs, exact = REFERENCE_SHAPE_CASES[name]
    return factory().eval(), inputs(), exact


def build_case(name):
    torch.manual_seed(0)
    factory, inputs, exact = OP_CASES[name]
    return factory().eval(), inputs(), exact
