"""Execution engines with the reference's names (llcompiler/executor/engine.py:14-78).

``Torch_ExecutionEngine.run(*args)`` takes python ints (symbol values) and torch tensors
and returns torch tensors, like the reference.  Differences: tensors may live on the GPU
(then nothing is copied and the call only enqueues work on the current CUDA stream) or
on the host (then the C ABI stages them through device memory, which is the reference's
calling convention); outputs are sized by the plan's symbolic shapes through
``Execution.output_shapes`` instead of a FakeTensorProp pass per call
(llcompiler/executor/out_put_call.py:154-170).
"""
from __future__ import annotations

import sys
from typing import Any, List, Optional

import torch

try:
    from llcompiler_.executor import Execution
    from llcompiler_.tensor import Tensor
except ImportError as e:  # the CUDA path is the only path: fail loudly
    raise ImportError("the llcompiler_ extension module is not built; run `python -m llcompiler_b200.build`") from e

# reference codes 0..6 (engine.py:11) plus FLOAT16=7, BFLOAT16=8
TORCH_DTYPE_TO_TYPE = {torch.int8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3, torch.float32: 4,
                       torch.float64: 5, torch.bool: 6, torch.float16: 7, torch.bfloat16: 8}
TYPE_TO_TORCH_DTYPE = {v: k for k, v in TORCH_DTYPE_TO_TYPE.items()}


class ExecutionEngine:
    def __init__(self, so_file: str, device: Optional[int] = None, weight_dir: Optional[str] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("the B200 backend needs a CUDA device; there is no CPU fallback")
        self.device = torch.cuda.current_device() if device is None else int(device)
        self.executor = Execution()
        # `weight_dir`: where the plan's .npy files live (looked up by name) and where the uploaded weight pool is kept
        self.executor.load(so_file, self.device, weight_dir or "")
        self.gen_outs_call = None
        self._out_meta = {}
        self._pinned = {}

    def _host_output(self, shape, dtype) -> torch.Tensor:
        """A page-locked host tensor for a result that goes back to the host (a device-to-host copy into pageable
        memory runs at a fraction of the link rate).  Buffers are kept and handed out again only when nothing else
        refers to them any more: neither the tensor object nor, through a view or a numpy array, its storage."""
        use_count = getattr(torch._C, "_storage_Use_Count", None)
        pool = self._pinned.setdefault((shape, dtype), [])
        if use_count is not None:
            for t in pool:
                if sys.getrefcount(t) <= 3 and use_count(t.untyped_storage()._cdata) <= 2:
                    return t
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        if use_count is not None and len(pool) < 4:
            pool.append(t)
        return t

    def run(self, *args) -> Any:
        raise NotImplementedError

    def __call__(self, *args) -> Any:
        return self.run(*args)


class Torch_ExecutionEngine(ExecutionEngine):
    def trans_to_tensor(self, *args) -> List[Tensor]:
        out = []
        for a in args:
            if isinstance(a, torch.Tensor):
                dev = a.device.index if a.is_cuda else -1
                # data_ptr() already includes the storage offset (the reference adds it twice,
                # engine.py:39-46, which is only right for offset 0)
                out.append(Tensor(a.data_ptr(), a.data_ptr(), TORCH_DTYPE_TO_TYPE[a.dtype], a.storage_offset(),
                                  list(a.shape), list(a.stride()), dev))
            elif isinstance(a, int) or a is None:
                continue
            else:
                raise TypeError(f"Unsupported type: {type(a)}")
        return out

    def run(self, *args) -> Any:
        if len(args) == 1 and isinstance(args[0], (list, tuple)):
            args = tuple(args[0])
        symbols = [int(a) for a in args if isinstance(a, int) and not isinstance(a, bool)]
        tensors = [a if a.is_contiguous() else a.contiguous() for a in args if isinstance(a, torch.Tensor)]
        inputs = self.trans_to_tensor(*tensors)
        on_gpu = any(t.is_cuda for t in tensors)
        out_device = torch.device("cuda", self.device) if on_gpu else torch.device("cpu")
        # output extents depend only on the symbol values and the input extents: ask once per signature
        key = (tuple(symbols), tuple(tuple(t.shape) for t in tensors))
        meta = self._out_meta.get(key)
        if meta is None:
            meta = [(tuple(shape), TYPE_TO_TORCH_DTYPE[code]) for shape, code in self.executor.output_shapes(symbols, inputs)]
            self._out_meta[key] = meta
        outputs = [torch.empty(shape, dtype=dt, device=out_device) if on_gpu else self._host_output(shape, dt) for shape, dt in meta]
        outputs_ = self.trans_to_tensor(*outputs)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if symbols:
            self.executor.run_with_symbols(symbols, inputs, outputs_, stream)
        else:
            self.executor.run(inputs, outputs_, stream)
        return outputs

    def status(self):
        """Waits for the device and raises if a kernel of an earlier call recorded a failure: a tensor-core kernel whose
        bounded wait gave up, or embedding indices outside their table (those rows are zeros).  ``run`` makes this check
        itself when its tensors live on the host; with device tensors the call returns before the kernels have run, so
        the caller asks here after its own synchronisation.  Returns the three status words (all zero when healthy)."""
        return self.executor.status()

    def profile(self, *args, reps: int = 5):
        """Per-kernel CUDA-event timing of one call: list of dicts with kernel, launches, ms, flops, bytes."""
        symbols = [int(a) for a in args if isinstance(a, int) and not isinstance(a, bool)]
        tensors = [a.detach().contiguous() for a in args if isinstance(a, torch.Tensor)]
        inputs = self.trans_to_tensor(*tensors)
        on_gpu = any(t.is_cuda for t in tensors)
        dev = torch.device("cuda", self.device) if on_gpu else torch.device("cpu")
        outputs = [torch.empty(shape, dtype=TYPE_TO_TORCH_DTYPE[code], device=dev) for shape, code in self.executor.output_shapes(symbols, inputs)]
        report = self.executor.profile(symbols, inputs, self.trans_to_tensor(*outputs), reps, torch.cuda.current_stream(self.device).cuda_stream)
        rows, steps = [], []
        for line in report.splitlines():
            f = line.split()
            if f and f[0] == "kernel":
                rows.append({"kernel": f[1], "launches": int(f[2]), "ms": float(f[3]), "flops": float(f[4]), "bytes": float(f[5])})
            elif f and f[0] == "step":
                steps.append({"index": int(f[1]), "kernel": f[2], "ms": float(f[3]), "flops": float(f[4]), "bytes": float(f[5])})
        self.last_profile_steps = steps
        return rows
