"""Batch-sharded execution over the GPUs of one node: one process per GPU, replicated weights,
every rank runs its slice of the batch through the same compiled function and the outputs are
all-gathered (NCCL over NVLink on GPUs; gloo in the CPU tests).  The reference has no
distributed code; the batch symbol of its symbolic-shape machinery is what makes one compiled
plan serve the per-rank slice."""
from __future__ import annotations

import collections
from typing import Callable, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split: the first ``total % world`` ranks get one extra sample."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _world_and_rank(group=None) -> Tuple[int, int]:
    """Size and rank of the group; a process without a process group is a group of one."""
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def gather_batch(local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """All-gathers per-rank output slices (dim 0) into the full batch on every rank."""
    world, rank = _world_and_rank(group)
    if world == 1:
        return local
    sizes = [shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0] for r in range(world)]
    if len(set(sizes)) == 1 and local.is_cuda:
        out = local.new_empty((total,) + tuple(local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    pad = max(sizes)
    buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
    buf[: sizes[rank]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


class BatchShardedRunner:
    """Wraps a compiled callable: ``runner(*full_batch_inputs)`` runs this rank's slice and returns the
    gathered full-batch output.  Inputs whose leading extent is not the batch are passed whole.

    With ``device`` set (GPU ranks over NCCL) host inputs are accepted too: the rank's slice is copied to the
    device (asynchronously when the host tensor is page-locked), the gather runs over the device tensors, and the
    gathered batch is copied back to page-locked host memory on the ranks listed in ``host_result_ranks``
    (default: every rank); the other ranks copy back their own slice only.

    ``gather="peer"`` (GPU ranks of one node) replaces the NCCL all-gather by this library's own kernel: the gathered
    batch lives in symmetric memory (two buffers per result shape, used in turn), every rank stores its slice straight
    into every rank's buffer over NVLink (``llc_cuda_push_rows``), with a barrier before (the buffer is free everywhere)
    and after (every slice has arrived).  The tensor returned is one of those two buffers: it is overwritten by the
    next-but-one call.  If symmetric memory cannot be set up the runner falls back to NCCL and says so in
    ``gather_fallback``."""

    def __init__(self, fn: Callable, group=None, device: Optional[torch.device] = None, host_result_ranks: Optional[Sequence[int]] = None,
                 gather: str = "nccl"):
        if gather not in ("nccl", "peer"):
            raise ValueError("gather must be 'nccl' or 'peer'")
        self.fn, self.group, self.device = fn, group, device
        self.gather_mode, self.gather_fallback = gather, None
        self._peer = {}
        self.host_result_ranks = None if host_result_ranks is None else set(host_result_ranks)
        self._host_out = {}
        self._copy_stream = None
        self._upload_stream = None
        self._ring = {}

    def _to_host(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        buf = self._host_out.get(key)
        if buf is None:
            buf = self._host_out[key] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        buf.copy_(t, non_blocking=True)
        torch.cuda.current_stream(t.device).synchronize()
        return buf

    def _peer_state(self, local: torch.Tensor, total: int):
        key = (total, tuple(local.shape[1:]), local.dtype)
        st = self._peer.get(key)
        if st is None:
            import ctypes
            import torch.distributed._symmetric_memory as symm_mem
            buf = symm_mem.empty((2, total) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
            hdl = symm_mem.rendezvous(buf, group=self.group if self.group is not None else dist.group.WORLD)
            ptrs = (ctypes.c_void_p * hdl.world_size)(*[int(p) for p in hdl.buffer_ptrs])
            st = self._peer[key] = {"buf": buf, "hdl": hdl, "ptrs": ptrs, "next": 0, "guard": [None, None]}
        return st

    def gather(self, local: torch.Tensor, total: int):
        """The full batch from every rank's slice: (tensor, token).  With the peer gather the token names the buffer
        used, so that ``pipelined`` can keep it from being overwritten while a copy still reads it."""
        world, rank = _world_and_rank(self.group)
        if self.gather_mode != "peer" or world == 1 or not local.is_cuda or total % world or world > 8:
            return gather_batch(local, total, self.group), None
        try:
            st = self._peer_state(local, total)
        except Exception as e:  # symmetric memory is not available here: the NCCL path is always there
            self.gather_mode, self.gather_fallback = "nccl", f"{type(e).__name__}: {e}"
            return gather_batch(local, total, self.group), None
        from .. import _capi as C
        local = local.contiguous()
        k = st["next"] & 1
        st["next"] += 1
        main = torch.cuda.current_stream(local.device)
        if st["guard"][k] is not None:                 # a read-back of this buffer's previous contents is still in flight
            main.wait_event(st["guard"][k])
            st["guard"][k] = None
        hdl = st["hdl"]
        hdl.barrier(channel=0)                         # every rank is done with buffer k: it may be overwritten
        lo, _ = shard_bounds(total, world, rank)
        row_bytes = local[0].numel() * local.element_size() if local.shape[0] else 0
        C.check(C.lib().llc_cuda_push_rows(local.data_ptr(), st["ptrs"], world, (k * total + lo) * row_bytes,
                                           local.numel() * local.element_size(), main.cuda_stream))
        hdl.barrier(channel=1)                         # every slice has arrived everywhere
        return st["buf"][k], (st, k)

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        world, rank = _world_and_rank(self.group)
        total = inputs[0].shape[0]
        lo, hi = shard_bounds(total, world, rank)
        local = [i[lo:hi] if i.dim() > 0 and i.shape[0] == total else i for i in inputs]
        from_host = self.device is not None and world > 1 and not any(i.is_cuda for i in inputs)
        if from_host:
            local = [i.to(self.device, non_blocking=True) for i in local]
        out = self.fn(*local)
        if isinstance(out, (list, tuple)):
            out = out[0]
        full, _ = self.gather(out, total)
        if from_host:
            wants_full = self.host_result_ranks is None or rank in self.host_result_ranks
            return self._to_host(full if wants_full else out)
        return full

    def pipelined(self, batches: Iterable[Sequence[torch.Tensor]], depth: int = 2) -> Iterator[torch.Tensor]:
        """Runs a stream of batches with up to ``depth`` of them in flight and yields their results, in order, as
        page-locked host tensors: the device-to-host copy of one batch runs on a stream of its own under the kernels
        of the next (and so does the upload of the next batch's inputs), so a result or an input of hundreds of megabytes
        does not add its transfer time to every step.  Each batch is
        what ``__call__`` takes (host or device tensors); sharding, the gather and ``host_result_ranks`` are as there.
        A yielded tensor belongs to a ring of ``depth + 1`` buffers per result shape: it stays valid until ``depth``
        more results have been taken."""
        if self.device is None:
            raise ValueError("pipelined() needs the runner's device")
        if depth < 1:
            raise ValueError("depth must be at least 1")
        world, rank = _world_and_rank(self.group)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._upload_stream = torch.cuda.Stream(device=self.device)
        copy, up = self._copy_stream, self._upload_stream
        main = torch.cuda.current_stream(self.device)
        pending = collections.deque()
        for inputs in batches:
            total = inputs[0].shape[0]
            lo, hi = shard_bounds(total, world, rank)
            local = [i[lo:hi] if i.dim() > 0 and i.shape[0] == total else i for i in inputs]
            if any(not i.is_cuda for i in local):    # uploads have a stream of their own too: they run under the previous batch's kernels
                with torch.cuda.stream(up):
                    local = [i if i.is_cuda else i.to(self.device, non_blocking=True) for i in local]
                    uploaded = torch.cuda.Event()
                    uploaded.record(up)
                main.wait_event(uploaded)
                for i in local:
                    i.record_stream(main)
            out = self.fn(*local)
            if isinstance(out, (list, tuple)):
                out = out[0]
            full, token = self.gather(out, total)
            wants_full = self.host_result_ranks is None or rank in self.host_result_ranks
            src = full if wants_full else out
            key = (tuple(src.shape), src.dtype)
            ring = self._ring.setdefault(key, {"bufs": [], "next": 0})
            while len(ring["bufs"]) < depth + 1:
                ring["bufs"].append(torch.empty(src.shape, dtype=src.dtype, pin_memory=True))
            host = ring["bufs"][ring["next"] % (depth + 1)]
            ring["next"] += 1
            ready, done = torch.cuda.Event(), torch.cuda.Event()
            ready.record(main)
            copy.wait_event(ready)
            with torch.cuda.stream(copy):
                host.copy_(src, non_blocking=True)
                done.record(copy)
            src.record_stream(copy)          # the allocator must not hand the result's memory out again before the copy has read it
            if token is not None and wants_full:
                token[0]["guard"][token[1]] = done   # ... nor may the peers overwrite the gather buffer before that
            pending.append((done, host))
            if len(pending) >= depth:
                d, h = pending.popleft()
                d.synchronize()
                yield h
        while pending:
            d, h = pending.popleft()
            d.synchronize()
            yield h
