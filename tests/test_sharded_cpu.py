"""Batch sharding across ranks, exercised with two gloo processes on the CPU: every rank compiles
the same model (plans run on the CPU oracle interpreter here), runs its slice of the batch through
the symbolic-batch plan and all-gathers; the result must equal the full-batch eager output."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llcompiler_b200.executor import shard_bounds


def test_shard_bounds_cover_the_batch():
    for total in (0, 1, 7, 64, 257):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank, world, port, total, q):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import InterpreterCompiler, compile_with
        from llcompiler_b200.executor import BatchShardedRunner
        from oracle.models import build_model
        model = build_model("mlp")
        x = torch.randn(total, 784, generator=torch.Generator().manual_seed(5))
        comp = InterpreterCompiler()
        fn = compile_with(comp, model, dynamic=True)
        runner = BatchShardedRunner(fn)
        with torch.no_grad():
            got = runner(x)
            want = model(x)
        q.put((rank, tuple(got.shape), float((got - want).abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total", [(2, 64), (2, 7), (8, 64), (8, 20)])
def test_ranks_gather_the_full_batch(world, total):
    # eight ranks also compile the same graph at the same time through one cache directory, as the ranks of an 8-GPU job do
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 1000) + total + 100 * world
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, shape, err in results:
        assert shape == (total, 10) and err < 1e-4


def test_pipelined_refuses_what_it_cannot_do():
    from llcompiler_b200.executor import BatchShardedRunner
    r = BatchShardedRunner(lambda x: x)
    with pytest.raises(ValueError):
        next(r.pipelined([(torch.zeros(2, 2),)]))          # no device: the pipelined call needs CUDA streams
    with pytest.raises(ValueError):
        BatchShardedRunner(lambda x: x, gather="ring")      # only "nccl" and "peer"
    # without a process group the gather of a one-rank "group" is the local tensor itself, whatever the mode asked for
    t = torch.arange(6.0).view(3, 2)
    got, token = BatchShardedRunner(lambda x: x, gather="peer").gather(t, 3)
    assert got is t and token is None
