#!/usr/bin/env python
"""Benchmark of the compiled-model inference path.

  python bench.py --gpus N --steps K --warmup W [--config bert] [--impl reference]

A step is one forward of the configured model over one GLOBAL batch of seeded synthetic input.  The default workload
is the largest single-GPU configuration, BERT-base x12 bf16 on ids[256,384].  At N > 1 (one rank per GPU, launched with
torch.distributed.run) the global batch is split evenly over the ranks (strong scaling: 256 -> 256/N per GPU) by
llcompiler_b200.executor.BatchShardedRunner: weights replicated, every rank runs its slice, the outputs are
all-gathered over NCCL inside the timed step.  The line printed by rank 0 carries:
  value      samples/s with inputs resident in HBM, device-timed with CUDA events, max over ranks
  e2e        the same metric with page-locked HOST tensors in and out, the host->device and device->host copies
             inside the timed region: K batches through BatchShardedRunner.pipelined (two in flight: every rank uploads
             its slice, runs it, the gather follows, rank 0 reads the gathered batch back on a copy stream while the
             next batch computes); `one_batch_at_a_time` is the same K batches through the plain call, each finished
             before the next starts (N = 1: Torch_ExecutionEngine.run on host tensors, i.e. the C ABI's host path)
  roofline   the dominant kernel family (GEMM / convolution): algorithmic FLOPs / CUDA-event duration of its launches
  cpu_baseline  the CPU oracle (PyTorch CPU eager fp32, what the reference pins itself to) on a bounded sample of
             the same workload, on this box's host cores; N = 1 only
`--impl reference` times that CPU path alone with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (oracle config, global batch, extra make_inputs kwargs, dtype label, precision option)
    "mlp": ("mlp", 64, {}, "f32", "auto"),
    "resnet18": ("resnet18", 32, {}, "f32", "tf32x3"),      # fp32 storage, three-pass TF32 on tensor cores (1e-4)
    "encoder128": ("encoder", 8, {"seq": 128}, "f32", "tf32"),  # the configuration names TF32 matmuls (2e-2)
    "encoder512": ("encoder", 8, {"seq": 512}, "f32", "tf32"),
    "resnet50": ("resnet50", 256, {}, "bf16", "auto"),
    "bert": ("bert", 256, {}, "bf16", "auto"),
}
DEFAULT_WORKLOAD = "bert"      # the largest configuration that fits one GPU
DESCRIPTION = {
    "resnet18": "ResNet-18 fp32 NCHW [32,3,224,224] (configs[1])",
    "mlp": "MLP 784-512-10 fp32 B=64 (configs[0])",
    "encoder128": "pre-LN encoder layer d768 h12 [8,128,768] (configs[2], S=128)",
    "encoder512": "pre-LN encoder layer d768 h12 [8,512,768] (configs[2], S=512)",
    "resnet50": "ResNet-50 bf16 [256,3,224,224] (configs[3])",
    "bert": "BERT-base x12 bf16 ids[256,384] (configs[4])",
}


# DRAM bytes per launch of the dominant kernel family (dram__bytes_read.sum + dram__bytes_write.sum averaged over the
# launches of one forward), from an ncu capture of this command (20 tensor-core launches of one forward).
NCU_TRAFFIC = {("resnet18", "conv", 32): 23.0e6,
               # the four GEMMs of a BERT layer at 98304 rows: 2304x768 (557.2 MB), 768x768 (258.8 MB), 3072x768 (708.0 MB),
               # 768x3072 (743.1 MB)
               ("bert", "gemm", 256): 566.8e6}


def config_dict(name: str, batch: int, world: int, prec: str) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": DESCRIPTION[name], "global_batch": batch, "per_gpu_batch": batch // world,
            "parallelism": f"batch split over {world} GPU(s), weights replicated, outputs all-gathered",
            "l2": "flushed between timed iterations (256 MB write)", "precision": prec}
# Share of the measured bf16 peak a precision can reach at best: tf32 MMAs run at half the bf16 rate, tf32x3 issues
# three of them per algorithmic multiply-add.
PRECISION_CEILING = {"bf16": 1.0, "auto": 1.0, "tf32": 0.5, "tf32x3": 1.0 / 6.0, "fp32": None}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 6 and f[0].isdigit():
                self.samples.append(f)

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons}


def build_workload(name: str, batch: int, kw: dict):
    from oracle.models import CONFIGS, build_model
    cfg = CONFIGS[name]
    model = build_model(name)
    inputs = cfg.make_inputs(batch=batch, **kw)
    return cfg, model, inputs


def cpu_oracle_rate(model, inputs, batch: int, budget_s: float, threads: int, sample_batch: int):
    """samples/s of PyTorch CPU eager fp32 on a bounded sample of the workload."""
    torch.set_num_threads(threads)
    sub = tuple(i[:sample_batch] for i in inputs)
    with torch.no_grad():
        model(*sub)
        t0 = time.perf_counter()
        n = 0
        while True:
            model(*sub)
            n += 1
            dt = time.perf_counter() - t0
            if dt > budget_s or n >= 50:
                break
    return sample_batch * n / dt, n, dt


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    oname, batch, kw, dtype, prec = WORKLOADS[args.config]
    cfg, model, inputs = build_workload(oname, batch, kw)
    threads = os.cpu_count() or 1
    sample_batch = min(batch, 8 if oname in ("resnet50", "bert") else batch)
    if oname == "bert":
        sample_batch = 2
    torch.set_num_threads(threads)
    sub = tuple(i[:sample_batch] for i in inputs)
    times = []
    with torch.no_grad():
        for _ in range(max(args.warmup, 1)):
            model(*sub)
        for _ in range(args.steps):
            t0 = time.perf_counter()
            model(*sub)
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = sample_batch * args.steps / total
    sample = f"{args.steps} forwards of a {sample_batch}-sample slice of the batch, PyTorch CPU eager fp32 (the reference's own parity pin; its CPU lowering cannot be built offline)"
    line = {
        "impl": "reference", "metric": "inferences_per_sec", "value": value, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,      # one step = one forward of the sample, see cpu_baseline.sample
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.config, batch, max(args.gpus, 1), args.precision or prec),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--precision", default=None)
    ap.add_argument("--gather", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: this library's peer-store gather or NCCL's all_gather; auto = peer up to 4 GPUs (the sizes it was "
                         "measured at), NCCL above")
    ap.add_argument("--steps-out", default=None, help="write the per-plan-step CUDA-event table here")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    from __graft_entry__ import build
    if rank == 0:
        build()
    import torch.distributed as dist
    dev = torch.device("cuda", local if world > 1 else 0)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    from llcompiler_b200.compiler import LLCompiler
    from llcompiler_b200.executor import BatchShardedRunner, shard_bounds

    oname, batch, kw, dtype, prec = WORKLOADS[args.config]
    prec = args.precision or prec
    if batch % world:
        raise SystemExit(f"the global batch of {batch} does not split evenly over {world} GPUs")
    cfg, model, inputs = build_workload(oname, batch, kw)
    lo, hi = shard_bounds(batch, world, rank)
    import copy
    gmodel = copy.deepcopy(model)
    if dtype == "bf16":
        gmodel = gmodel.to(torch.bfloat16)
    gmodel = gmodel.to(dev)
    cast = (lambda t: t.to(torch.bfloat16)) if dtype == "bf16" else (lambda t: t)
    host_inputs = tuple((cast(i) if i.is_floating_point() else i).contiguous().pin_memory() for i in inputs)   # the global batch
    dev_inputs = tuple(i.to(dev) for i in host_inputs)

    comp = LLCompiler(precision=prec, device=dev.index)
    torch._dynamo.reset()
    fn = torch.compile(gmodel, backend=comp, dynamic=False, fullgraph=True)
    with torch.no_grad():
        out = fn(*(i[lo:hi] for i in dev_inputs))          # compiled for this rank's slice
    torch.cuda.synchronize()
    eng = comp.compiled[0].engine
    launches_per_step = eng.executor.last_launch_count()
    gather_mode = "nccl" if world == 1 else (("peer" if world <= 4 else "nccl") if args.gather == "auto" else args.gather)
    # N > 1: the gather is this library's own kernel (every rank stores its slice into every rank's buffer over NVLink);
    # it is checked against NCCL's all_gather once, on this step's real output, before anything is timed
    runner = BatchShardedRunner(lambda *a: eng.run(*a), device=dev, host_result_ranks=(0,), gather=gather_mode)
    if gather_mode == "peer":
        from llcompiler_b200.executor.sharded import gather_batch
        with torch.no_grad():
            local_out = eng.run(*(i[lo:hi] for i in dev_inputs))[0]
        want_full = gather_batch(local_out, batch)
        got_full, _ = runner.gather(local_out, batch)
        torch.cuda.synchronize()
        assert torch.equal(got_full, want_full), "the peer-store gather differs from NCCL's all_gather"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2

    for _ in range(args.warmup):                # the executor captures its CUDA graph on the second of these calls
        full = runner(*dev_inputs)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(dev.index) as clocks:
        torch.cuda.synchronize()
        for i in range(args.steps):
            flush.zero_()                       # evict L2 between timed iterations (outside the timed span)
            starts[i].record()
            full = runner(*dev_inputs)          # this rank's slice + the all-gather of every rank's outputs
            ends[i].record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        total_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
        # end to end: page-locked host inputs, host outputs, copies inside the timed region
        for _ in range(2):
            runner(*host_inputs)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            o_host = runner(*host_inputs)
        torch.cuda.synchronize()
        e2e_sync_s = time.perf_counter() - t0
        # the same K steps through the runner's pipelined call: two batches in flight, the device-to-host copy of one
        # under the kernels of the next; every copy still lies inside the timed region
        for o_host in runner.pipelined((host_inputs for _ in range(2)), depth=2):
            pass
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for o_host in runner.pipelined((host_inputs for _ in range(args.steps)), depth=2):
            pass
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    eng.status()                                # raises if any kernel of the run reported a failure
    assert tuple(full.shape)[0] == batch and not o_host.is_cuda
    t = torch.tensor([total_ms, e2e_s * 1e3, e2e_sync_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, e2e_sync_ms = float(t[0]), float(t[1]), float(t[2])

    # dominant kernel: event-timed per kernel family over a profiled pass (events around every launch)
    local_dev_inputs = tuple(i[lo:hi] for i in dev_inputs)
    prof = eng.profile(*local_dev_inputs, reps=5)
    if args.steps_out and rank == 0:
        with open(args.steps_out, "w") as f:
            f.write("# step kernel ms GFLOP MB  TFLOP/s GB/s\n")
            for r in eng.last_profile_steps:
                f.write(f"{r['index']:4d} {r['kernel']:10s} {r['ms']:9.4f} {r['flops'] / 1e9:10.3f} {r['bytes'] / 1e6:10.2f} "
                        f"{r['flops'] / max(r['ms'], 1e-9) / 1e9:9.1f} {r['bytes'] / max(r['ms'], 1e-9) / 1e6:9.1f}\n")
    roof = None
    pk = peaks()
    if prof:
        pass_ms = max(sum(r["ms"] for r in prof), 1e-9)
        top = max(prof, key=lambda r: r["ms"])
        common = {"kernel": top["kernel"], "peak_source": pk["source"], "launches": top["launches"],
                  "ms_per_launch": top["ms"] / max(top["launches"], 1),
                  # both figures come from the same pass: events around every launch of one forward, 5 repetitions
                  "share_of_profiled_pass": top["ms"] / pass_ms, "profiled_pass_ms": pass_ms,
                  "traffic": NCU_TRAFFIC.get((args.config, top["kernel"], batch // world))}
        if top["flops"] > 0 and top["kernel"] in ("conv", "gemm", "attention"):
            achieved = top["flops"] / (top["ms"] * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                    "frac_of_sustained_peak": achieved / pk["tflops_sustained"] if pk.get("tflops_sustained") else None,
                    "precision_ceiling_frac": PRECISION_CEILING.get(prec), **common}
        else:
            achieved = top["bytes"] / (top["ms"] * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], **common}
        roof["families"] = {r["kernel"]: {"launches": r["launches"], "ms": round(r["ms"], 4),
                                          "tflops": round(r["flops"] / max(r["ms"], 1e-9) / 1e9, 1), "gbs": round(r["bytes"] / max(r["ms"], 1e-9) / 1e6, 1)}
                            for r in prof}

    if rank == 0:
        cpu = None
        if world == 1:          # the other ranks of a multi-GPU run would spin in a barrier meanwhile: N = 1 only
            cpu_val, cpu_n, cpu_dt = cpu_oracle_rate(model, inputs, batch, args.cpu_budget, os.cpu_count() or 1,
                                                     2 if oname == "bert" else (8 if oname == "resnet50" else batch))
            cpu = {"value": cpu_val, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "port",
                   "sample": f"{cpu_n} forwards in {cpu_dt:.1f} s, PyTorch CPU eager fp32 (CPU oracle)"}
        h2d = sum(i.numel() * i.element_size() for i in host_inputs)           # every rank uploads its slice: the whole batch
        d2h = full.numel() * full.element_size()                               # rank 0 reads the gathered batch back
        line = {
            "metric": "inferences_per_sec", "value": batch * args.steps / (total_ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": config_dict(args.config, batch, world, prec),
            "clocks": clocks.summary(),
            "e2e": {"value": batch * args.steps / (e2e_ms * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "call": "BatchShardedRunner.pipelined(depth=2): two batches in flight",
                    "one_batch_at_a_time": batch * args.steps / (e2e_sync_ms * 1e-3)},
            # this library's kernels inside the timed region: the plan's launches, plus the gather's push kernel at N > 1
            "gpu_launches": int((launches_per_step + (1 if world > 1 and runner.gather_mode == "peer" else 0)) * args.steps),
            "gather": ("none (one GPU)" if world == 1 else
                       "llc_cuda_push_rows: peer stores over NVLink into symmetric memory, checked against NCCL all_gather" if runner.gather_mode == "peer"
                       else "NCCL all_gather_into_tensor" + (f" (peer gather unavailable: {runner.gather_fallback})" if runner.gather_fallback else "")),
            "roofline": roof,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
