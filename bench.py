#!/usr/bin/env python
"""Headline benchmark: GPT-2-medium data-parallel training step over this
library's torch.distributed backend (25 MB gradient buckets, bf16, random
weights, random tokens), plus a bus-bandwidth probe of the all-reduce kernel.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Rank 0 prints ONE JSON line. ``value`` is whole-job tokens/s, device-timed
(CUDA events, max over ranks) over exactly ``--steps`` steps; ``e2e`` repeats
the measurement through ``DDPTrainer.step`` with a host-to-device copy of the
batch from pinned memory and a device-to-host read of the loss every step.
``--impl reference`` is the arm for the reference implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REF_UNAVAILABLE = ("the reference cannot run this configuration on this image: it is not a Python project (pip install of the tree: "
                   "'Neither setup.py nor pyproject.toml found'), its multipath build libampccl_nccl.so does not compile against its "
                   "CUDA PCCL ('pcclDataType_t has not been declared'), and its only PyTorch route, LD_PRELOAD=libpccl.so under "
                   "backend=nccl, stops at communicator set-up on a B200 box ('sysfs reports invalid NUMA node -1', then with "
                   "PCCL_GPU_NUMA_MAP 'NCCL error invalid argument, NCCL version 2.17.1' under PyTorch 2.11); record: "
                   "profiles/reference_arm_probe.md")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.rows = []
        self.proc = None
        self.thread = None
        self.t_begin = self.t_end = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        import datetime as _dt

        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                ts = _dt.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                # samples outside the timed region (warm-up, set-up) are not evidence about it
                if self.t_begin and self.t_end and not (self.t_begin - 0.05 <= ts <= self.t_end + 0.25):
                    continue
            except ValueError:
                pass
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_arm(backend: str, args, tokens_shape):
    """Builds the model on `backend`, returns (device ms/step, e2e ms/step, launches, loss, stats)."""
    import torch
    import torch.distributed as dist

    from hylink_b200.models.gpt2 import GPT2, GPT2Config
    from hylink_b200.parallel.trainer import DDPTrainer, init_distributed

    rank, world, dev = init_distributed(backend)
    torch.manual_seed(1234)
    cfg = GPT2Config.by_name(args.model)
    trainer = DDPTrainer(GPT2(cfg), dev, bucket_cap_mb=args.bucket_mb)
    batch, seq = tokens_shape
    g = torch.Generator().manual_seed(100 + rank)
    host_tokens = [torch.randint(0, cfg.vocab_size, (batch, seq + 1), generator=g).pin_memory() for _ in range(4)]
    dev_tokens = [t.to(dev) for t in host_tokens]

    def stats():
        if backend != "hylink":
            return {}
        from hylink_b200.parallel import backend_stats

        return backend_stats()

    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: start it before the warm-up
    for i in range(args.warmup):
        t = dev_tokens[i % len(dev_tokens)]
        trainer.step_device(t[:, :-1], t[:, 1:])
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sampler.mark_begin()
    before = stats().get("kernel_launches", 0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = None
    for i in range(args.steps):
        t = dev_tokens[i % len(dev_tokens)]
        loss = trainer.step_device(t[:, :-1], t[:, 1:])
    e1.record()
    torch.cuda.synchronize()
    sampler.mark_end()
    dist.barrier()
    torch.cuda.synchronize()
    dev_ms = e0.elapsed_time(e1) / args.steps
    launches = stats().get("kernel_launches", 0) - before
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the public trainer API: pinned H2D of the batch and D2H of the loss every step
    for i in range(2):
        trainer.step(host_tokens[i % len(host_tokens)])
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        last = trainer.step(host_tokens[i % len(host_tokens)])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    both = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(both, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(both[0]), float(both[1])
    final_stats = stats()
    del trainer
    torch.cuda.empty_cache()
    return dev_ms, e2e_ms, launches, float(last), clocks, final_stats, host_tokens[0].numel() * host_tokens[0].element_size()


def allreduce_probe(world: int):
    """busbw of a 64 MiB bf16 all-reduce on the library's communicator vs the NCCL group (device-timed, max over ranks)."""
    import torch
    import torch.distributed as dist

    from hylink_b200.utils.sweep import bus_factor, time_op

    out = {}
    if world < 2:
        return out
    n = (64 << 20) // 2
    pool = torch.randn(4 * n, device="cuda").to(torch.bfloat16)
    for name, group in (("hylink", None), ("nccl", dist.new_group(backend="nccl"))):
        fn = lambda i, g=group: dist.all_reduce(pool[i * n:(i + 1) * n], group=g)
        ms = time_op(fn, 4, 10, 3)
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name + "_busbw_GBs"] = round(n * 2 / float(t[0]) / 1e6 * bus_factor("allreduce", world), 1)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hylink", choices=["hylink", "reference", "nccl"])
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--no-nccl-arm", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    import torch
    import torch.distributed as dist

    backend = "hylink" if args.impl == "hylink" else "nccl"
    dev_ms, e2e_ms, launches, loss, clocks, stats, h2d = run_arm(backend, args, (args.micro_batch, args.seq))
    tokens = args.micro_batch * args.seq * world
    probe = allreduce_probe(world) if backend == "hylink" else {}
    if rank == 0:
        rec = {
            "metric": "gpt2_medium_ddp_tokens_per_s", "value": round(tokens / dev_ms * 1e3, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": args.micro_batch * world, "seq_len": args.seq,
                       "parallelism": f"dp{world}", "bucket_mb": args.bucket_mb, "backend": backend,
                       "l2_policy": "working set larger than L2: 0.7 GB of bf16 weights plus activations are re-read every step",
                       "optimizer": "fused AdamW inside the timed region"},
            "clocks": clocks,
            "e2e": {"value": round(tokens / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "loss": round(loss, 4),
            "comm": {k: stats.get(k) for k in ("nvls", "symm_mode", "calls", "nvl_bytes", "pcie_bytes", "kernel_launches")},
            "allreduce_64MiB_bf16": probe,
        }
        print(json.dumps(rec), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
