#!/usr/bin/env python
"""Headline benchmark: bus bandwidth of all-reduce, reduce-scatter and all-gather against message size.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

The collectives are issued through the product API — ``torch.distributed`` on
this library's ``hylink`` backend — on bf16 buffers of 1 MiB to 1 GiB (powers
of two; the size is the nccl-tests message size: the whole buffer for
all-reduce, all n segments for reduce-scatter and all-gather). One *step* is
one pass over the whole table (33 cells), every cell bracketed by its own pair
of CUDA events; a cell's time is its mean over the timed steps, max over ranks.
``value`` is the geometric mean of the bus bandwidth over all cells
(busbw = bytes / time * 2(n-1)/n for all-reduce, * (n-1)/n for the other two;
with one GPU the factor is 1). The same cells are timed on a NCCL process group
in the same run (``nccl`` column), and the per-cell table, the split ratio and a
GPT-2-medium DDP training step are reported as extra keys.

``e2e`` repeats the table with, inside the timed region of every cell, the copy
of the cell's input from pinned host memory to the device and a copy of the
first 4 KiB of the result back to the host (wall clock around stream
synchronisation).

``--impl reference`` times the same cells on the unmodified reference library
(``baseline/reference_arm.py``); ``--impl nccl`` on NCCL alone.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "allreduce/RS/AG busbw GB/s vs size (geomean over 1 MiB-1 GiB cells, max over ranks)"
COLLS = ("allreduce", "reducescatter", "allgather")


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


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mul = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}.get(s[-1], 1)
    return int(float(s[:-1]) * mul) if s[-1] in "KMG" else int(s)


def size_list(lo: int, hi: int):
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= 2
    return out


def bus_factor(coll: str, n: int) -> float:
    if n <= 1:
        return 1.0
    return 2.0 * (n - 1) / n if coll == "allreduce" else (n - 1) / n


def geomean(xs):
    xs = [x for x in xs if x and x > 0]
    return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else 0.0


def human(nbytes: int) -> str:
    for unit, sh in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if nbytes >= 1 << sh:
            return f"{nbytes >> sh} {unit}"
    return f"{nbytes} B"


# --------------------------------------------------------------------------- the sweep through torch.distributed
class Table:
    """Buffers and the per-cell calls of one process group."""

    def __init__(self, dtype, sizes, world, group=None, registered=False):
        import torch

        self.torch = torch
        self.registered = registered
        self.dtype, self.sizes, self.world, self.group = dtype, sizes, world, group
        self.es = torch.empty((), dtype=dtype).element_size()
        self.cells = [(c, s) for c in COLLS for s in sizes]
        self._views = {}
        top = max(sizes)
        self.slots = 2
        # rotating buffers: between two timed calls of one cell a whole pass (> 4 GiB of traffic) goes through L2
        if registered:
            # the library's allocator (hylink_b200.parallel.symmetric_empty): registered memory, collectives run zero-copy
            from hylink_b200.parallel import symmetric_empty

            import torch.distributed as dist

            try:
                self.inp = [symmetric_empty(top // self.es, dtype) for _ in range(self.slots)]
                self.out = [symmetric_empty(top // self.es, dtype) for _ in range(self.slots)]
                ok = 1
            except RuntimeError as e:   # no registered heap on this machine (no peer mapping, out of address space ...)
                print(f"[bench] registered memory unavailable on rank {dist.get_rank()}: {e}", file=sys.stderr, flush=True)
                self.inp = self.out = None
                ok = 0
            # all ranks use registered buffers or none does: the buffers must sit at the same heap offset everywhere
            agree = torch.tensor([ok], device="cuda", dtype=torch.int32)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=group)
            if int(agree.item()) == 0:
                self.inp = self.out = None
                self.registered = False
        if self.registered:
            for t in self.inp:
                t.copy_((torch.rand(top // self.es, device="cuda") * 2 - 1).to(dtype))
        else:
            self.inp = [(torch.rand(top // self.es, device="cuda") * 2 - 1).to(dtype) for _ in range(self.slots)]
            self.out = [torch.empty(top // self.es, dtype=dtype, device="cuda") for _ in range(self.slots)]

    def elems(self, nbytes):
        n_el = max(self.world, (nbytes // self.es) // self.world * self.world)
        return n_el, n_el // self.world

    def input_bytes(self, coll, nbytes):
        n_el, seg = self.elems(nbytes)
        return (seg if coll == "allgather" else n_el) * self.es

    def call(self, coll, nbytes, it):
        import torch.distributed as dist

        # the views of a cell are made once: slicing a tensor costs a microsecond or two of host time, which is all
        # there is to a collective of one rank
        key = (coll, nbytes, it % self.slots)
        v = self._views.get(key)
        if v is None:
            n_el, seg = self.elems(nbytes)
            a, b = self.inp[it % self.slots], self.out[it % self.slots]
            v = self._views[key] = (a, b, a[:n_el], a[:seg], b[:n_el], b[:seg])
        a, b, a_all, a_seg, b_all, b_seg = v
        if coll == "allreduce":
            dist.all_reduce(a_all, group=self.group)        # in place, as torch.distributed defines it
            return a
        if coll == "reducescatter":
            dist.reduce_scatter_tensor(b_seg, a_all, group=self.group)
            return b
        dist.all_gather_into_tensor(b_all, a_seg, group=self.group)
        return b


def timed_passes(tab: Table, steps: int, warmup: int, launches=None):
    """W warm-up and K timed passes; returns (per-cell mean ms on this rank, device ms of the K passes, launches)."""
    import torch
    import torch.distributed as dist

    for it in range(warmup):
        for coll, nbytes in tab.cells:
            tab.call(coll, nbytes, it)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    before = launches() if launches else 0
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in tab.cells] for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for it in range(steps):
        for ci, (coll, nbytes) in enumerate(tab.cells):
            ev[it][ci][0].record()
            tab.call(coll, nbytes, warmup + it)
            ev[it][ci][1].record()
    t1.record()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    after = launches() if launches else 0
    per_cell = [sum(ev[it][ci][0].elapsed_time(ev[it][ci][1]) for it in range(steps)) / steps for ci in range(len(tab.cells))]
    tab.last_min_ms = [min(ev[it][ci][0].elapsed_time(ev[it][ci][1]) for it in range(steps)) for ci in range(len(tab.cells))]
    return per_cell, t0.elapsed_time(t1), after - before


def e2e_passes(tab: Table, steps: int):
    """Per-cell wall ms with the H2D copy of the input and a D2H read of the result inside the timed region."""
    import torch
    import torch.distributed as dist

    top = max(tab.sizes)
    host = torch.empty(top // tab.es, dtype=tab.dtype).pin_memory()
    host.uniform_(-1, 1)
    back = torch.empty(4096 // tab.es, dtype=tab.dtype).pin_memory()
    sums = [0.0] * len(tab.cells)
    stream = torch.cuda.current_stream()
    # views made once per (cell, buffer slot): the timed region holds the copies and the call, not tensor slicing
    plan = {}
    for ci, (coll, nbytes) in enumerate(tab.cells):
        n_el, seg = tab.elems(nbytes)
        k = seg if coll == "allgather" else n_el
        for slot in range(tab.slots):
            res = tab.inp[slot] if coll == "allreduce" else tab.out[slot]
            plan[(ci, slot)] = (tab.inp[slot][:k], host[:k], res[:back.numel()])
    for it in range(2 + steps):
        for ci, (coll, nbytes) in enumerate(tab.cells):
            if it == 2 and ci == 0:
                torch.cuda.synchronize()
                dist.barrier()
                torch.cuda.synchronize()
            dst, src, res = plan[(ci, it % tab.slots)]
            t0 = time.perf_counter()
            dst.copy_(src, non_blocking=True)
            tab.call(coll, nbytes, it)
            back.copy_(res, non_blocking=True)
            stream.synchronize()
            if it >= 2:
                sums[ci] += (time.perf_counter() - t0) * 1e3
    h2d = sum(tab.input_bytes(c, s) for c, s in tab.cells)
    return [x / steps for x in sums], h2d, 4096 * len(tab.cells)


def max_over_ranks(values, group=None):
    import torch
    import torch.distributed as dist

    t = torch.tensor(values, device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]


# --------------------------------------------------------------------------- extra: the DDP training step
def ddp_step(args, backend: str):
    import torch
    import torch.distributed as dist

    from hylink_b200.models.gpt2 import GPT2, GPT2Config
    from hylink_b200.parallel.trainer import DDPTrainer

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1234)
    cfg = GPT2Config.by_name(args.model)
    trainer = DDPTrainer(GPT2(cfg), dev, bucket_cap_mb=args.bucket_mb)
    g = torch.Generator().manual_seed(100 + rank)
    host_tokens = [torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq + 1), generator=g).pin_memory() for _ in range(4)]
    dev_tokens = [t.to(dev) for t in host_tokens]
    steps = args.ddp_steps
    for i in range(3):
        t = dev_tokens[i % 4]
        trainer.step_device(t[:, :-1], t[:, 1:])
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        t = dev_tokens[i % 4]
        trainer.step_device(t[:, :-1], t[:, 1:])
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    dev_ms = e0.elapsed_time(e1) / steps
    for i in range(2):
        trainer.step(host_tokens[i % 4])
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    loss = 0.0
    for i in range(steps):
        loss = trainer.step(host_tokens[i % 4])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    dev_ms, e2e_ms = max_over_ranks([dev_ms, e2e_ms])
    tokens = args.micro_batch * args.seq * world
    trainer.close()
    del trainer
    torch.cuda.empty_cache()
    return {"model": args.model, "backend": backend, "tokens_per_s": round(tokens / dev_ms * 1e3, 1), "ms_per_step": round(dev_ms, 3),
            "e2e_tokens_per_s": round(tokens / e2e_ms * 1e3, 1), "steps": steps, "micro_batch": args.micro_batch, "seq_len": args.seq,
            "bucket_mb": args.bucket_mb, "loss": round(float(loss), 4), "dtype": "bf16"}


# --------------------------------------------------------------------------- arms
def reference_arm(args, rank: int, world: int) -> int:
    """The unmodified reference, thread-per-GPU in rank 0's process (its single-process mode); other ranks stand by."""
    if rank != 0:
        return 0
    sizes = size_list(parse_size(args.lo), parse_size(args.hi))
    n = args.gpus
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm as ref

        sampler = ClockSampler(0)
        sampler.start()
        sampler.mark_begin()
        res = ref.run(n, args.steps, args.warmup, COLLS, sizes, e2e=True)
        sampler.mark_end()
        clocks = sampler.stop()
    except Exception as ex:  # noqa: BLE001 - whatever stopped the reference is the answer
        msg = " ".join(f"{type(ex).__name__}: {ex}".split())
        print(json.dumps({"impl": "reference", "unavailable": msg[:600], "n_gpus": n}), flush=True)
        return 0
    cells = res["cells"]
    table, bw, bw_e2e = [], [], []
    for i, (coll, nbytes) in enumerate(cells):
        f = bus_factor(coll, n)
        b = nbytes / res["dev_ms"][i] / 1e6 * f
        e = nbytes / res["e2e_ms"][i] / 1e6 * f
        bw.append(b)
        bw_e2e.append(e)
        table.append({"coll": coll, "bytes": nbytes, "ms": round(res["dev_ms"][i], 4), "busbw_GBs": round(b, 2), "e2e_busbw_GBs": round(e, 2)})
    h2d = sum((s // n if c == "allgather" else s) for c, s in cells)
    rec = {"metric": METRIC, "value": round(geomean(bw), 3), "unit": "GB/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": round(sum(res["dev_ms"]), 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "fp32 (the reference's public API reduces fp32 only; same byte sizes as the bf16 cells)", "data": "synthetic",
           "impl": "reference",
           "config": {"model": "collective sweep", "collectives": list(COLLS), "bytes": [sizes[0], sizes[-1]], "global_batch": None,
                      "seq_len": None, "parallelism": f"{n} ranks as threads of one process (the reference's single-process mode)",
                      "library": "baseline/_ref/libpccl.so through pcclAllReduce / pcclReduceScatter / pcclAllGather"
                      if n > 1 else "baseline/_ref/libpccl.so through its ncclAllReduce / ncclReduceScatter / ncclAllGather (one rank)",
                      "l2_policy": "two rotating buffer pairs of 1 GiB; a whole pass over the table lies between two timed calls of a cell"},
           "clocks": clocks,
           "e2e": {"value": round(geomean(bw_e2e), 3), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4096 * len(cells)},
           "table": table, "wall_s": round(res["wall_s"], 1)}
    print(json.dumps(rec), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hylink", choices=["hylink", "reference", "nccl"])
    ap.add_argument("--bytes-from", dest="lo", default="1M")
    ap.add_argument("--bytes-to", dest="hi", default="1G")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32", "fp16"])
    ap.add_argument("--no-nccl-arm", action="store_true", help="skip the NCCL column")
    ap.add_argument("--no-ddp", action="store_true", help="skip the GPT-2-medium DDP step")
    ap.add_argument("--unregistered", action="store_true", help="headline on ordinary torch tensors (staged) instead of registered memory")
    ap.add_argument("--ddp-only", action="store_true", help="only the GPT-2-medium DDP step (prints its record alone)")
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--ddp-steps", type=int, default=10)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        return reference_arm(args, rank, world)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    import torch
    import torch.distributed as dist

    from hylink_b200.parallel.trainer import init_distributed

    backend = "hylink" if args.impl == "hylink" else "nccl"
    rank, world, dev = init_distributed(backend)
    if args.ddp_only:
        rec = ddp_step(args, backend)
        if rank == 0:
            print(json.dumps({"metric": "gpt2_medium_ddp_tokens_per_s", "impl": args.impl, "n_gpus": world, **rec}), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return 0
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[args.dtype]
    sizes = size_list(parse_size(args.lo), parse_size(args.hi))
    registered = backend == "hylink" and not args.unregistered and world > 1
    tab = Table(dtype, sizes, world, registered=registered)
    registered = tab.registered   # False when the machine could not provide registered memory

    def stats():
        if backend != "hylink":
            return {}
        from hylink_b200.parallel import backend_stats

        return backend_stats()

    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to come up: start it before the warm-up
        sampler.mark_begin()
    launches = (lambda: stats().get("kernel_launches", 0)) if backend == "hylink" else None
    cell_ms, region_ms, n_launch = timed_passes(tab, args.steps, args.warmup, launches)
    cell_min_ms = list(tab.last_min_ms)
    alpha = stats().get("last_alpha", 0.0)
    cell_ms = max_over_ranks(cell_ms)
    region_ms = max_over_ranks([region_ms])[0]

    nccl_ms = None
    if backend == "hylink" and not args.no_nccl_arm:
        nccl_group = dist.new_group(backend="nccl")
        ntab = Table(dtype, sizes, world, group=nccl_group)
        ntab.inp, ntab.out = tab.inp, tab.out
        nccl_ms, _, _ = timed_passes(ntab, args.steps, args.warmup)
        nccl_ms = max_over_ranks(nccl_ms)
        del ntab

    e2e_ms, h2d, d2h = e2e_passes(tab, args.steps)
    e2e_ms = max_over_ranks(e2e_ms)
    staged_ms = None
    if registered:
        # the same cells on ordinary torch tensors: every byte goes through the library's staging region
        ptab = Table(dtype, sizes, world)
        staged_ms, _, _ = timed_passes(ptab, args.steps, args.warmup)
        staged_ms = max_over_ranks(staged_ms)
        del ptab
    if rank == 0:
        sampler.mark_end()   # the clocks cover all timed passes: this library's, NCCL's and the end-to-end ones
    clocks = sampler.stop() if rank == 0 else None

    table, bw, bw_nccl, bw_e2e = [], [], [], []
    for i, (coll, nbytes) in enumerate(tab.cells):
        n_el, _ = tab.elems(nbytes)
        real = n_el * tab.es
        f = bus_factor(coll, world)
        b = real / cell_ms[i] / 1e6 * f
        e = real / e2e_ms[i] / 1e6 * f
        row = {"coll": coll, "bytes": real, "ms": round(cell_ms[i], 4), "ms_min_rank0": round(cell_min_ms[i], 4), "busbw_GBs": round(b, 2),
               "e2e_busbw_GBs": round(e, 2)}
        bw.append(b)
        bw_e2e.append(e)
        if nccl_ms:
            nb = real / nccl_ms[i] / 1e6 * f
            bw_nccl.append(nb)
            row.update({"nccl_busbw_GBs": round(nb, 2), "vs_nccl": round(b / nb, 3)})
        if staged_ms:
            row["unregistered_busbw_GBs"] = round(real / staged_ms[i] / 1e6 * f, 2)
        table.append(row)
    del tab
    torch.cuda.empty_cache()

    ddp = None
    if not args.no_ddp:
        ddp = {backend: ddp_step(args, backend)}
    final_stats = stats()

    if rank == 0:
        rec = {
            "metric": METRIC, "value": round(geomean(bw), 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(region_ms / args.steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic", "impl": args.impl,
            "config": {"model": "collective sweep", "collectives": list(COLLS), "bytes": [sizes[0], sizes[-1]],
                       "global_batch": None, "seq_len": None, "parallelism": f"{world} ranks, one process per GPU",
                       "api": f"torch.distributed all_reduce / reduce_scatter_tensor / all_gather_into_tensor, backend {backend}",
                       "buffers": ("registered memory from hylink_b200.parallel.symmetric_empty (zero-copy kernels); the "
                                   "unregistered_busbw_GBs column repeats every cell on ordinary torch tensors (staged kernels)")
                       if registered else "ordinary torch tensors",
                       "busbw": "bytes/time * 2(n-1)/n (all-reduce), * (n-1)/n (reduce-scatter, all-gather); factor 1 with one GPU",
                       "scaling_note": ("bus bandwidth is the rate every GPU's link sustains, not a sum over GPUs: compare the value at N GPUs "
                                        "with the link rate (770 GB/s per direction measured for a peer copy) and with NCCL at the same N; "
                                        "with one GPU nothing crosses a link (the cells are a no-op and two device copies at HBM rate), "
                                        "so N x the one-GPU value is not a target for N GPUs"),
                       "l2_policy": "two rotating buffer pairs of 1 GiB; a whole pass over the table (> 4 GiB of traffic) lies "
                                    "between two timed calls of a cell, so no cell is served from L2"},
            "clocks": clocks,
            "e2e": {"value": round(geomean(bw_e2e), 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(n_launch),
            "nccl": {"value": round(geomean(bw_nccl), 2), "cells_at_or_above_nccl": sum(1 for r in table if r.get("vs_nccl", 0) >= 1.0),
                     "cells": len(table), "worst": min((r["vs_nccl"] for r in table), default=None)} if nccl_ms else None,
            "unregistered": {"value": round(geomean([r["unregistered_busbw_GBs"] for r in table]), 2)} if staged_ms else None,
            "split_ratio_pcie": round(float(alpha), 4),
            "table": table,
            "ddp": ddp,
            "comm": {k: final_stats.get(k) for k in ("nvls", "symm_mode", "calls", "nvl_bytes", "pcie_bytes", "kernel_launches")},
        }
        print(json.dumps(rec), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def _main_with_clean_stdout() -> int:
    """Libraries underneath print to stdout from C (NCCL its version line, the reference its log): everything that is
    not a JSON record of this script goes to stderr, so that stdout carries the record alone."""
    import builtins
    import ctypes

    sys.stdout.flush()
    real_out = os.dup(1)
    os.dup2(2, 1)
    plain_print = builtins.print

    def record_print(*a, **kw):
        text = " ".join(str(x) for x in a)
        if kw.get("file") is None and text.startswith("{"):
            os.write(real_out, (text + "\n").encode())
        else:
            plain_print(*a, **kw)

    builtins.print = record_print
    try:
        return main()
    finally:
        builtins.print = plain_print
        sys.stdout.flush()
        try:
            ctypes.CDLL(None).fflush(None)
        except (OSError, AttributeError):
            pass
        os.dup2(real_out, 1)
        os.close(real_out)


if __name__ == "__main__":
    sys.exit(_main_with_clean_stdout())
