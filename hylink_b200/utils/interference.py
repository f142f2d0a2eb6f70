"""PCIe-interference experiment: does the balancer retune the NVLink:PCIe split?

One process per GPU::

    python -m torch.distributed.run --nproc-per-node 8 -m hylink_b200.utils.interference \
        --size 256M --iters 60 --levels 0,25,50,75 --controller split_ratio --out interference.jsonl

Every rank runs an all-reduce loop on a forked (NVLink + PCIe) communicator
while a background thread keeps its own PCIe link busy with pinned
host<->device copies paced to a given percentage of the link's measured
bandwidth. Per iteration rank 0 logs the device time (max over ranks), the bus
bandwidth, the PCIe byte share the controller chose, and both paths' times.
With ``--controller static`` the share stays where it started — the contrast
the reference's experiment plots (multipath-orchestrator/tests/nccl_test/
allgather/allgather_with_pcie.cc:122-283 and pcie_interference.sh:10; paced
copies as in tests/pcie_test/mem_test/d2h_paced_test.cpp:21-27).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch
import torch.distributed as dist


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mul = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}.get(s[-1], 1)
    return int(float(s[:-1]) * mul) if s[-1] in "KMG" else int(s)


def measure_pcie_gbs(dev, nbytes=256 << 20, reps=4):
    """(d2h, h2d) GB/s of this GPU's link with pinned memory."""
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = []
    for src, dst in ((devbuf, host), (host, devbuf)):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        out.append(nbytes * reps / e0.elapsed_time(e1) / 1e6)
    return out[0], out[1]


class Interferer(threading.Thread):
    """Keeps the PCIe link busy at `percent` of `link_gbs` with chunked pinned copies in both directions."""

    def __init__(self, dev, link_gbs: float, chunk=16 << 20):
        super().__init__(daemon=True)
        self.dev, self.link, self.chunk = dev, link_gbs, chunk
        self.percent = 0
        self.stop_flag = False
        self.moved = 0

    def run(self):
        torch.cuda.set_device(self.dev)
        stream = torch.cuda.Stream(device=self.dev)
        host = torch.empty(self.chunk, dtype=torch.uint8).pin_memory()
        devbuf = torch.empty(self.chunk, dtype=torch.uint8, device=self.dev)
        flip = False
        while not self.stop_flag:
            p = self.percent
            if p <= 0:
                time.sleep(0.001)
                continue
            t0 = time.perf_counter()
            with torch.cuda.stream(stream):
                (host if flip else devbuf).copy_(devbuf if flip else host, non_blocking=True)
            stream.synchronize()
            flip = not flip
            self.moved += self.chunk
            # pace: this chunk should have taken chunk / (p% of the link)
            want = self.chunk / (self.link * 1e9 * p / 100.0)
            spare = want - (time.perf_counter() - t0)
            if spare > 0:
                time.sleep(spare)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--size", default="256M")
    ap.add_argument("--iters", type=int, default=60, help="iterations per interference level")
    ap.add_argument("--levels", default="0,25,50,75")
    ap.add_argument("--controller", default="split_ratio", choices=["split_ratio", "tcp", "static"])
    ap.add_argument("--static-alpha", type=float, default=0.05)
    ap.add_argument("--coll", default="allreduce", choices=["allreduce", "allgather", "reducescatter"])
    ap.add_argument("--out", default="")
    ap.add_argument("--charts", default="", metavar="DIR", help="with --out: also draw the per-call bandwidth and PCIe-share charts (SVG) into DIR")
    a = ap.parse_args(argv)

    os.environ["HYLINK_ORCH_ENABLE"] = "1"
    os.environ["HYLINK_ALGO"] = a.controller
    os.environ["HYLINK_STATIC_ALPHA"] = str(a.static_alpha)
    os.environ.setdefault("HYLINK_ORCH_GUARD", "0")  # keep forking so that the retuning itself can be observed
    os.environ.setdefault("HYLINK_MIN_MSG_SIZE", "4M")
    os.environ.setdefault("HYLINK_MIN_MSG_SIZE_8", "4M")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from hylink_b200.parallel.comm import Communicator, unique_id

    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)

    d2h, h2d = measure_pcie_gbs(dev)
    link = min(d2h, h2d)
    nbytes = parse_size(a.size)
    n_el = nbytes // 2 // world * world
    # registered buffers: the NVLink half of every forked call runs zero-copy
    x = comm.alloc_registered(n_el, torch.bfloat16)
    y = comm.alloc_registered(n_el, torch.bfloat16)
    x.copy_((torch.rand(n_el, device=dev) * 2 - 1).to(torch.bfloat16))
    seg = n_el // world
    bg = Interferer(dev, link)
    bg.start()
    outf = open(a.out, "a") if (a.out and rank == 0) else None
    if rank == 0:
        print(json.dumps({"event": "link", "d2h_GBs": round(d2h, 1), "h2d_GBs": round(h2d, 1), "world": world,
                          "controller": a.controller}), flush=True)
    factor = 2.0 * (world - 1) / world if a.coll == "allreduce" else (world - 1) / world
    align = torch.zeros(1, device=dev)
    it = 0
    for level in [int(v) for v in a.levels.split(",")]:
        bg.percent = level
        dist.barrier()
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # Line the ranks up on the device before the timed call: a delay long enough for the host to queue
            # everything behind it, then a tiny NCCL all-reduce that ends on all GPUs within microseconds. Without
            # this the maximum over ranks also counts how much earlier one rank reached the call than another.
            torch.cuda._sleep(2_000_000)
            dist.all_reduce(align)
            e0.record()
            if a.coll == "allreduce":
                comm.all_reduce(x, y, path="auto")
            elif a.coll == "allgather":
                comm.all_gather(x[:seg], y, path="auto")
            else:
                comm.reduce_scatter(x, y[:seg], path="auto")
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            st = comm.stats()
            if rank == 0:
                rec = {"iter": it, "interference_pct": level, "ms": round(float(t[0]), 4),
                       "busbw_GBs": round(n_el * 2 / float(t[0]) / 1e6 * factor, 1), "alpha": round(st["last_alpha"], 5),
                       "fast_ms": round(st["last_fast_ms"], 4), "pcie_ms": round(st["last_pcie_ms"], 4)}
                line = json.dumps(rec)
                print(line, flush=True)
                if outf:
                    outf.write(line + "\n")
            it += 1
    # the dedicated link alone, without interference and under the heaviest level: what forking has to beat
    for level in (0, max(int(v) for v in a.levels.split(","))):
        bg.percent = level
        dist.barrier()
        times = []
        for _ in range(max(8, a.iters // 4)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(2_000_000)
            dist.all_reduce(align)
            e0.record()
            if a.coll == "allreduce":
                comm.all_reduce(x, y, path="nvlink")
            elif a.coll == "allgather":
                comm.all_gather(x[:seg], y, path="nvlink")
            else:
                comm.reduce_scatter(x, y[:seg], path="nvlink")
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t[0]))
        if rank == 0:
            med = sorted(times)[len(times) // 2]
            line = json.dumps({"event": "nvlink_only", "interference_pct": level, "ms": round(med, 4), "busbw_GBs": round(n_el * 2 / med / 1e6 * factor, 1)})
            print(line, flush=True)
            if outf:
                outf.write(line + "\n")
    bg.stop_flag = True
    bg.join(2)
    if rank == 0:
        print(json.dumps({"event": "done", "tuning": json.loads(comm.dump_tuning())}), flush=True)
        if outf:
            outf.close()
            if a.charts:
                from hylink_b200.utils.compare import plot_interference

                for path in plot_interference([a.out], a.charts):
                    print(json.dumps({"event": "chart", "file": path}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
