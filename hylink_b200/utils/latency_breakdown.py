"""Where the time of a small collective goes: kernel phases, the launch around it, the backend around that.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m hylink_b200.utils.latency_breakdown [--bytes 1M,2M,4M] [--colls allreduce,reducescatter,allgather]

For every collective and size, on registered buffers, three nested measurements, each the median over `--iters`
calls that were queued behind a short sleep kernel so that the GPU, not the host, sets the pace:

* ``kernel_us`` and ``phases``: from the kernel timeline (``%globaltimer`` stamps inside the kernel). Barrier-based
  kernels: entry to the first barrier, the barrier itself (it also absorbs the skew between the ranks' launches),
  the transfer, the closing barrier; the low-latency kernels have no barrier, so only entry to exit;
* ``direct_us``: CUDA events around the C API call on one stream (launch gap + kernel);
* ``backend_us``: CUDA events around ``torch.distributed`` on backend ``hylink`` (synchronous calls run on the
  caller's stream; with ``HYLINK_TORCH_SYNC_INLINE=0`` they hop to the communication stream and back, which adds two
  events and two stream waits);
* ``nccl_us``: the same around the NCCL backend, for comparison.

All figures are from rank 0 except the event times, which are the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys


def _timed(torch, fn, iters, sleep_cycles):
    """Median microseconds between two events around fn(), the call queued behind a sleep kernel."""
    out = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(sleep_cycles)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(out)


def main(argv=None) -> int:
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--bytes", default="64K,1M,2M,4M")
    ap.add_argument("--colls", default="allreduce,reducescatter,allgather")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--sleep-cycles", type=int, default=400_000, help="length of the sleep kernel in front of each timed call")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    os.environ["HYLINK_KERNEL_TIMELINE"] = "1"
    from hylink_b200.parallel import register_backend, symmetric_empty
    from hylink_b200.parallel.comm import Communicator, unique_id
    from hylink_b200.utils.kernel_timeline import summarise
    from hylink_b200.utils.microbench import _size

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    register_backend()
    dist.init_process_group("nccl", device_id=dev)
    hl_group = dist.new_group(backend="hylink")
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    sizes = [_size(s) for s in a.bytes.split(",")]
    top = max(sizes) // 2 // world * world
    # buffers of the direct path come from its own communicator, those of the backend path from the backend's
    x, y = comm.alloc_registered(top, torch.bfloat16), comm.alloc_registered(top, torch.bfloat16)
    x.fill_(1.0)
    dist.all_reduce(torch.zeros(1, device=dev), group=hl_group)   # the backend's communicator exists from here on
    bx, by = symmetric_empty(top, torch.bfloat16, group=hl_group), symmetric_empty(top, torch.bfloat16, group=hl_group)
    bx.fill_(1.0)
    nx, ny = torch.ones(top, device=dev, dtype=torch.bfloat16), torch.empty(top, device=dev, dtype=torch.bfloat16)
    outf = open(a.out, "a") if (a.out and rank == 0) else None
    for coll in a.colls.split(","):
        for size in sizes:
            n_el = size // 2 // world * world
            seg = n_el // world
            if coll == "allreduce":
                direct = lambda: comm.all_reduce(x[:n_el], y[:n_el], path="nvlink")
                back = lambda g, i, o: dist.all_reduce(i[:n_el], group=g)
            elif coll == "reducescatter":
                direct = lambda: comm.reduce_scatter(x[:n_el], y[:seg], path="nvlink")
                back = lambda g, i, o: dist.reduce_scatter_tensor(o[:seg], i[:n_el], group=g)
            elif coll == "allgather":
                direct = lambda: comm.all_gather(x[:seg], y[:n_el], path="nvlink")
                back = lambda g, i, o: dist.all_gather_into_tensor(o[:n_el], i[:seg], group=g)
            else:
                raise SystemExit(f"unknown collective {coll}")
            for _ in range(3):
                direct()
                back(hl_group, bx, by)
                back(None, nx, ny)
            torch.cuda.synchronize()
            dist.barrier()
            t_direct = _timed(torch, direct, a.iters, a.sleep_cycles)
            tl = summarise(comm.kernel_timeline()[-1])
            dist.barrier()
            t_back = _timed(torch, lambda: back(hl_group, bx, by), a.iters, a.sleep_cycles)
            dist.barrier()
            t_nccl = _timed(torch, lambda: back(None, nx, ny), a.iters, a.sleep_cycles)
            t = torch.tensor([t_direct, t_back, t_nccl], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rec = {"coll": coll, "bytes": n_el * 2, "world": world, "kernel": tl.get("kind"), "blocks": tl.get("blocks"),
                   "kernel_us": tl.get("total_us"), "entry_spread_us": tl.get("entry_spread_us"), "phases": tl.get("phases"),
                   "direct_us": round(float(t[0]), 2), "backend_us": round(float(t[1]), 2), "nccl_us": round(float(t[2]), 2)}
            if rank == 0:
                line = json.dumps(rec)
                print(line, flush=True)
                if outf:
                    outf.write(line + "\n")
    dist.barrier()
    del x, y, bx, by
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
