"""Device and host micro-benchmarks that size the PCIe path and characterise overlap.

    python -m hylink_b200.utils.microbench h2h  [--bytes 64M] [--threads 1,2,4,8,16]     # no GPU needed
    python -m hylink_b200.utils.microbench dma  [--bytes 256M] [--gpus all]
    torchrun --nproc-per-node N -m hylink_b200.utils.microbench overlap [--bytes 128M] [--backend hylink|nccl]

* ``h2h``: rate of the NUMA worker pool's copy and three-address reduction against the number of workers, inside
  a NUMA node and across two (pcie-ccl-cuda/tests/dev/test_h2h.cpp).
* ``dma``: pinned host <-> device copy rate per GPU, one direction at a time, both at once, and all GPUs at once
  (pcie-ccl-cuda/tests/dev/test_gpu_dma_single.cpp, test_gpu_dma_all.cpp).
* ``overlap``: all-reduce / all-gather / reduce-scatter time alone and next to a GEMM that keeps the SMs busy, and
  the GEMM's slowdown (pcie-ccl-cuda/tests/dev/test_nccl_compute_overlap.cu:41-59,309-327).

* ``p2p`` (``torchrun --nproc-per-node 2 -m hylink_b200.utils.microbench p2p``): rate of a bare copy kernel
  between this rank's symmetric staging and the next rank's, for a grid of CTA counts, CTA sizes, unroll depths,
  directions (posted stores to the peer, loads from the peer, local copy) and address layouts. All ranks run the
  same configuration at the same time, so the figures are per direction under bidirectional load.

Every line of output is one JSON object.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys


def _size(text: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    t = text.strip().upper()
    return int(float(t[:-1]) * mult[t[-1]]) if t[-1] in mult else int(t)


def h2h(args) -> int:
    from hylink_b200._native import check, lib

    nodes = max(1, lib.hlHostNumaNodes())
    pairs = [(0, 0)] + ([(0, 1)] if nodes > 1 else [])
    dtype = {"fp32": 7, "bf16": 9, "fp16": 6}[args.dtype]
    for src, dst in pairs:
        for reduce in (0, 1):
            for th in [int(v) for v in args.threads.split(",")]:
                mean, best = C.c_double(), C.c_double()
                check(lib.hlHostBench(reduce, args.bytes, th, src, dst, args.iters, 1, dtype, C.byref(mean), C.byref(best)), "hlHostBench")
                print(json.dumps({"bench": "h2h", "op": "reduce" if reduce else "copy", "dtype": args.dtype, "bytes": args.bytes,
                                  "threads": th, "src_numa": src, "dst_numa": dst, "simd_level": lib.hlHostSimdLevel(),
                                  "GBs": round(mean.value, 2), "best_GBs": round(best.value, 2)}), flush=True)
    return 0


def dma(args) -> int:
    import torch

    n = torch.cuda.device_count()
    gpus = list(range(n)) if args.gpus == "all" else [int(v) for v in args.gpus.split(",")]
    el = args.bytes // 4
    host = {g: (torch.empty(el, dtype=torch.float32).pin_memory(), torch.empty(el, dtype=torch.float32).pin_memory()) for g in gpus}
    devb = {g: (torch.empty(el, device=f"cuda:{g}"), torch.empty(el, device=f"cuda:{g}")) for g in gpus}
    streams = {g: (torch.cuda.Stream(device=g), torch.cuda.Stream(device=g)) for g in gpus}

    def run(active, d2h, h2d):
        """Copies on every GPU of `active` at once; returns GB/s per GPU (max time over its streams)."""
        ev = {}
        for _ in range(2):  # first pass warms up
            for g in active:
                with torch.cuda.device(g):
                    s0, s1 = streams[g]
                    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                    e[0].record(s0)
                    e[2].record(s1)
                    for _ in range(args.iters):
                        if d2h:
                            with torch.cuda.stream(s0):
                                host[g][0].copy_(devb[g][0], non_blocking=True)
                        if h2d:
                            with torch.cuda.stream(s1):
                                devb[g][1].copy_(host[g][1], non_blocking=True)
                    e[1].record(s0)
                    e[3].record(s1)
                    ev[g] = e
            for g in active:
                torch.cuda.synchronize(g)
        out = {}
        for g in active:
            e = ev[g]
            ms = max(e[0].elapsed_time(e[1]) if d2h else 0.0, e[2].elapsed_time(e[3]) if h2d else 0.0)
            out[g] = args.bytes * args.iters * (int(d2h) + int(h2d)) / ms / 1e6
        return out

    for g in gpus:
        for name, d2h, h2d in (("d2h", True, False), ("h2d", False, True), ("bidir", True, True)):
            r = run([g], d2h, h2d)
            print(json.dumps({"bench": "dma", "mode": name, "gpu": g, "concurrent_gpus": 1, "bytes": args.bytes, "GBs": round(r[g], 2)}), flush=True)
    if len(gpus) > 1:
        for name, d2h, h2d in (("d2h", True, False), ("h2d", False, True), ("bidir", True, True)):
            r = run(gpus, d2h, h2d)
            print(json.dumps({"bench": "dma", "mode": name, "gpu": "all", "concurrent_gpus": len(gpus), "bytes": args.bytes,
                              "GBs_per_gpu": {str(g): round(v, 2) for g, v in r.items()}, "GBs_total": round(sum(r.values()), 2)}), flush=True)
    return 0


def overlap(args) -> int:
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.backend == "hylink":
        from hylink_b200.parallel import register_backend

        register_backend()
    dist.init_process_group(args.backend, device_id=dev)
    n_el = args.bytes // 2 // world * world
    x = torch.ones(n_el, device=dev, dtype=torch.bfloat16)
    seg = torch.ones(n_el // world, device=dev, dtype=torch.bfloat16)
    a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    b = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    comm_stream = torch.cuda.Stream()

    def coll(kind):
        if kind == "allreduce":
            dist.all_reduce(x)
        elif kind == "allgather":
            dist.all_gather_into_tensor(x, seg)
        else:
            dist.reduce_scatter_tensor(seg, x)

    def timed(kind, with_gemm, with_coll):
        res = []
        for it in range(args.iters + 2):
            dist.barrier()
            torch.cuda.synchronize()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            comm_stream.wait_stream(torch.cuda.current_stream())
            if with_gemm:
                e[0].record()
                for _ in range(args.gemms):
                    a @ b
                e[1].record()
            if with_coll:
                with torch.cuda.stream(comm_stream):
                    e[2].record()
                    coll(kind)
                    e[3].record()
            torch.cuda.synchronize()
            if it >= 2:
                res.append((e[0].elapsed_time(e[1]) if with_gemm else 0.0, e[2].elapsed_time(e[3]) if with_coll else 0.0))
        t = torch.tensor([sum(r[0] for r in res) / len(res), sum(r[1] for r in res) / len(res)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1])

    gemm_alone, _ = timed("allreduce", True, False)
    for kind in ("allreduce", "allgather", "reducescatter"):
        _, coll_alone = timed(kind, False, True)
        gemm_with, coll_with = timed(kind, True, True)
        if rank == 0:
            print(json.dumps({"bench": "overlap", "backend": args.backend, "coll": kind, "bytes": n_el * 2, "world": world,
                              "coll_alone_ms": round(coll_alone, 4), "coll_beside_gemm_ms": round(coll_with, 4),
                              "gemm_alone_ms": round(gemm_alone, 4), "gemm_beside_coll_ms": round(gemm_with, 4),
                              "serial_ms": round(coll_alone + gemm_alone, 4),
                              "overlapped_ms": round(max(coll_with, gemm_with), 4)}), flush=True)
    dist.destroy_process_group()
    return 0


def p2p(args) -> int:
    import torch
    import torch.distributed as dist

    from hylink_b200._native import check, lib
    from hylink_b200.parallel.comm import Communicator, unique_id

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    align = torch.zeros(1, device=dev)
    modes = {"push": 0, "pull": 1, "local": 2, "store": 3, "load": 4, "bulk": 5, "bulk-local": 6}

    def measure(mode, blocks, threads, unroll, layout):
        times = []
        for it in range(args.iters + 1):
            torch.cuda._sleep(1_000_000)   # lets the host queue everything; the tiny all-reduce then lines the ranks up
            dist.all_reduce(align)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            check(lib.hlNvlLinkProbe(comm._h, modes[mode], blocks, threads, unroll, layout, args.bytes, stream), "hlNvlLinkProbe")
            e1.record()
            torch.cuda.synchronize()
            if it:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor([sum(times) / len(times)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    grid = []
    for mode in args.modes.split(","):
        if mode.startswith("bulk"):   # bulk-copy engine: the "threads" slot carries the tile size
            for tile in [_size(v) for v in args.tiles.split(",")]:
                for blocks in [int(v) for v in args.blocks.split(",")]:
                    grid.append((mode, blocks, tile, 0, 0))
            continue
        for threads in [int(v) for v in args.threads.split(",")]:
            for blocks in [int(v) for v in args.blocks.split(",")]:
                for unroll in [int(v) for v in args.unroll.split(",")]:
                    if unroll == 16 and threads > 512:
                        continue
                    for layout in [int(v) for v in args.layouts.split(",")]:
                        grid.append((mode, blocks, threads, unroll, layout))
    for mode, blocks, threads, unroll, layout in grid:
        ms = measure(mode, blocks, threads, unroll, layout)
        if rank == 0:
            shape = ({"tile_bytes": threads} if mode.startswith("bulk") else
                     {"threads": threads, "unroll": unroll, "layout": "cta-contiguous" if layout else "grid-strided"})
            print(json.dumps({"bench": "p2p", "mode": mode, "blocks": blocks, **shape, "bytes": args.bytes, "world": world,
                              "ms": round(ms, 4), "GBs": round(args.bytes / ms / 1e6, 1),
                              "GBs_per_cta": round(args.bytes / ms / 1e6 / blocks, 2)}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("h2h")
    p.add_argument("--bytes", type=_size, default=64 << 20)
    p.add_argument("--threads", default="1,2,4,8,16")
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"])
    p = sub.add_parser("dma")
    p.add_argument("--bytes", type=_size, default=256 << 20)
    p.add_argument("--gpus", default="all")
    p.add_argument("--iters", type=int, default=4)
    p = sub.add_parser("overlap")
    p.add_argument("--bytes", type=_size, default=128 << 20)
    p.add_argument("--backend", default="hylink", choices=["hylink", "nccl"])
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--gemms", type=int, default=4)
    p = sub.add_parser("p2p")
    p.add_argument("--bytes", type=_size, default=256 << 20)
    p.add_argument("--modes", default="push,pull,local,store,load,bulk,bulk-local")
    p.add_argument("--tiles", default="4K,8K,16K,24K", help="tile sizes of the bulk-copy-engine modes")
    p.add_argument("--blocks", default="16,37,74,148,296")
    p.add_argument("--threads", default="256,512,1024")
    p.add_argument("--unroll", default="4,8")
    p.add_argument("--layouts", default="0,1")
    p.add_argument("--iters", type=int, default=3)
    args = ap.parse_args(argv)
    return {"h2h": h2h, "dma": dma, "overlap": overlap, "p2p": p2p}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
