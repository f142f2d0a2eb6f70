"""Bus-bandwidth sweep: this library's collectives against NCCL on the same GPUs.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m hylink_b200.utils.sweep --colls allreduce,reducescatter,allgather --dtypes bf16,fp32 \
        --bytes-from 1K --bytes-to 1G --check --out sweep.jsonl

Every number is timed on the device with CUDA events and is the MAX over ranks.
busbw = algbw * 2(n-1)/n for all-reduce and * (n-1)/n for reduce-scatter /
all-gather / all-to-all (the nccl-tests convention, also used by the
reference: pcie-ccl-cuda/tests/common/test_common.hpp:108-121). Buffers rotate
through a pool larger than the 126 MB L2 so that small sizes are not served
from cache.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mul = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}.get(s[-1], 1)
    return int(float(s[:-1]) * mul) if s[-1] in "KMG" else int(s)


DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "fp64": torch.float64, "int32": torch.int32}


def bus_factor(coll: str, n: int) -> float:
    return 2.0 * (n - 1) / n if coll == "allreduce" else (n - 1) / n


def time_op(fn, nslots: int, iters: int, warmup: int) -> float:
    """Mean milliseconds per call, device-timed."""
    for i in range(warmup):
        fn(i % nslots)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        starts[i].record()
        fn((warmup + i) % nslots)
        ends[i].record()
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--colls", default="allreduce,reducescatter,allgather")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--bytes-from", dest="lo", default="1K")
    ap.add_argument("--bytes-to", dest="hi", default="256M")
    ap.add_argument("--factor", type=int, default=2)
    ap.add_argument("--iters", type=int, default=0, help="0 = by size")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--algo", default="auto", help="auto|oneshot|twoshot|nvls|pipelined|push|zerocopy|zerocopy_nvls|zerocopy_p2p|ll")
    ap.add_argument("--path", default="nvlink", help="nvlink|pcie|split|auto")
    ap.add_argument("--blocks", dest="max_blocks", type=int, default=0)
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--registered", action="store_true", help="buffers from the library's registered memory (zero-copy kernels)")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from hylink_b200.parallel.comm import Communicator, unique_id

    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    st = comm.stats()
    if rank == 0:
        print(json.dumps({"event": "init", "world": world, "nvls": st["nvls"], "symm_mode": st["symm_mode"]}), flush=True)

    lo, hi = parse_size(a.lo), parse_size(a.hi)
    sizes = []
    s = lo
    while s <= hi:
        sizes.append(s)
        s *= a.factor
    pool_bytes = max(hi, 256 << 20)
    results, failures = [], 0
    outf = open(a.out, "a") if (a.out and rank == 0) else None
    kw = dict(algo=a.algo, path=a.path, max_blocks=a.max_blocks, deterministic=a.deterministic)
    for coll in a.colls.split(","):
        for dname in a.dtypes.split(","):
            dt = DT[dname]
            es = torch.empty((), dtype=dt).element_size()
            # `size` is the nccl-tests message size: AR total bytes; RS/AG/A2A the FULL buffer (n segments)
            pool_in = pool_out = want = got = None   # registered memory is handed out in call order: release before asking again
            if a.registered:
                pool_in = comm.alloc_registered(pool_bytes // es, dt)
                pool_out = comm.alloc_registered(pool_bytes // es, dt)
            else:
                pool_in = torch.empty(pool_bytes // es, dtype=dt, device="cuda")
                pool_out = torch.empty(pool_bytes // es, dtype=dt, device="cuda")
            if dt.is_floating_point:
                pool_in.copy_((torch.rand(pool_in.numel(), device="cuda") * 2 - 1) if coll == "allreduce"
                              else torch.randn(pool_in.numel(), device="cuda"))
            else:
                pool_in.copy_(torch.randint(-100, 100, (pool_in.numel(),), device="cuda"))
            for size in sizes:
                n_el = max(world, (size // es) // world * world)
                seg = n_el // world
                nslots = max(1, pool_in.numel() // n_el)

                def bufs(i):
                    return pool_in[i * n_el:(i + 1) * n_el], pool_out[i * n_el:(i + 1) * n_el]

                if coll == "allreduce":
                    ours = lambda i: comm.all_reduce(bufs(i)[0], bufs(i)[1], **kw)
                    ref = lambda i: (bufs(i)[1].copy_(bufs(i)[0]), dist.all_reduce(bufs(i)[1]))
                elif coll == "reducescatter":
                    ours = lambda i: comm.reduce_scatter(bufs(i)[0], bufs(i)[1][:seg], **kw)
                    ref = lambda i: dist.reduce_scatter_tensor(bufs(i)[1][:seg], bufs(i)[0])
                elif coll == "allgather":
                    ours = lambda i: comm.all_gather(bufs(i)[0][:seg], bufs(i)[1], path=a.path, max_blocks=a.max_blocks,
                                                     algo=a.algo if a.algo in ("twoshot", "pipelined", "nvls", "ll", "zerocopy", "zerocopy_nvls", "zerocopy_p2p") else "auto")
                    ref = lambda i: dist.all_gather_into_tensor(bufs(i)[1], bufs(i)[0][:seg])
                elif coll == "alltoall":
                    ours = lambda i: comm.all_to_all(bufs(i)[0], bufs(i)[1], path=a.path, max_blocks=a.max_blocks)
                    ref = lambda i: dist.all_to_all_single(bufs(i)[1], bufs(i)[0])
                else:
                    raise SystemExit(f"unknown collective {coll}")

                ok = None
                if a.check:
                    ours(0)
                    torch.cuda.synchronize()
                    got = bufs(0)[1].clone()
                    ref(0)
                    torch.cuda.synchronize()
                    want = bufs(0)[1]
                    span = seg if coll == "reducescatter" else n_el
                    if coll in ("allgather", "alltoall") or not dt.is_floating_point:
                        ok = bool(torch.equal(got[:span], want[:span]))
                    else:
                        tol = 2e-2 if dt in (torch.bfloat16, torch.float16) else 1e-5
                        ok = bool(torch.allclose(got[:span].float(), want[:span].float(), rtol=tol, atol=tol * world))
                    flag = torch.tensor([0 if ok else 1], device="cuda")
                    dist.all_reduce(flag)
                    ok = int(flag.item()) == 0
                    failures += 0 if ok else 1
                iters = a.iters or (50 if size <= (1 << 20) else (20 if size <= (64 << 20) else 8))
                dist.barrier()
                t_ours = time_op(ours, nslots, iters, a.warmup)
                t_ref = float("nan")
                if not a.no_nccl:
                    dist.barrier()
                    if coll == "allreduce":  # time NCCL in place, without the extra copy
                        ref_t = lambda i: dist.all_reduce(bufs(i)[1])
                    else:
                        ref_t = ref
                    t_ref = time_op(ref_t, nslots, iters, a.warmup)
                tt = torch.tensor([t_ours, t_ref if t_ref == t_ref else 0.0], device="cuda", dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                t_ours, t_ref = float(tt[0]), float(tt[1])
                nbytes = n_el * es
                f = bus_factor(coll, world)
                rec = {"coll": coll, "dtype": dname, "bytes": nbytes, "n": world, "ms": round(t_ours, 5),
                       "busbw_GBs": round(nbytes / t_ours / 1e6 * f, 2),
                       "nccl_ms": round(t_ref, 5) if t_ref else None,
                       "nccl_busbw_GBs": round(nbytes / t_ref / 1e6 * f, 2) if t_ref else None,
                       "speedup": round(t_ref / t_ours, 3) if t_ref else None, "ok": ok, "algo": a.algo, "path": a.path,
                       "registered": bool(a.registered)}
                if a.path in ("split", "auto"):
                    rec["pcie_share"] = round(float(comm.stats()["last_alpha"]), 4)   # share of the bytes the PCIe path carried in the latest call
                if rank == 0:
                    line = json.dumps(rec)
                    print(line, flush=True)
                    if outf:
                        outf.write(line + "\n")
                        outf.flush()
                results.append(rec)
            del pool_in, pool_out
    if rank == 0:
        done = {"event": "done", "failures": failures, "stats": comm.stats()}
        try:   # present when the interposers of blocking CUDA calls are preloaded (libhylink_cudashim.so)
            import ctypes

            fn = ctypes.CDLL(None).hlBlockShimDrains
            fn.restype = ctypes.c_ulonglong
            done["block_shim_drains"] = int(fn())
        except (AttributeError, OSError):
            pass
        print(json.dumps(done), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
