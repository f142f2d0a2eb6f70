"""Every NVLink/NVSwitch kernel by name on real GPUs, against an fp32 oracle.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m hylink_b200.utils.kernel_check [--max-bytes 64M]

Each collective is run with every algorithm it has (one-shot, two-shot pull,
NVLS, stores-only push, pipelined / lane kernels) on sizes that include odd
element counts. Every rank can rebuild all ranks' inputs (seeded by rank), so
the expected result is computed locally in plain PyTorch: fp32 accumulation in
ascending rank order, rounded once. Kernels that add in that order (all but
the NVLS ones, where the switch picks the order) must match bit for bit; the
NVLS kernels must match to one rounding step of the element type.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

AR_ALGOS = ["oneshot", "twoshot", "push", "pipelined", "nvls"]
RS_ALGOS = ["twoshot", "push", "pipelined", "nvls"]
AG_ALGOS = ["twoshot", "auto", "pipelined", "nvls"]


def _inputs(world, n_el, dtype, seed):
    out = []
    for r in range(world):
        g = torch.Generator(device="cuda").manual_seed(seed * 131 + r)
        out.append((torch.rand(n_el, generator=g, device="cuda") * 2 - 1).to(dtype))
    return out


def _ordered_sum(parts, dtype):
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    return acc.to(dtype)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", default="32M")
    ap.add_argument("--dtypes", default="bf16,fp32")
    a = ap.parse_args(argv)
    from .sweep import DT, parse_size

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    from ..parallel.comm import Communicator, unique_id

    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    nvls = bool(comm.stats()["nvls"])
    top = parse_size(a.max_bytes)
    failures, checks = [], 0

    def verdict(name, algo, dname, n_el, got, want, exact):
        nonlocal checks
        checks += 1
        if exact:
            ok = bool(torch.equal(got, want))
        else:
            tol = 1e-2 if got.dtype in (torch.bfloat16, torch.float16) else 1e-5
            ok = bool(torch.allclose(got.float(), want.float(), rtol=tol, atol=tol))
        if not ok:
            bad = int((got != want).sum())
            failures.append({"coll": name, "algo": algo, "dtype": dname, "elems": n_el, "rank": rank, "mismatches": bad})

    for dname in a.dtypes.split(","):
        dt = DT[dname]
        es = torch.empty((), dtype=dt).element_size()
        # per-rank element counts: tiny, odd, one around a CTA's share, and the largest asked for
        # ... plus two whole-packet sizes for the kernels that want them (zero-copy, low-latency)
        seg_counts = sorted({1, 7, 4099, (1 << 20) // es + 3, top // es // world, 3 * (16 // es), (256 << 10) // es})
        for si, seg in enumerate(seg_counts):
            n_el = seg * world
            ins = _inputs(world, n_el, dt, 7 + si)
            want_sum = _ordered_sum(ins, dt)
            for algo in AR_ALGOS:
                if algo == "nvls" and not nvls:
                    continue
                if algo == "oneshot" and n_el * es > (4 << 20):
                    continue
                out = torch.full((n_el + 16,), 3.0, device="cuda", dtype=dt)
                comm.all_reduce(ins[rank], out[8:8 + n_el], algo=algo)
                torch.cuda.synchronize()
                # with multicast memory the pipelined kernel reduces in the switch too
                exact = algo not in ("nvls",) and not (algo == "pipelined" and nvls and world >= 2)
                verdict("allreduce", algo, dname, n_el, out[8:8 + n_el], want_sum, exact)
                if not (bool((out[:8] == 3.0).all()) and bool((out[8 + n_el:] == 3.0).all())):
                    failures.append({"coll": "allreduce", "algo": algo, "dtype": dname, "elems": n_el, "rank": rank, "guard": True})
            for algo in RS_ALGOS:
                if algo == "nvls" and not nvls:
                    continue
                out = torch.full((seg + 16,), 3.0, device="cuda", dtype=dt)
                comm.reduce_scatter(ins[rank], out[8:8 + seg], algo=algo)
                torch.cuda.synchronize()
                exact = algo != "nvls" and not (algo == "pipelined" and nvls)
                verdict("reducescatter", algo, dname, seg, out[8:8 + seg], want_sum[rank * seg:(rank + 1) * seg], exact)
                if not (bool((out[:8] == 3.0).all()) and bool((out[8 + seg:] == 3.0).all())):
                    failures.append({"coll": "reducescatter", "algo": algo, "dtype": dname, "elems": seg, "rank": rank, "guard": True})
            want_gather = torch.cat([p[:seg] for p in ins])
            for algo in AG_ALGOS:
                if algo == "nvls" and not nvls:
                    continue
                out = torch.full((n_el + 16,), 3.0, device="cuda", dtype=dt)
                comm.all_gather(ins[rank][:seg], out[8:8 + n_el], algo=algo)
                torch.cuda.synchronize()
                verdict("allgather", algo, dname, n_el, out[8:8 + n_el], want_gather, True)
                if not (bool((out[:8] == 3.0).all()) and bool((out[8 + n_el:] == 3.0).all())):
                    failures.append({"coll": "allgather", "algo": algo, "dtype": dname, "elems": n_el, "rank": rank, "guard": True})
            for root in {0, world - 1}:
                for algo in (["nvls", "twoshot"] if nvls else ["twoshot"]):
                    buf = ins[rank].clone()
                    comm.broadcast(buf, root=root, algo=algo)
                    torch.cuda.synchronize()
                    verdict("broadcast", algo, dname, n_el, buf, ins[root], True)
            # zero-copy kernels on registered memory (both flavours), buffers allocated in the same order on every rank
            if n_el * es % 16 == 0 and seg * es % 16 == 0:
                rin = comm.alloc_registered(n_el, dt)
                rout = comm.alloc_registered(n_el + 32, dt)
                assert comm.is_registered(rin) and comm.is_registered(rout)
                pad = 16 // es
                for algo in (["zerocopy_nvls", "zerocopy_p2p", "auto"] if nvls else ["zerocopy_p2p", "auto"]):
                    rin.copy_(ins[rank])
                    rout.fill_(3.0)
                    comm.all_reduce(rin, rout[pad:pad + n_el], algo=algo)
                    torch.cuda.synchronize()
                    verdict("zc-allreduce", algo, dname, n_el, rout[pad:pad + n_el], want_sum, algo == "zerocopy_p2p")
                    if not (bool((rout[:pad] == 3.0).all()) and bool((rout[pad + n_el:] == 3.0).all())):
                        failures.append({"coll": "zc-allreduce", "algo": algo, "dtype": dname, "elems": n_el, "rank": rank, "guard": True})
                    # in place
                    comm.all_reduce(rin, rin, algo=algo)
                    torch.cuda.synchronize()
                    verdict("zc-allreduce-inplace", algo, dname, n_el, rin, want_sum, algo == "zerocopy_p2p")
                    rin.copy_(ins[rank])
                    part = torch.full((seg,), 3.0, device="cuda", dtype=dt)
                    comm.reduce_scatter(rin, part, algo=algo)
                    torch.cuda.synchronize()
                    verdict("zc-reducescatter", algo, dname, seg, part, want_sum[rank * seg:(rank + 1) * seg], algo == "zerocopy_p2p")
                    rout.fill_(3.0)
                    comm.all_gather(ins[rank][:seg], rout[pad:pad + n_el], algo=algo)
                    torch.cuda.synchronize()
                    verdict("zc-allgather", algo, dname, n_el, rout[pad:pad + n_el], want_gather, True)
                    rin.copy_(ins[rank])
                    comm.broadcast(rin, root=world - 1, algo=algo)
                    torch.cuda.synchronize()
                    verdict("zc-broadcast", algo, dname, n_el, rin, ins[world - 1], True)
                # staged and zero-copy calls interleaved without host synchronisation
                for _ in range(3):
                    rin.copy_(ins[rank])
                    comm.all_reduce(rin, rin)
                    comm.all_reduce(ins[rank], rout[pad:pad + n_el], algo="push")
                    comm.all_gather(rin[:seg], rout[pad:pad + n_el])
                torch.cuda.synchronize()
                verdict("zc-mixed", "auto", dname, n_el, rout[pad:pad + n_el], torch.cat([want_sum[:seg]] * world), not nvls or world < 4)
                del rin, rout
            # barrier-free small-message kernels: any memory, whole 16-byte packets, a segment that fits a slot
            if n_el * es % 16 == 0 and seg * es % 16 == 0 and seg * es <= (2 << 20):
                pad = 16 // es
                for rep in range(3):   # consecutive calls alternate the two halves of the low-latency region
                    out = torch.full((n_el + 2 * pad,), 3.0, device="cuda", dtype=dt)
                    comm.all_reduce(ins[rank], out[pad:pad + n_el], algo="ll")
                    torch.cuda.synchronize()
                    verdict("ll-allreduce", "ll", dname, n_el, out[pad:pad + n_el], want_sum, True)
                    if not (bool((out[:pad] == 3.0).all()) and bool((out[pad + n_el:] == 3.0).all())):
                        failures.append({"coll": "ll-allreduce", "algo": "ll", "dtype": dname, "elems": n_el, "rank": rank, "guard": True})
                    part = torch.full((seg + 2 * pad,), 3.0, device="cuda", dtype=dt)
                    comm.reduce_scatter(ins[rank], part[pad:pad + seg], algo="ll")
                    torch.cuda.synchronize()
                    verdict("ll-reducescatter", "ll", dname, seg, part[pad:pad + seg], want_sum[rank * seg:(rank + 1) * seg], True)
                    if not (bool((part[:pad] == 3.0).all()) and bool((part[pad + seg:] == 3.0).all())):
                        failures.append({"coll": "ll-reducescatter", "algo": "ll", "dtype": dname, "elems": seg, "rank": rank, "guard": True})
                    out.fill_(3.0)
                    comm.all_gather(ins[rank][:seg], out[pad:pad + n_el], algo="ll")
                    torch.cuda.synchronize()
                    verdict("ll-allgather", "ll", dname, n_el, out[pad:pad + n_el], want_gather, True)
                x2 = torch.full((n_el + 2 * pad,), 3.0, device="cuda", dtype=dt)
                comm.all_to_all(ins[rank], x2[pad:pad + n_el], algo="ll")
                torch.cuda.synchronize()
                verdict("ll-alltoall", "ll", dname, n_el, x2[pad:pad + n_el], torch.cat([p[rank * seg:(rank + 1) * seg] for p in ins]), True)
                # back to back without host synchronisation, mixed with barrier kernels, in place
                a1 = ins[rank].clone()
                a2 = torch.empty(n_el, device="cuda", dtype=dt)
                a3 = torch.empty(seg, device="cuda", dtype=dt)
                for _ in range(4):
                    a1.copy_(ins[rank])
                    comm.all_reduce(a1, a1, algo="ll")
                    comm.all_gather(a1[:seg], a2, algo="ll")
                    comm.all_reduce(ins[rank], a2, algo="push")
                    comm.reduce_scatter(ins[rank], a3, algo="ll")
                    comm.all_gather(a3, a2, algo="ll")
                torch.cuda.synchronize()
                verdict("ll-mixed", "ll", dname, n_el, a1, want_sum, True)
                verdict("ll-mixed-gather", "ll", dname, n_el, a2, want_sum, True)
            # calls of different sizes and kinds back to back, no host synchronisation in between: the staging
            # hand-over from one kernel to the next
            big, small = ins[rank], ins[rank][:max(1, n_el // 3)]
            o1 = torch.empty_like(big)
            o2 = torch.empty_like(small)
            o3 = torch.empty(n_el, device="cuda", dtype=dt)
            for _ in range(3):
                comm.all_reduce(small, o2, algo="nvls" if nvls else "twoshot")
                comm.all_gather(big[:seg], o3, algo="auto")
                comm.all_reduce(big, o1, algo="push")
                comm.all_reduce(small, o2, algo="push")
            torch.cuda.synchronize()
            verdict("mixed", "push", dname, n_el, o1, want_sum, True)
            verdict("mixed", "gather", dname, n_el, o3, want_gather, True)
            verdict("mixed", "push-small", dname, small.numel(), o2, _ordered_sum([p[:small.numel()] for p in ins], dt), True)
    all_fail = [None] * world
    dist.all_gather_object(all_fail, failures)
    flat = [f for fs in all_fail for f in fs]
    if rank == 0:
        print(json.dumps({"event": "kernel_check", "world": world, "nvls": nvls, "checks_per_rank": checks, "failures": len(flat),
                          "first": flat[:5]}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 1 if flat else 0


if __name__ == "__main__":
    sys.exit(main())
