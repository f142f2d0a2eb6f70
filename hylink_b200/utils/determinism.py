"""Bitwise determinism of reduce-scatter / all-reduce and agreement with an fp64 host oracle.

    python -m torch.distributed.run --nproc-per-node 8 -m hylink_b200.utils.determinism --bytes-to 64M

For every size and dtype (normal(0,1) data): the collective is run three times
with ``deterministic=True`` (fixed ascending-rank summation order in the peer
kernels) and the three results must be bit-identical; every rank's result must
be bit-identical to a host computation that adds the ranks' inputs in the same
order in fp32; and the distance to the fp64 sum must stay within the rounding
budget (half a unit in the last place of the output type plus the fp32
accumulation error of `world` terms).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--bytes-from", dest="lo", default="1M")
    ap.add_argument("--bytes-to", dest="hi", default="16M")
    ap.add_argument("--dtypes", default="fp32,bf16")
    a = ap.parse_args(argv)
    from hylink_b200.parallel.comm import Communicator, unique_id
    from hylink_b200.utils.sweep import DT, parse_size

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    failures = 0
    size = parse_size(a.lo)
    while size <= parse_size(a.hi):
        for dname in a.dtypes.split(","):
            dt = DT[dname]
            es = torch.empty((), dtype=dt).element_size()
            n_el = max(world, size // es // world * world)
            seg = n_el // world
            g = torch.Generator(device="cuda").manual_seed(1000 + rank)
            x = torch.randn(n_el, generator=g, device="cuda").to(dt)
            # every rank needs all inputs for the oracle of its own segment
            allx = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(allx, x)
            mine = [t[rank * seg:(rank + 1) * seg] for t in allx]
            acc32 = mine[0].float().clone()
            for t in mine[1:]:
                acc32 += t.float()
            same_order = acc32.to(dt)
            exact = sum(t.double() for t in mine)
            runs = []
            for _ in range(3):
                out = torch.empty(seg, dtype=dt, device="cuda")
                comm.reduce_scatter(x, out, deterministic=True)
                torch.cuda.synchronize()
                runs.append(out)
            ar = torch.empty_like(x)
            comm.all_reduce(x, ar, deterministic=True)
            torch.cuda.synchronize()
            repeatable = all(torch.equal(runs[0], r) for r in runs[1:])
            bitwise = torch.equal(runs[0], same_order) and torch.equal(ar[rank * seg:(rank + 1) * seg], same_order)
            # error budget: one rounding to the output type plus the fp32 accumulation of `world` terms
            mag = sum(t.double().abs() for t in mine)
            budget = 0.51 * torch.finfo(dt).eps * exact.abs() + world * torch.finfo(torch.float32).eps * mag + 1e-30
            near = bool(((runs[0].double() - exact).abs() <= budget).all())
            flag = torch.tensor([int(repeatable), int(bitwise), int(near)], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = flag.tolist()
            failures += 0 if all(ok) else 1
            if rank == 0:
                print(json.dumps({"bytes": n_el * es, "dtype": dname, "n": world, "repeatable": bool(ok[0]),
                                  "bitwise_vs_fixed_order_host": bool(ok[1]), "within_rounding_budget_of_fp64": bool(ok[2])}), flush=True)
        size *= 4
    if rank == 0:
        print(json.dumps({"event": "done", "failures": failures}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
