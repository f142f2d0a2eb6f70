"""Decoder of the kernel timeline ring (``HYLINK_KERNEL_TIMELINE=1``).

Every NVLink-path kernel stamps ``%globaltimer`` for its first 148 CTAs at entry, at arrival at and release from
each of its cross-GPU barriers, and at exit. The intervals between the stamps are the kernel's phases — for the
stores-only all-reduce: push of the shards, wait for the peers' pushes, fold and push of the results, wait for the
peers' results, copy-out. They show where a multi-GPU launch spends its time without a profiler attached (kernels of
several ranks that wait on one another cannot be replayed under one).

``decode(words)`` returns one dict per recorded launch, oldest first; ``summarise`` turns the per-CTA stamps into
per-phase medians. ``python -m hylink_b200.utils.kernel_timeline`` under torchrun runs a few collectives and prints
the summary of each rank-0 launch.
"""
from __future__ import annotations

import json
import os
import statistics
import sys

TL_CALLS, TL_BLOCKS, TL_PHASES = 16, 148, 8
KINDS = {0: "barrier", 1: "allreduce_oneshot", 2: "allreduce_twoshot", 3: "allreduce_nvls", 4: "reducescatter",
         5: "reducescatter_nvls", 6: "allgather", 7: "broadcast", 8: "alltoall", 9: "allgather_nvls", 10: "broadcast_nvls",
         11: "allreduce_pipelined_p2p", 12: "allreduce_pipelined_nvls", 13: "reducescatter_pipelined_p2p",
         14: "reducescatter_pipelined_nvls", 15: "allreduce_push", 16: "reducescatter_push", 17: "allgather_push", 18: "allgather_lanes",
         19: "zerocopy_allreduce_nvls", 20: "zerocopy_allreduce_p2p", 21: "zerocopy_reducescatter_nvls",
         22: "zerocopy_reducescatter_p2p", 23: "zerocopy_allgather_nvls", 24: "zerocopy_allgather_p2p",
         25: "zerocopy_broadcast_nvls", 26: "zerocopy_broadcast_p2p",
         27: "lowlatency_allreduce", 28: "lowlatency_reducescatter", 29: "lowlatency_allgather", 30: "lowlatency_alltoall"}
PHASE_NAMES = ["entry", "arrive1", "leave1", "arrive2", "leave2", "arrive3", "leave3", "exit"]


def decode(words):
    """``words``: the ring as a list of ints. Returns launches sorted by flag base."""
    stamps_end = TL_CALLS * TL_BLOCKS * TL_PHASES
    out = []
    for slot in range(TL_CALLS):
        seq, kb, count, _ = words[stamps_end + 4 * slot: stamps_end + 4 * slot + 4]
        blocks = kb & 0xFFFFFFFF
        if blocks == 0:
            continue
        n = min(blocks, TL_BLOCKS)
        per_block = []
        for b in range(n):
            base = (slot * TL_BLOCKS + b) * TL_PHASES
            per_block.append(words[base: base + TL_PHASES])
        out.append({"seq": seq, "kind": KINDS.get(kb >> 32, str(kb >> 32)), "blocks": blocks, "count": count, "stamps": per_block})
    out.sort(key=lambda d: d["seq"])
    return out


def summarise(launch):
    """Median, over the recorded CTAs, of the time between consecutive stamps that the kernel took (microseconds)."""
    st = launch["stamps"]
    if launch["kind"].endswith("pipelined_p2p"):
        return _summarise_lanes(launch)
    entry0 = min(s[0] for s in st if s[0])
    used = [p for p in range(TL_PHASES) if all(s[p] >= s[0] and s[p] != 0 for s in st)]
    # a stamp of an earlier launch in the same ring slot is older than this launch's entry: the filter above drops it
    phases, prev = {}, used[0]
    for p in used[1:]:
        d = [(s[p] - s[prev]) / 1e3 for s in st]
        phases[f"{PHASE_NAMES[prev]}->{PHASE_NAMES[p]}"] = {"median_us": round(statistics.median(d), 2), "max_us": round(max(d), 2)}
        prev = p
    total = [(s[used[-1]] - entry0) / 1e3 for s in st]
    return {"kind": launch["kind"], "blocks": launch["blocks"], "count": launch["count"],
            "entry_spread_us": round((max(s[0] for s in st) - entry0) / 1e3, 2),
            "total_us": round(max(total), 2), "phases": phases}


def _summarise_lanes(launch):
    """The lane kernels record sums instead of boundaries: per CTA, the time spent waiting for tiles, handing tiles
    on and working, and which stage the CTA ran (slots 1-4 as entry + value)."""
    roles = {0: "push", 1: "fold", 2: "copy-out"}
    per_role = {}
    for s in launch["stamps"]:
        if not s[0] or not s[7]:
            continue
        role = roles.get(round((s[4] - s[0]) / 1e6), "?")
        per_role.setdefault(role, []).append(((s[1] - s[0]) / 1e3, (s[2] - s[0]) / 1e3, (s[3] - s[0]) / 1e3, (s[7] - s[0]) / 1e3))
    out = {"kind": launch["kind"], "blocks": launch["blocks"], "count": launch["count"], "stages": {}}
    for role, rows in per_role.items():
        med = lambda i: round(statistics.median(r[i] for r in rows), 2)  # noqa: E731
        out["stages"][role] = {"ctas": len(rows), "waiting_us": med(0), "handing_on_us": med(1), "working_us": med(2), "total_us": med(3)}
    out["total_us"] = round(max(r[3] for rows in per_role.values() for r in rows), 2) if per_role else 0.0
    return out


def main(argv=None) -> int:
    import argparse

    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--bytes", default="256M")
    ap.add_argument("--colls", default="allreduce,reducescatter,allgather")
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--blocks", type=int, default=0)
    a = ap.parse_args(argv)
    os.environ["HYLINK_KERNEL_TIMELINE"] = "1"
    from hylink_b200.parallel.comm import Communicator, unique_id
    from hylink_b200.utils.microbench import _size

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = Communicator(rank, world, uid=box[0], device=local)
    n_el = _size(a.bytes) // 2 // world * world
    x = torch.ones(n_el, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    seg = n_el // world
    align = torch.zeros(1, device=dev)
    for coll in a.colls.split(","):
        for _ in range(3):
            torch.cuda._sleep(1_000_000)
            dist.all_reduce(align)
            if coll == "allreduce":
                comm.all_reduce(x, y, path="nvlink", algo=a.algo, max_blocks=a.blocks)
            elif coll == "allgather":
                comm.all_gather(x[:seg], y, path="nvlink", max_blocks=a.blocks)
            else:
                comm.reduce_scatter(x, y[:seg], path="nvlink", algo=a.algo, max_blocks=a.blocks)
            torch.cuda.synchronize()
        if rank == 0:
            last = comm.kernel_timeline()[-1]
            print(json.dumps({"coll": coll, "bytes": n_el * 2, "world": world, **summarise(last)}), flush=True)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
