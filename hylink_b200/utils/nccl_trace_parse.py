"""Summarises the JSON-lines files written by ``libhylink_nccltrace.so``.

    LD_PRELOAD=hylink_b200/lib/libhylink_nccltrace.so HYLINK_NCCL_TRACE_FILE=trace.%p.jsonl python train.py
    python -m hylink_b200.utils.nccl_trace_parse trace.*.jsonl

Prints, per call name and message size, the number of calls, the bytes moved,
the host-side call time and how many calls were issued under CUDA-graph
capture; ``--timeline`` dumps the merged, time-ordered call list instead.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

TYPE_BYTES = {0: 1, 1: 1, 2: 4, 3: 4, 4: 8, 5: 8, 6: 2, 7: 4, 8: 8, 9: 2}


def load(paths):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        rows.append(json.loads(line))
                    except json.JSONDecodeError:
                        pass
    rows.sort(key=lambda r: (r.get("t", 0), r.get("seq", 0)))
    return rows


def summarise(rows):
    agg = defaultdict(lambda: {"calls": 0, "bytes": 0, "host_us": 0.0, "captured": 0, "errors": 0})
    for r in rows:
        nbytes = r["count"] * TYPE_BYTES.get(r.get("dtype", -1), 0) if r.get("dtype", -1) >= 0 else 0
        a = agg[(r["call"], nbytes)]
        a["calls"] += 1
        a["bytes"] += nbytes
        a["host_us"] += r.get("host_us", 0.0)
        a["captured"] += 1 if r.get("capturing") == 1 else 0
        a["errors"] += 1 if r.get("rc", 0) != 0 else 0
    return agg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--timeline", action="store_true")
    a = ap.parse_args(argv)
    rows = load(a.files)
    if a.timeline:
        t0 = rows[0]["t"] if rows else 0
        for r in rows:
            print(f"{r['t'] - t0:10.6f}s pid {r['pid']:>7} {r['call']:<24} count={r['count']:<12} dtype={r['dtype']:<2} "
                  f"op={r['op']:<2} peer={r['peer']:<3} capturing={r['capturing']} rc={r['rc']}")
        return 0
    agg = summarise(rows)
    print(f"{'call':<24} {'msg bytes':>14} {'calls':>8} {'total MiB':>12} {'host us/call':>13} {'captured':>9} {'errors':>7}")
    for (call, nbytes), a_ in sorted(agg.items()):
        print(f"{call:<24} {nbytes:>14} {a_['calls']:>8} {a_['bytes'] / 2**20:>12.1f} {a_['host_us'] / a_['calls']:>13.2f} "
              f"{a_['captured']:>9} {a_['errors']:>7}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
