"""Post-processing of the library's Chrome-trace files (``HYLINK_TRACE_FILE``).

    python -m hylink_b200.utils.trace_analysis trace.0.json trace.1.json [--per-op] [--merge merged.json]

Reports, per category (``pcie`` = whole collectives on the PCIe path, ``dma`` =
individual slices by kind: D2H, H2D, D2D, D2DReduce, H2H, H2HReduce), the
number of events, total and mean duration and the busy fraction of the traced
span; ``--merge`` writes one file with every rank's events on a common clock
(each file carries the wall-clock epoch of its monotonic timestamps).
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict


def load(path):
    text = open(path).read().rstrip().rstrip(",")
    if not text.endswith("]"):
        text += "\n]"
    return json.loads(text)


def clock_offset_us(events) -> float:
    """Microseconds to add to `ts` to obtain wall-clock microseconds."""
    for e in events:
        if e.get("ph") == "M" and e.get("name") == "clock":
            a = e["args"]
            return a["wall_epoch_us"] - a["steady_ns"] / 1000.0
    return 0.0


def analyse(events, per_op=False):
    spans = defaultdict(list)
    for e in events:
        if e.get("ph") != "X":
            continue
        key = (e.get("cat", ""), e.get("name", "")) if per_op else (e.get("cat", ""),)
        spans[key].append((e["ts"], e["dur"]))
    out = {}
    for key, xs in spans.items():
        t0 = min(t for t, _ in xs)
        t1 = max(t + d for t, d in xs)
        total = sum(d for _, d in xs)
        out[key] = {"events": len(xs), "total_us": total, "mean_us": total / len(xs), "span_us": t1 - t0,
                    "busy": total / (t1 - t0) if t1 > t0 else 0.0}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--per-op", action="store_true")
    ap.add_argument("--merge", metavar="OUT")
    a = ap.parse_args(argv)
    merged = []
    for path in a.files:
        ev = load(path)
        off = clock_offset_us(ev)
        print(f"== {path}: {len(ev)} events")
        for key, s in sorted(analyse(ev, a.per_op).items()):
            print(f"  {'/'.join(key):<24} n={s['events']:<7} total={s['total_us'] / 1e3:9.3f} ms mean={s['mean_us']:9.2f} us "
                  f"busy={100 * s['busy']:5.1f}%")
        for e in ev:
            if "ts" in e:
                e = dict(e, ts=e["ts"] + off)
            merged.append(e)
    if a.merge:
        with open(a.merge, "w") as f:
            json.dump(merged, f)
        print(f"merged {len(merged)} events into {a.merge}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
