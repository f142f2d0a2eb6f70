"""Post-processing of the library's Chrome-trace files (``HYLINK_TRACE_FILE``).

    python -m hylink_b200.utils.trace_analysis summary  trace.0.json trace.1.json [--per-op]
    python -m hylink_b200.utils.trace_analysis phases   trace.0.json
    python -m hylink_b200.utils.trace_analysis by-size  trace.0.json
    python -m hylink_b200.utils.trace_analysis host     trace.0.json
    python -m hylink_b200.utils.trace_analysis compare  a.json labelA b.json labelB [--op D2H]
    python -m hylink_b200.utils.trace_analysis merge    trace.*.json -o merged.json [--timeline kernels.json]

What the trace holds: one ``pcie`` event per collective round on the PCIe path (name = the collective, ``args.bytes``
= message bytes), one ``dma`` event per slice (name = the schedule op: D2H, H2D, D2D, D2DReduce, H2H, H2HReduce;
``args.bytes`` = slice bytes), ``collective`` events for every API call and ``orch`` events for fork / join.

* ``summary``  events, total / mean duration and busy fraction per category (per op with ``--per-op``).
* ``phases``   per collective ("iteration"): the span of its D2H, host (H2H / H2HReduce), H2D and device-reduce
               slices, how much the phases overlap, and the time no slice was in flight.
* ``by-size``  iterations grouped by message size: latency percentiles, achieved algorithm bandwidth, slice
               statistics.
* ``host``     duration distribution of the host copy / reduce slices and the stragglers among them (a slice far
               above the median was most likely preempted).
* ``compare``  per-slice latency percentiles of one op across several trace files (e.g. two pool flavours).
* ``merge``    all files on one wall clock (every file carries the wall-clock epoch of its monotonic timestamps),
               optionally together with a kernel timeline written by ``utils.kernel_timeline``.

Parity: pcie-ccl-cuda/tests/trace/{analyze_trace,analyze_phases,analyze_by_size,analyze_h2h,compare_d2h_latency,
merge_msprof,trace_common}.py.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

PHASES = {"D2H": "d2h", "H2D": "h2d", "H2H": "host", "H2HReduce": "host", "D2D": "d2d", "D2DReduce": "reduce"}


def load(path):
    text = open(path).read().rstrip().rstrip(",")
    if not text.endswith("]") and not text.endswith("}"):
        text += "\n]"
    data = json.loads(text)
    return data.get("traceEvents", []) if isinstance(data, dict) else data


def clock_offset_us(events) -> float:
    """Microseconds to add to `ts` to obtain wall-clock microseconds."""
    for e in events:
        if e.get("ph") == "M" and e.get("name") == "clock":
            a = e["args"]
            return a["wall_epoch_us"] - a["steady_ns"] / 1000.0
    return 0.0


def percentile(xs, p):
    if not xs:
        return 0.0
    xs = sorted(xs)
    k = (len(xs) - 1) * p / 100.0
    lo, hi = int(k), min(int(k) + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def pct_str(xs):
    return " ".join(f"p{p}={percentile(xs, p):.1f}" for p in (0, 50, 90, 99, 100))


def human(n):
    for unit, sh in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= 1 << sh:
            return f"{n / (1 << sh):.4g} {unit}"
    return f"{n} B"


def complete_events(events, cat=None):
    return [e for e in events if e.get("ph") == "X" and (cat is None or e.get("cat") == cat)]


def iterations(events):
    """(collective event, its slices) per round on the PCIe path, per executor thread."""
    out = []
    by_tid = defaultdict(list)
    for e in complete_events(events, "dma"):
        by_tid[e.get("tid")].append(e)
    for it in sorted(complete_events(events, "pcie"), key=lambda e: e["ts"]):
        t0, t1 = it["ts"], it["ts"] + it["dur"]
        slices = [s for s in by_tid.get(it.get("tid"), []) if t0 <= s["ts"] and s["ts"] + s["dur"] <= t1 + 1.0]
        out.append((it, slices))
    return out


def span(evts):
    if not evts:
        return 0.0, 0.0
    return min(e["ts"] for e in evts), max(e["ts"] + e["dur"] for e in evts)


def union_length(evts):
    total, end = 0.0, None
    for s, d in sorted((e["ts"], e["dur"]) for e in evts):
        if end is None or s > end:
            total += d
            end = s + d
        elif s + d > end:
            total += s + d - end
            end = s + d
    return total


# ------------------------------------------------------------------ sub-commands
def cmd_summary(a):
    for path in a.files:
        ev = load(path)
        spans = defaultdict(list)
        for e in complete_events(ev):
            key = (e.get("cat", ""), e.get("name", "")) if a.per_op else (e.get("cat", ""),)
            spans[key].append(e)
        print(f"== {path}: {len(ev)} events")
        for key, xs in sorted(spans.items()):
            t0, t1 = span(xs)
            total = sum(e["dur"] for e in xs)
            nbytes = sum(e.get("args", {}).get("bytes", 0) for e in xs)
            bw = f" {nbytes / total / 1e3:8.2f} GB/s" if nbytes and total else ""
            print(f"  {'/'.join(key):<28} n={len(xs):<7} total={total / 1e3:9.3f} ms mean={total / len(xs):9.2f} us "
                  f"busy={100 * total / (t1 - t0) if t1 > t0 else 0:5.1f}%{bw}")
    return 0


def cmd_phases(a):
    for path in a.files:
        its = iterations(load(path))
        print(f"== {path}: {len(its)} collectives on the PCIe path")
        agg = defaultdict(list)
        for k, (it, slices) in enumerate(its):
            ph = defaultdict(list)
            for s in slices:
                ph[PHASES.get(s["name"], "other")].append(s)
            busy = union_length(slices)
            parts = []
            for name in ("d2h", "host", "h2d", "reduce", "d2d"):
                if ph[name]:
                    t0, t1 = span(ph[name])
                    parts.append(f"{name} {t1 - t0:8.1f} us")
                    agg[name].append(t1 - t0)
            overlap = sum(union_length(v) for v in ph.values()) - busy
            agg["idle"].append(it["dur"] - busy)
            agg["overlap"].append(overlap)
            if k < a.show:
                print(f"  #{k:<3} {it['name']:<14} {human(it.get('args', {}).get('bytes', 0)):>10} total {it['dur']:9.1f} us | " + " | ".join(parts) +
                      f" | overlapped {overlap:8.1f} us | nothing in flight {it['dur'] - busy:8.1f} us")
        for name, xs in agg.items():
            print(f"  {name:<8} {pct_str(xs)} (us)")
    return 0


def cmd_by_size(a):
    for path in a.files:
        groups = defaultdict(list)
        for it, slices in iterations(load(path)):
            groups[(it["name"], it.get("args", {}).get("bytes", 0))].append((it, slices))
        print(f"== {path}")
        print(f"  {'collective':<14} {'bytes':>10} {'n':>4} {'p50 us':>10} {'p99 us':>10} {'algbw GB/s':>11} {'slices':>7} {'slice p50 us':>13}")
        for (name, nbytes), xs in sorted(groups.items(), key=lambda kv: (kv[0][0], kv[0][1])):
            lat = [it["dur"] for it, _ in xs]
            sl = [s["dur"] for _, ss in xs for s in ss]
            p50 = percentile(lat, 50)
            print(f"  {name:<14} {human(nbytes):>10} {len(xs):>4} {p50:>10.1f} {percentile(lat, 99):>10.1f} "
                  f"{nbytes / p50 / 1e3 if p50 else 0:>11.2f} {len(sl) // max(1, len(xs)):>7} {percentile(sl, 50):>13.1f}")
    return 0


def cmd_host(a):
    for path in a.files:
        host = [e for e in complete_events(load(path), "dma") if e["name"] in ("H2H", "H2HReduce")]
        print(f"== {path}: {len(host)} host slices")
        if not host:
            continue
        for name in ("H2H", "H2HReduce"):
            xs = [e for e in host if e["name"] == name]
            if not xs:
                continue
            dur = [e["dur"] for e in xs]
            med = percentile(dur, 50)
            nbytes = sum(e.get("args", {}).get("bytes", 0) for e in xs)
            slow = [e for e in xs if e["dur"] > a.straggler * med]
            print(f"  {name:<10} n={len(xs)} {pct_str(dur)} us, {nbytes / sum(dur) / 1e3 if nbytes else 0:.2f} GB/s per slice, "
                  f"{len(slow)} stragglers (> {a.straggler:g} x median)")
            by_tid = defaultdict(int)
            for e in slow:
                by_tid[e.get("tid")] += 1
            for tid, k in sorted(by_tid.items(), key=lambda kv: -kv[1])[:8]:
                print(f"    thread {tid}: {k}")
    return 0


def cmd_compare(a):
    if len(a.files) % 2:
        raise SystemExit("compare takes pairs: <trace> <label> ...")
    print(f"per-slice latency of {a.op} (us)")
    for path, label in zip(a.files[::2], a.files[1::2]):
        ev = [e for e in complete_events(load(path), "dma") if e["name"] == a.op]
        dur = [e["dur"] for e in ev]
        nbytes = sum(e.get("args", {}).get("bytes", 0) for e in ev)
        t0, t1 = span(ev)
        print(f"  {label:<16} n={len(ev):<6} {pct_str(dur)} | span {t1 - t0:10.1f} us | {nbytes / (t1 - t0) / 1e3 if t1 > t0 else 0:7.2f} GB/s over the span")
    return 0


def cmd_merge(a):
    merged = []
    for path in a.files:
        ev = load(path)
        off = clock_offset_us(ev)
        for e in ev:
            merged.append(dict(e, ts=e["ts"] + off) if "ts" in e else e)
    if a.timeline:
        # a kernel timeline (utils.kernel_timeline --json): records {"rank", "call", "kernel", "phases": [[name, t0_ns, t1_ns], ...], "wall_offset_us"}
        for rec in json.load(open(a.timeline)):
            off = rec.get("wall_offset_us", 0.0)
            for name, t0, t1 in rec.get("phases", []):
                merged.append({"name": f"{rec.get('kernel', 'kernel')}:{name}", "cat": "kernel", "ph": "X", "pid": 0, "tid": 900000 + rec.get("rank", 0),
                               "ts": t0 / 1000.0 + off, "dur": (t1 - t0) / 1000.0})
    with open(a.out, "w") as f:
        json.dump(merged, f)
    print(f"merged {len(merged)} events into {a.out}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd")
    p = sub.add_parser("summary")
    p.add_argument("files", nargs="+")
    p.add_argument("--per-op", action="store_true")
    p = sub.add_parser("phases")
    p.add_argument("files", nargs="+")
    p.add_argument("--show", type=int, default=8, help="iterations printed one by one")
    p = sub.add_parser("by-size")
    p.add_argument("files", nargs="+")
    p = sub.add_parser("host")
    p.add_argument("files", nargs="+")
    p.add_argument("--straggler", type=float, default=3.0)
    p = sub.add_parser("compare")
    p.add_argument("files", nargs="+")
    p.add_argument("--op", default="D2H")
    p = sub.add_parser("merge")
    p.add_argument("files", nargs="+")
    p.add_argument("-o", "--out", required=True)
    p.add_argument("--timeline")
    import sys

    args = list(sys.argv[1:] if argv is None else argv)
    # the old form (files first, --per-op / --merge OUT as options) keeps working
    if args and args[0] not in ("summary", "phases", "by-size", "host", "compare", "merge", "-h", "--help"):
        if "--merge" in args:   # the summary first, then the merged file
            k = args.index("--merge")
            out = args[k + 1]
            rest = [x for i, x in enumerate(args) if i not in (k, k + 1)]
            cmd_summary(ap.parse_args(["summary"] + rest))
            args = ["merge"] + [x for x in rest if x != "--per-op"] + ["-o", out]
        else:
            args = ["summary"] + args
    a = ap.parse_args(args)
    if not a.cmd:
        ap.print_help()
        return 1
    return {"summary": cmd_summary, "phases": cmd_phases, "by-size": cmd_by_size, "host": cmd_host, "compare": cmd_compare,
            "merge": cmd_merge}[a.cmd](a)


if __name__ == "__main__":
    raise SystemExit(main())
