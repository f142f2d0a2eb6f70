"""Comparison pipeline: turn bandwidth sweeps and orchestrator logs into tables.

    python -m hylink_b200.utils.compare sweeps nccl_vs_ours.jsonl [more.jsonl ...] [--csv out.csv] [--md out.md]
    python -m hylink_b200.utils.compare logs run.log [--csv per_call.csv]
    python -m hylink_b200.utils.compare pipeline --gpus 2,4,8 --out results/ [--bytes-from 1K --bytes-to 1G --factor 4]
    python -m hylink_b200.utils.compare plot nvlink_2gpu.jsonl adaptive_2gpu.jsonl ... --out charts/ [--dtype bf16]
    python -m hylink_b200.utils.compare interference split_ratio.jsonl static.jsonl --out charts/

* ``sweeps`` merges the JSON lines written by ``hylink_b200.utils.sweep`` (one file per configuration, the file
  name is the label) into one table: a row per (collective, dtype, bytes, ranks), the bus bandwidth of every
  labelled run, NCCL's, and the ratios.
* ``logs`` reads the aggregate lines that the orchestrator prints for forked collectives (``aggregate op=…``,
  ``(max) fast_time=…``, ``(max) pcie_time=…``, ``Total bw is …``) and writes one row per call: bytes on each
  path, the split, per-path and bus bandwidth. The wording of those lines is the reference's
  (multipath-orchestrator/libampccl/core/shm_store.cc:372-412), so its own post-processor
  (tests/nccl_test/test_scripts/process_compare_logs.py:36-38) reads them too.
* ``plot`` draws one chart per collective from sweep files (bus bandwidth against message size, log x axis, one
  line per file plus NCCL's per rank count) as plain SVG, written without any plotting library
  (tests/nccl_test/test_scripts/plot_bw_comparison.py in the reference, which needs matplotlib). ``pipeline`` calls it.
* ``interference`` draws the two charts of the interference experiment from the files written by
  ``hylink_b200.utils.interference --out``: bus bandwidth per call and PCIe share per call, one line per controller,
  the load levels marked.
* ``pipeline`` runs the sweep for every GPU count in two configurations — NVLink kernels only, and the adaptive
  multipath split — each against NCCL in the same process, and merges the results
  (tests/nccl_test/test_scripts/run_full_pipeline.sh in the reference: baseline vs adaptive x {AG, AR, RS} x
  {2, 4, 8} GPUs x 1 KB…1 GB).
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import subprocess
import sys

_AGG = re.compile(
    r"aggregate op=(?P<op>\S+) op_key_bytes=(?P<key>\d+) base_bytes=\d+ alg_bytes=(?P<alg>[\d.]+) n=(?P<n>\d+) \| "
    r"fast_bytes=(?P<fast_bytes>\d+) pcie_bytes=(?P<pcie_bytes>\d+) split_fast=(?P<split_fast>[\d.]+) split_pcie=(?P<split_pcie>[\d.]+) \| "
    r"fast_bw\(GB/s,decimal\)=(?P<fast_bw>[\d.]+) pcie_bw\(GB/s,decimal\)=(?P<pcie_bw>[\d.]+) \| "
    r"algbw\(GB/s,decimal\)=(?P<algbw>[\d.]+) busbw\(GB/s,decimal\)=(?P<busbw>[\d.]+) bus_factor=(?P<factor>[\d.]+)")
_FAST = re.compile(r"\(max\) fast_time=([\d.eE+-]+)s")
_PCIE = re.compile(r"\(max\) pcie_time=([\d.eE+-]+)s")
_TOTAL = re.compile(r"Total bw is ([\d.]+) GB/s")


def parse_log(lines):
    """One dict per forked call, in log order."""
    out, fast_t, pcie_t = [], None, None
    for line in lines:
        m = _FAST.search(line)
        if m:
            fast_t = float(m.group(1))
            continue
        m = _PCIE.search(line)
        if m:
            pcie_t = float(m.group(1))
            continue
        m = _AGG.search(line)
        if m:
            d = m.groupdict()
            rec = {"call": len(out), "op": d["op"], "bytes": int(d["key"]), "nranks": int(d["n"]),
                   "fast_bytes": int(d["fast_bytes"]), "pcie_bytes": int(d["pcie_bytes"]),
                   "split_pcie": float(d["split_pcie"]), "fast_time_s": fast_t, "pcie_time_s": pcie_t,
                   "fast_bw_GBs": float(d["fast_bw"]), "pcie_bw_GBs": float(d["pcie_bw"]),
                   "algbw_GBs": float(d["algbw"]), "busbw_GBs": float(d["busbw"])}
            out.append(rec)
            fast_t = pcie_t = None
            continue
        m = _TOTAL.search(line)
        if m and out and "total_bw_GBs" not in out[-1]:
            out[-1]["total_bw_GBs"] = float(m.group(1))
    return out


def merge_sweeps(files):
    """rows keyed by (coll, dtype, bytes, n) -> {label: busbw, 'nccl': busbw}."""
    table, labels = {}, []
    for f in files:
        label = os.path.splitext(os.path.basename(f))[0]
        labels.append(label)
        with open(f) as fh:
            for line in fh:
                if not line.startswith('{"coll"'):
                    continue
                r = json.loads(line)
                key = (r["coll"], r["dtype"], r["bytes"], r["n"])
                row = table.setdefault(key, {})
                row[label] = r["busbw_GBs"]
                if r.get("nccl_busbw_GBs"):
                    row["nccl"] = max(row.get("nccl", 0.0), r["nccl_busbw_GBs"])
    return labels, table


def write_sweep_tables(labels, table, csv_path=None, md_path=None, out=sys.stdout):
    head = ["collective", "dtype", "bytes", "ranks"] + [f"{l} GB/s" for l in labels] + ["NCCL GB/s"] + [f"{l}/NCCL" for l in labels]
    rows = []
    for key in sorted(table, key=lambda k: (k[3], k[0], k[1], k[2])):
        row = table[key]
        nccl = row.get("nccl")
        rows.append(list(key) + [row.get(l, "") for l in labels] + [nccl if nccl else ""] +
                    [round(row[l] / nccl, 3) if (nccl and l in row) else "" for l in labels])
    if csv_path:
        with open(csv_path, "w", newline="") as fh:
            w = csv.writer(fh)
            w.writerow(head)
            w.writerows(rows)
    md = ["| " + " | ".join(head) + " |", "|" + "|".join(["---"] * len(head)) + "|"] + \
         ["| " + " | ".join(str(v) for v in r) + " |" for r in rows]
    if md_path:
        with open(md_path, "w") as fh:
            fh.write("\n".join(md) + "\n")
    else:
        print("\n".join(md), file=out)
    return rows


_COLOURS = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e", "#8c564b", "#17becf", "#7f7f7f", "#bcbd22", "#e377c2"]


def _size_label(b: int) -> str:
    for unit, sh in (("G", 30), ("M", 20), ("K", 10)):
        if b >= 1 << sh:
            v = b / (1 << sh)
            return (f"{v:.0f}" if v == int(v) else f"{v:.1f}") + unit
    return str(b)


def svg_chart(title: str, series: dict, path: str, width: int = 860, height: int = 480, logx: bool = True,
              xlabel: str = "message size (bytes)", ylabel: str = "bus bandwidth (GB/s)", marks=None) -> None:
    """series: label -> [(x, y), ...]. Log2 (message sizes) or linear x axis, linear y axis, dashed lines for labels
    that start with 'NCCL'; `marks`: [(x, text), ...] vertical lines with a caption. Plain SVG text, no dependencies."""
    import math

    fx = (lambda v: math.log2(v)) if logx else (lambda v: float(v))

    pts = [p for v in series.values() for p in v]
    if not pts:
        return
    x0, x1 = fx(min(p[0] for p in pts)), fx(max(p[0] for p in pts))
    if x1 == x0:
        x1 = x0 + 1
    ymax = max(p[1] for p in pts) * 1.08 or 1.0
    step = 10 ** math.floor(math.log10(ymax / 4))
    step = step * (5 if ymax / step > 20 else (2 if ymax / step > 8 else 1))
    ml, mr, mt, mb = 64, 190, 40, 48
    pw, ph = width - ml - mr, height - mt - mb

    def sx(b):
        return ml + (fx(b) - x0) / (x1 - x0) * pw

    def sy(v):
        return mt + ph - v / ymax * ph

    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
         f'<rect width="{width}" height="{height}" fill="white"/>',
         f'<text x="{ml + pw / 2}" y="22" text-anchor="middle" font-size="15">{title}</text>',
         f'<rect x="{ml}" y="{mt}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>']
    v = 0.0
    while v <= ymax:
        y = sy(v)
        o.append(f'<line x1="{ml}" y1="{y:.1f}" x2="{ml + pw}" y2="{y:.1f}" stroke="#ddd"/>')
        o.append(f'<text x="{ml - 6}" y="{y + 4:.1f}" text-anchor="end">{v:g}</text>')
        v += step
    xs = sorted({p[0] for p in pts})
    every = max(1, len(xs) // 10)
    for i, b in enumerate(xs):
        if i % every:
            continue
        x = sx(b)
        o.append(f'<line x1="{x:.1f}" y1="{mt + ph}" x2="{x:.1f}" y2="{mt + ph + 5}" stroke="#444"/>')
        o.append(f'<text x="{x:.1f}" y="{mt + ph + 20}" text-anchor="middle">{_size_label(b) if logx else b}</text>')
    for mx, text in (marks or []):
        x = sx(mx)
        o.append(f'<line x1="{x:.1f}" y1="{mt}" x2="{x:.1f}" y2="{mt + ph}" stroke="#999" stroke-dasharray="3 3"/>')
        o.append(f'<text x="{x + 4:.1f}" y="{mt + 12}" fill="#666">{text}</text>')
    o.append(f'<text x="{ml + pw / 2}" y="{height - 8}" text-anchor="middle">{xlabel}</text>')
    o.append(f'<text x="16" y="{mt + ph / 2}" text-anchor="middle" transform="rotate(-90 16 {mt + ph / 2})">{ylabel}</text>')
    for i, (label, data) in enumerate(series.items()):
        col = _COLOURS[i % len(_COLOURS)]
        data = sorted(data)
        dash = ' stroke-dasharray="6 4"' if label.startswith("NCCL") else ""
        o.append(f'<polyline fill="none" stroke="{col}" stroke-width="2"{dash} points="' +
                 " ".join(f"{sx(b):.1f},{sy(v):.1f}" for b, v in data) + '"/>')
        for b, v in data if len(data) <= 64 else []:
            o.append(f'<circle cx="{sx(b):.1f}" cy="{sy(v):.1f}" r="3" fill="{col}"/>')
        ly = mt + 14 + 18 * i
        o.append(f'<line x1="{ml + pw + 12}" y1="{ly - 4}" x2="{ml + pw + 36}" y2="{ly - 4}" stroke="{col}" stroke-width="2"{dash}/>')
        o.append(f'<text x="{ml + pw + 42}" y="{ly}">{label}</text>')
    o.append("</svg>")
    with open(path, "w") as fh:
        fh.write("\n".join(o) + "\n")


def plot_sweeps(files, out_dir: str, dtype: str = "bf16"):
    """One SVG per collective: a line per (file label, rank count) and NCCL's line per rank count."""
    os.makedirs(out_dir, exist_ok=True)
    labels, table = merge_sweeps(files)
    charts = {}
    for (coll, dt, nbytes, n), row in table.items():
        if dt != dtype:
            continue
        series = charts.setdefault(coll, {})
        for l in labels:
            if l in row:
                name = l if l.endswith("gpu") else f"{l} ({n} GPUs)"
                series.setdefault(name, []).append((nbytes, row[l]))
        if row.get("nccl"):
            series.setdefault(f"NCCL ({n} GPUs)", []).append((nbytes, row["nccl"]))
    written = []
    for coll, series in sorted(charts.items()):
        path = os.path.join(out_dir, f"busbw_{coll}_{dtype}.svg")
        svg_chart(f"{coll} - bus bandwidth ({dtype})", dict(sorted(series.items())), path)
        written.append(path)
    return written


def plot_interference(files, out_dir: str):
    """Per-call bus bandwidth and PCIe share of interference runs (the JSON lines of ``hylink_b200.utils.interference``,
    one file per controller), with the load levels marked: the two charts of the reference's experiment
    (tests/hccl_test/inference_experiment in the reference draws them with matplotlib)."""
    os.makedirs(out_dir, exist_ok=True)
    bw, share, marks = {}, {}, []
    for f in files:
        label = os.path.splitext(os.path.basename(f))[0]
        level = None
        with open(f) as fh:
            for line in fh:
                r = json.loads(line)
                if "iter" not in r:
                    continue
                bw.setdefault(label, []).append((r["iter"], r["busbw_GBs"]))
                share.setdefault(label, []).append((r["iter"], 100.0 * r["alpha"]))
                if r["interference_pct"] != level and f == files[0]:
                    level = r["interference_pct"]
                    marks.append((r["iter"], f"{level} % load"))
    a, b = os.path.join(out_dir, "interference_busbw_per_call.svg"), os.path.join(out_dir, "interference_pcie_share_per_call.svg")
    svg_chart("forked all-reduce under PCIe load - bus bandwidth per call", bw, a, logx=False, xlabel="call", marks=marks)
    svg_chart("forked all-reduce under PCIe load - share of the bytes on PCIe", share, b, logx=False, xlabel="call",
              ylabel="PCIe share (%)", marks=marks)
    return [a, b]


def run_pipeline(args) -> int:
    os.makedirs(args.out, exist_ok=True)
    produced = []
    for n in [int(v) for v in args.gpus.split(",")]:
        for label, path, env in (("nvlink", "nvlink", {}), ("adaptive", "auto", {"HYLINK_ORCH_ENABLE": "1", "HYLINK_PCIE_ENABLE": "1"})):
            dst = os.path.join(args.out, f"{label}_{n}gpu.jsonl")
            if os.path.exists(dst):
                os.remove(dst)
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
                   "127.0.0.1", "--master-port", str(args.port), "-m", "hylink_b200.utils.sweep", "--colls", args.colls,
                   "--dtypes", args.dtypes, "--bytes-from", args.lo, "--bytes-to", args.hi, "--factor", str(args.factor),
                   "--path", path, "--out", dst] + (["--iters", str(args.iters)] if args.iters else [])
            print("+", " ".join(cmd), flush=True)
            p = subprocess.run(cmd, env=dict(os.environ, **env))
            if p.returncode != 0:
                print(f"sweep failed for {label} on {n} GPUs (exit {p.returncode})", file=sys.stderr)
                return p.returncode
            produced.append(dst)
    labels, table = merge_sweeps(produced)
    write_sweep_tables(labels, table, os.path.join(args.out, "summary.csv"), os.path.join(args.out, "summary.md"))
    print("wrote", os.path.join(args.out, "summary.csv"))
    for dt in args.dtypes.split(","):
        for path in plot_sweeps(produced, args.out, dt):
            print("wrote", path)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("sweeps")
    p.add_argument("files", nargs="+")
    p.add_argument("--csv")
    p.add_argument("--md")
    p = sub.add_parser("logs")
    p.add_argument("files", nargs="+")
    p.add_argument("--csv")
    p = sub.add_parser("pipeline")
    p.add_argument("--gpus", default="2,4,8")
    p.add_argument("--out", required=True)
    p.add_argument("--colls", default="allreduce,reducescatter,allgather")
    p.add_argument("--dtypes", default="bf16")
    p.add_argument("--bytes-from", dest="lo", default="1K")
    p.add_argument("--bytes-to", dest="hi", default="1G")
    p.add_argument("--factor", type=int, default=4)
    p.add_argument("--iters", type=int, default=0)
    p.add_argument("--port", type=int, default=29671)
    p = sub.add_parser("plot")
    p.add_argument("files", nargs="+")
    p.add_argument("--out", default=".")
    p.add_argument("--dtype", default="bf16")
    p = sub.add_parser("interference")
    p.add_argument("files", nargs="+")
    p.add_argument("--out", default=".")
    args = ap.parse_args(argv)
    if args.cmd == "interference":
        for path in plot_interference(args.files, args.out):
            print("wrote", path)
        return 0
    if args.cmd == "plot":
        for path in plot_sweeps(args.files, args.out, args.dtype):
            print("wrote", path)
        return 0
    if args.cmd == "sweeps":
        labels, table = merge_sweeps(args.files)
        write_sweep_tables(labels, table, args.csv, args.md)
        return 0
    if args.cmd == "logs":
        recs = []
        for f in args.files:
            with open(f) as fh:
                recs += parse_log(fh)
        if args.csv and recs:
            with open(args.csv, "w", newline="") as fh:
                w = csv.DictWriter(fh, fieldnames=sorted({k for r in recs for k in r}))
                w.writeheader()
                w.writerows(recs)
        for r in recs:
            print(json.dumps(r))
        return 0
    return run_pipeline(args)


if __name__ == "__main__":
    sys.exit(main())
