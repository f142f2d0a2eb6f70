"""Comparison pipeline: turn bandwidth sweeps and orchestrator logs into tables.

    python -m hylink_b200.utils.compare sweeps nccl_vs_ours.jsonl [more.jsonl ...] [--csv out.csv] [--md out.md]
    python -m hylink_b200.utils.compare logs run.log [--csv per_call.csv]
    python -m hylink_b200.utils.compare pipeline --gpus 2,4,8 --out results/ [--bytes-from 1K --bytes-to 1G --factor 4]

* ``sweeps`` merges the JSON lines written by ``hylink_b200.utils.sweep`` (one file per configuration, the file
  name is the label) into one table: a row per (collective, dtype, bytes, ranks), the bus bandwidth of every
  labelled run, NCCL's, and the ratios.
* ``logs`` reads the aggregate lines that the orchestrator prints for forked collectives (``aggregate op=…``,
  ``(max) fast_time=…``, ``(max) pcie_time=…``, ``Total bw is …``) and writes one row per call: bytes on each
  path, the split, per-path and bus bandwidth. The wording of those lines is the reference's
  (multipath-orchestrator/libampccl/core/shm_store.cc:372-412), so its own post-processor
  (tests/nccl_test/test_scripts/process_compare_logs.py:36-38) reads them too.
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
    args = ap.parse_args(argv)
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
