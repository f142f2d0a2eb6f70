"""Chrome-trace writer and the analysis / tracer-parser tools (no GPU)."""
import json
import os
import subprocess
import sys

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _traced_worker(rank, n, uid, path):
    import torch

    from hylink_b200._native import lib
    from hylink_b200.parallel.comm import Communicator

    lib.hlTraceOpen(path.replace("%r", str(rank)).encode(), rank)
    c = Communicator(rank, n, uid=uid, device=-2)
    x = torch.ones(1 << 18)
    for _ in range(3):
        c.all_reduce(x)
        c.drain()
    c.close()
    lib.hlTraceOpen(b"", rank)  # closes the file
    return True


def test_trace_file_is_valid_and_analysable(tmp_path):
    pat = str(tmp_path / "trace.%r.json")
    run_ranks(_traced_worker, 2, pat, env={"HYLINK_HOST_BUFFER_SIZE": "64M", "HYLINK_INTERNAL_BUFFER_BYTES": "32M"})
    files = [pat.replace("%r", str(r)) for r in range(2)]
    for f in files:
        ev = json.load(open(f))
        assert ev[0]["ph"] == "M" and "wall_epoch_us" in ev[0]["args"]
        names = {e["name"] for e in ev if e.get("ph") == "X"}
        assert "allreduce" in names and {"D2H", "H2D"} <= names
    merged = str(tmp_path / "merged.json")
    out = subprocess.run([sys.executable, "-m", "hylink_b200.utils.trace_analysis", *files, "--per-op", "--merge", merged],
                         cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "pcie/allreduce" in out.stdout, out.stdout + out.stderr
    assert len(json.load(open(merged))) > 20
    # the per-iteration, per-size, host-slice and cross-file reports
    for args, needle in ((["phases", files[0]], "nothing in flight"), (["by-size", files[0]], "algbw"), (["host", files[0]], "host slices"),
                         (["compare", files[0], "rank0", files[1], "rank1", "--op", "D2H"], "rank1"), (["summary", files[0]], "dma")):
        out = subprocess.run([sys.executable, "-m", "hylink_b200.utils.trace_analysis", *args], cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT),
                             capture_output=True, text=True, timeout=120)
        assert out.returncode == 0 and needle in out.stdout, (args, out.stdout + out.stderr)
    ev = json.load(open(merged))
    assert any(e.get("cat") == "dma" and e.get("args", {}).get("bytes", 0) > 0 for e in ev), "slices carry their byte counts"


def test_nccl_trace_parser(tmp_path):
    f = tmp_path / "t.jsonl"
    rows = [{"seq": i, "pid": 1, "call": "ncclAllReduce", "t": 10.0 + i, "host_us": 5.0, "count": 1 << 20, "dtype": 9, "op": 0,
             "peer": -1, "comm": "0x1", "stream": "0x2", "capturing": i % 2, "rc": 0} for i in range(4)]
    f.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    out = subprocess.run([sys.executable, "-m", "hylink_b200.utils.nccl_trace_parse", str(f)], cwd=ROOT,
                         env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=60)
    assert out.returncode == 0
    line = [l for l in out.stdout.splitlines() if l.startswith("ncclAllReduce")][0].split()
    assert line[1] == str(2 << 20) and line[2] == "4" and line[5] == "2"


def test_orchestrator_log_lines_parse_into_per_call_rows(tmp_path):
    from hylink_b200.utils import compare

    log = """[hylink] (max) fast_time=0.000498s
[hylink] (max) pcie_time=0.000626s
[hylink] aggregate op=AllReduce op_key_bytes=268435456 base_bytes=268435456 alg_bytes=268435456 n=2 | fast_bytes=264865280 pcie_bytes=3570176 split_fast=0.9867 split_pcie=0.0133 | fast_bw(GB/s,decimal)=531.858 pcie_bw(GB/s,decimal)=5.703 | algbw(GB/s,decimal)=428.811 busbw(GB/s,decimal)=428.811 bus_factor=1.0000
[hylink] Total bw is 428.811000 GB/s
noise line
[hylink] (max) fast_time=0.000500s
[hylink] (max) pcie_time=0.000600s
[hylink] aggregate op=AllGather op_key_bytes=1048576 base_bytes=1048576 alg_bytes=2097152 n=2 | fast_bytes=1000000 pcie_bytes=48576 split_fast=0.9537 split_pcie=0.0463 | fast_bw(GB/s,decimal)=2.000 pcie_bw(GB/s,decimal)=0.081 | algbw(GB/s,decimal)=3.495 busbw(GB/s,decimal)=1.748 bus_factor=0.5000
[hylink] Total bw is 1.748000 GB/s
"""
    recs = compare.parse_log(log.splitlines())
    assert [r["op"] for r in recs] == ["AllReduce", "AllGather"]
    assert recs[0]["pcie_bytes"] == 3570176 and abs(recs[0]["split_pcie"] - 0.0133) < 1e-9
    assert abs(recs[0]["fast_time_s"] - 0.000498) < 1e-12 and abs(recs[1]["pcie_time_s"] - 0.0006) < 1e-12
    assert recs[1]["total_bw_GBs"] == 1.748
    f = tmp_path / "run.log"
    f.write_text(log)
    assert compare.main(["logs", str(f), "--csv", str(tmp_path / "calls.csv")]) == 0
    assert (tmp_path / "calls.csv").read_text().count("\n") == 3


def test_sweep_files_merge_into_one_table(tmp_path):
    import json

    from hylink_b200.utils import compare

    def row(busbw, nccl):
        return json.dumps({"coll": "allreduce", "dtype": "bf16", "bytes": 1 << 20, "n": 2, "ms": 0.1, "busbw_GBs": busbw,
                           "nccl_ms": 0.1, "nccl_busbw_GBs": nccl, "speedup": 1.0, "ok": True, "algo": "auto", "path": "x"})

    (tmp_path / "nvlink_2gpu.jsonl").write_text(row(50.0, 40.0) + "\n")
    (tmp_path / "adaptive_2gpu.jsonl").write_text(row(30.0, 41.0) + "\n")
    labels, table = compare.merge_sweeps([str(tmp_path / "nvlink_2gpu.jsonl"), str(tmp_path / "adaptive_2gpu.jsonl")])
    rows = compare.write_sweep_tables(labels, table, str(tmp_path / "s.csv"), str(tmp_path / "s.md"))
    assert rows == [["allreduce", "bf16", 1 << 20, 2, 50.0, 30.0, 41.0, round(50 / 41, 3), round(30 / 41, 3)]]
    assert "nvlink_2gpu/NCCL" in (tmp_path / "s.md").read_text()


def test_sweep_files_plot_as_svg_without_a_plotting_library(tmp_path):
    import json
    import xml.dom.minidom

    from hylink_b200.utils import compare

    def rows(scale, n):
        return "\n".join(json.dumps({"coll": c, "dtype": "bf16", "bytes": 1 << s, "n": n, "ms": 0.1, "busbw_GBs": scale * s,
                                     "nccl_ms": 0.1, "nccl_busbw_GBs": 0.8 * scale * s, "speedup": 1.25, "ok": True,
                                     "algo": "auto", "path": "x"}) for c in ("allreduce", "allgather") for s in range(10, 31, 4)) + "\n"

    (tmp_path / "nvlink_2gpu.jsonl").write_text(rows(10.0, 2))
    (tmp_path / "nvlink_4gpu.jsonl").write_text(rows(12.0, 4))
    out = tmp_path / "charts"
    assert compare.main(["plot", str(tmp_path / "nvlink_2gpu.jsonl"), str(tmp_path / "nvlink_4gpu.jsonl"), "--out", str(out)]) == 0
    files = sorted(p.name for p in out.iterdir())
    assert files == ["busbw_allgather_bf16.svg", "busbw_allreduce_bf16.svg"]
    doc = xml.dom.minidom.parse(str(out / "busbw_allreduce_bf16.svg"))
    lines = doc.getElementsByTagName("polyline")
    assert len(lines) == 4                                   # two runs and NCCL's line for each rank count
    assert sum(1 for l in lines if l.getAttribute("stroke-dasharray")) == 2
    assert all(len(l.getAttribute("points").split()) == 6 for l in lines)
    labels = [t.firstChild.data for t in doc.getElementsByTagName("text") if t.firstChild]
    assert "nvlink_2gpu" in labels and "NCCL (4 GPUs)" in labels and "1G" in labels


def test_interference_runs_plot_as_two_charts(tmp_path):
    import json
    import xml.dom.minidom

    from hylink_b200.utils import compare

    def run(alpha):
        rows = [json.dumps({"event": "nvlink_only", "interference_pct": 0, "ms": 0.5, "busbw_GBs": 600.0})]
        for i in range(40):
            lvl = (0, 25, 50, 75)[i // 10]
            rows.append(json.dumps({"iter": i, "interference_pct": lvl, "ms": 1.0, "busbw_GBs": 400.0 - lvl, "alpha": alpha / (1 + lvl / 25),
                                    "fast_ms": 0.7, "pcie_ms": 0.9}))
        return "\n".join(rows) + "\n"

    (tmp_path / "split_ratio.jsonl").write_text(run(0.04))
    (tmp_path / "static.jsonl").write_text(run(0.05))
    out = tmp_path / "charts"
    assert compare.main(["interference", str(tmp_path / "split_ratio.jsonl"), str(tmp_path / "static.jsonl"), "--out", str(out)]) == 0
    for name in ("interference_busbw_per_call.svg", "interference_pcie_share_per_call.svg"):
        doc = xml.dom.minidom.parse(str(out / name))
        lines = doc.getElementsByTagName("polyline")
        assert len(lines) == 2 and all(len(l.getAttribute("points").split()) == 40 for l in lines)
        captions = [t.firstChild.data for t in doc.getElementsByTagName("text") if t.firstChild]
        assert [c for c in captions if c.endswith("% load")] == ["0 % load", "25 % load", "50 % load", "75 % load"]
        assert "split_ratio" in captions and "static" in captions


def test_kernel_timeline_decoder_on_a_synthetic_ring():
    from hylink_b200.utils import kernel_timeline as kt

    words = [0] * (kt.TL_CALLS * kt.TL_BLOCKS * kt.TL_PHASES + kt.TL_CALLS * 4)
    slot, blocks = 3, 2
    meta = kt.TL_CALLS * kt.TL_BLOCKS * kt.TL_PHASES + 4 * slot
    words[meta:meta + 4] = [12, (15 << 32) | blocks, 4096, 0]
    for b in range(blocks):
        base = (slot * kt.TL_BLOCKS + b) * kt.TL_PHASES
        t0 = 1_000_000 + 100 * b
        words[base:base + 8] = [t0, t0 + 5000, t0 + 6000, t0 + 9000, t0 + 9500, 0, 0, t0 + 12000]
    launches = kt.decode(words)
    assert len(launches) == 1 and launches[0]["kind"] == "allreduce_push" and launches[0]["blocks"] == 2
    s = kt.summarise(launches[0])
    assert s["phases"]["entry->arrive1"]["median_us"] == 5.0 and s["phases"]["leave2->exit"]["median_us"] == 2.5
    assert s["entry_spread_us"] == 0.1 and s["total_us"] == 12.1


def test_kernel_timeline_decoder_reads_lane_kernel_sums():
    from hylink_b200.utils import kernel_timeline as kt

    words = [0] * (kt.TL_CALLS * kt.TL_BLOCKS * kt.TL_PHASES + kt.TL_CALLS * 4)
    meta = kt.TL_CALLS * kt.TL_BLOCKS * kt.TL_PHASES
    words[meta:meta + 4] = [0, (13 << 32) | 4, 1 << 20, 0]   # reducescatter_pipelined_p2p, 4 CTAs = 2 lanes of push + fold
    for b in range(4):
        t0, role = 5_000_000, b % 2
        base = b * kt.TL_PHASES
        words[base:base + 8] = [t0, t0 + (3000 if role else 0), t0 + (0 if role else 40000), t0 + 60000, t0 + role * 1000000, 0, 0, t0 + 100000]
    s = kt.summarise(kt.decode(words)[0])
    assert s["stages"]["push"] == {"ctas": 2, "waiting_us": 0.0, "handing_on_us": 40.0, "working_us": 60.0, "total_us": 100.0}
    assert s["stages"]["fold"]["waiting_us"] == 3.0 and s["total_us"] == 100.0
