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
