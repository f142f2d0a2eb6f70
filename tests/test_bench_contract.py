"""The parts of ``bench.py`` that can be checked without a GPU: its helpers and what it prints on stdout."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    sys.path.insert(0, ROOT)
    try:
        import bench
    finally:
        sys.path.pop(0)
    return bench


def test_sizes_factors_and_geomean():
    b = _bench()
    sizes = b.size_list(b.parse_size("1M"), b.parse_size("1G"))
    assert sizes[0] == 1 << 20 and sizes[-1] == 1 << 30 and len(sizes) == 11          # powers of two, 33 cells with 3 collectives
    assert b.bus_factor("allreduce", 8) == 2 * 7 / 8 and b.bus_factor("allgather", 4) == 3 / 4
    assert b.bus_factor("allreduce", 1) == 1.0 and b.bus_factor("reducescatter", 1) == 1.0
    assert abs(b.geomean([1.0, 100.0]) - 10.0) < 1e-9
    assert b.human(1 << 30) == "1 GiB" and b.human(3 << 20) == "3 MiB"


def test_reference_arm_answers_with_one_json_line_when_it_cannot_run():
    """An N the reference ships no schedules for: exit code 0, stdout is the `unavailable` record and nothing else."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "3", "--steps", "1"],
                       cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, p.stdout
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["n_gpus"] == 3 and "3 GPUs" in rec["unavailable"]


def test_stdout_carries_records_only():
    """Whatever libraries print from C while the script runs goes to stderr; JSON records go to the real stdout."""
    code = (
        "import os, sys, ctypes\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import bench\n"
        "def fake_main():\n"
        "    ctypes.CDLL(None).puts(b'library chatter from C')\n"
        "    print('progress line')\n"
        "    print('{\"value\": 1}')\n"
        "    return 0\n"
        "bench.main = fake_main\n"
        "sys.exit(bench._main_with_clean_stdout())\n")
    p = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout == '{"value": 1}\n', (p.stdout, p.stderr)
    assert "library chatter from C" in p.stderr and "progress line" in p.stderr
