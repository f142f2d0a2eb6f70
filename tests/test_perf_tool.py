"""The stand-alone test executable (hl_perf), on the host-memory device: every collective, ranks as threads and as
forked processes, the strided configurations, and the output lines that log post-processors rely on.

Mirrors how the reference tests its libraries: stand-alone executables that return an exit code
(pcie-ccl-cuda/tests/coll/test_allreduce.cpp:52-113, tests/coll/test_reducescatter_strided.cpp:130-150)."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "hylink_b200", "bin", "hl_perf")


def _run(args, timeout=180):
    if not os.path.exists(BIN):
        from hylink_b200 import _build

        _build.build_core()
        _build.build_tools()
    env = dict(os.environ, HYLINK_HOST_BUFFER_SIZE="64M", HYLINK_INTERNAL_BUFFER_BYTES="32M")
    p = subprocess.run([BIN] + args, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env)
    return p.returncode, p.stdout


@pytest.mark.parametrize("coll", ["allreduce", "allgather", "reducescatter", "alltoall", "broadcast"])
def test_every_collective_with_ranks_as_threads(coll):
    rc, out = _run(["--coll", coll, "--ranks", "2", "--mode", "threads", "--device", "host", "--bytes-from", "1K",
                    "--bytes-to", "1M", "--factor", "32", "--iters", "2"])
    assert rc == 0 and "Test PASSED." in out, out[-2000:]
    assert out.count("| ") and " NO" not in out


def test_four_forked_ranks_bf16_and_output_contract():
    rc, out = _run(["--coll", "allreduce", "--ranks", "4", "--mode", "fork", "--device", "host", "--dtype", "bf16",
                    "--bytes-from", "64K", "--bytes-to", "64K", "--iters", "3", "--per-iter"])
    assert rc == 0, out[-2000:]
    assert "Warmup done (2 iters)" in out
    assert len(re.findall(r"^iter \d+: [\d.]+ ms \(host\), bandwidth: [\d.]+ GB/s$", out, re.M)) == 3
    assert re.search(r"^Average bandwidth over 3 iters \(host\): [\d.]+ GB/s$", out, re.M)
    assert re.search(r"Size \| Avg Lat\(ms\) \|\s+Alg BW\(GB/s\) \|\s+Bus BW\(GB/s\) \| Correct", out)
    for r in range(4):
        assert f"rank {r}: PASSED" in out
    assert out.rstrip().endswith("Test PASSED.")


@pytest.mark.parametrize("coll", ["allgather", "reducescatter", "alltoall"])
def test_strided_calls_leave_the_other_transports_prefix_alone(coll):
    rc, out = _run(["--coll", coll, "--ranks", "2", "--mode", "threads", "--device", "host", "--strided", "--dtype", "fp16",
                    "--bytes-from", "256K", "--bytes-to", "256K", "--iters", "2"])
    assert rc == 0 and "Test PASSED." in out, out[-2000:]
    for share in (75, 50, 25, 0):
        assert f"[{share}% other]" in out


def test_bad_arguments_are_refused():
    rc, out = _run(["--coll", "nonsense"])
    assert rc == 2 and "usage:" in out
