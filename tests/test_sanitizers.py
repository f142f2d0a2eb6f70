"""Host plumbing under ThreadSanitizer and AddressSanitizer: the library's C++ (control plane, schedule compiler,
executor, worker pool, SIMD kernels) is rebuilt instrumented and the stand-alone test executable runs the
collectives on the host-memory device with ranks as threads. Any report fails the test."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("kind", ["thread", "address"])
def test_collectives_on_the_host_device_are_clean(kind):
    from hylink_b200 import _build

    try:
        tool = _build.build_sanitized(kind)
    except RuntimeError as e:  # a toolchain without the sanitizer runtime
        if "sanitize" in str(e) or "tsan" in str(e) or "asan" in str(e):
            pytest.skip(f"sanitizer runtime not available: {str(e)[-200:]}")
        raise
    env = dict(os.environ, HYLINK_HOST_BUFFER_SIZE="64M", HYLINK_INTERNAL_BUFFER_BYTES="32M",
               TSAN_OPTIONS="halt_on_error=0 report_signal_unsafe=0 exitcode=66",
               ASAN_OPTIONS="detect_leaks=0 exitcode=66 protect_shadow_gap=0")
    for args in (["--coll", "allreduce", "--ranks", "4"], ["--coll", "reducescatter", "--ranks", "2", "--strided", "--dtype", "bf16"],
                 ["--coll", "allgather", "--ranks", "2"]):
        p = subprocess.run([str(tool)] + args + ["--mode", "threads", "--device", "host", "--bytes-from", "64K", "--bytes-to", "1M",
                                                 "--factor", "16", "--iters", "2"],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300, env=env)
        assert p.returncode == 0 and "Test PASSED." in p.stdout, p.stdout[-3000:]
        assert "WARNING: ThreadSanitizer" not in p.stdout and "ERROR: AddressSanitizer" not in p.stdout, p.stdout[-3000:]
    # worker-owned host ranges (two NUMA pools, reductions on the CPU) and rounds ordered by chunk guards (pools far
    # smaller than the message): the two places where threads of several ranks hand data on without the executor
    scenarios = [
        (dict(HYLINK_GPU_NUMA_MAP="0011", HYLINK_IR_VARIANT="host_reduce", HYLINK_H2H_WORKERS="2"),
         ["--coll", "allreduce", "--ranks", "4", "--bytes-from", "4M", "--bytes-to", "4M"]),
        (dict(HYLINK_GPU_NUMA_MAP="0011", HYLINK_IR_VARIANT="ring", HYLINK_H2H_WORKERS="1"),
         ["--coll", "allreduce", "--ranks", "4", "--bytes-from", "8M", "--bytes-to", "8M"]),
        (dict(HYLINK_GPU_NUMA_MAP="0011", HYLINK_HOST_BUFFER_SIZE="2M", HYLINK_INTERNAL_BUFFER_BYTES="1M"),
         ["--coll", "allgather", "--ranks", "4", "--bytes-from", "8M", "--bytes-to", "8M"]),
        (dict(HYLINK_HOST_BUFFER_SIZE="2M", HYLINK_INTERNAL_BUFFER_BYTES="1M"),
         ["--coll", "allreduce", "--ranks", "2", "--bytes-from", "8M", "--bytes-to", "8M"]),
    ]
    for extra, args in scenarios:
        p = subprocess.run([str(tool)] + args + ["--mode", "threads", "--device", "host", "--iters", "2"],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300, env=dict(env, **extra))
        assert p.returncode == 0 and "Test PASSED." in p.stdout, (extra, p.stdout[-3000:])
        assert "WARNING: ThreadSanitizer" not in p.stdout and "ERROR: AddressSanitizer" not in p.stdout, (extra, p.stdout[-3000:])
