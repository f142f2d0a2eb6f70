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
