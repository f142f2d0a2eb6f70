"""Every NVLink / NVSwitch kernel by name on 2, 4 and 8 real GPUs (skipped where the box has fewer)."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_every_kernel_against_the_fp32_oracle(world):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    e = dict(os.environ)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    # the switch kernels have to be reachable by name at every rank count, two included
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29641", "-m", "hylink_b200.utils.kernel_check", "--max-bytes", "48M"]
    p = subprocess.run(cmd, cwd=ROOT, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert p.returncode == 0 and '"failures": 0' in p.stdout, p.stdout[-4000:]
    assert '"nvls": true' in p.stdout, "multicast memory was not set up: the NVLS kernels did not run\n" + p.stdout[-2000:]
