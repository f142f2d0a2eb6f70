"""The stand-alone NCCL personality on whatever GPUs the box has (one is enough: a one-rank communicator)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_gpu_nccl_program():
    e = dict(os.environ, HYLINK_NCCL_STANDALONE="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "hylink_b200.utils.nccl_standalone_check", "--gpus", "1"], cwd=ROOT, env=e,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0 and "NCCL_STANDALONE_CHECK ok" in p.stdout, p.stdout[-4000:]
