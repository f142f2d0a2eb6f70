"""Tensor / sequence parallel blocks, sharded AdamW, expert-parallel MoE, Ulysses and all-gather context-parallel
attention and a GPipe schedule, each compared with its dense single-process counterpart. Real processes on CPU
tensors through the ``hylink`` torch.distributed backend (host-memory device)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [2, 4])
def test_parallel_schemes_match_dense_math_on_cpu(nproc):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", HYLINK_HOST_BUFFER_SIZE="64M",
               HYLINK_INTERNAL_BUFFER_BYTES="32M", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(29660 + nproc), "-m", "hylink_b200.utils.parallel_selftest", "--cpu"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=400)
    assert p.returncode == 0 and "PARALLEL SELFTEST PASSED" in p.stdout, p.stdout[-4000:]
