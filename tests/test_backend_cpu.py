"""The torch.distributed backend on CPU tensors: two real processes, every
collective plus a DDP model, served by the host-memory device of the
schedule-IR path (no GPU, no gloo)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c10d_backend_and_ddp_on_cpu():
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", HYLINK_HOST_BUFFER_SIZE="64M",
               HYLINK_INTERNAL_BUFFER_BYTES="32M", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", "-m", "hylink_b200.utils.selftest", "--cpu"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert p.returncode == 0 and "SELFTEST PASSED" in p.stdout, p.stdout[-4000:]
