"""Real multi-GPU runs (one process per GPU over NVLink): skipped below 2 GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, args, timeout=600, env=None):
    e = dict(os.environ)
    e.update(env or {})
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29631"] + args
    p = subprocess.run(cmd, cwd=ROOT, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout[-4000:]
    return p.stdout


def test_sweep_correct_against_nccl():
    out = _torchrun(2, ["-m", "hylink_b200.utils.sweep", "--bytes-from", "1K", "--bytes-to", "16M", "--factor", "8", "--check",
                        "--colls", "allreduce,reducescatter,allgather,alltoall", "--dtypes", "bf16,fp32", "--iters", "3"])
    assert '"failures": 0' in out, out[-3000:]


def test_c10d_backend_and_ddp():
    out = _torchrun(2, ["-m", "hylink_b200.utils.selftest"])
    assert "SELFTEST PASSED" in out, out[-3000:]


def test_pcie_path_alone_is_correct():
    """Collectives routed only through pinned host memory by the CPU executor."""
    env = {"HYLINK_PCIE_ENABLE": "1", "HYLINK_HOST_BUFFER_SIZE": "256M", "HYLINK_INTERNAL_BUFFER_BYTES": "128M"}
    out = _torchrun(2, ["-m", "hylink_b200.utils.sweep", "--bytes-from", "64K", "--bytes-to", "32M", "--factor", "8", "--check",
                        "--colls", "allreduce,reducescatter,allgather,alltoall", "--dtypes", "bf16,fp32", "--iters", "3",
                        "--path", "pcie", "--no-nccl"], env=env)
    assert '"failures": 0' in out, out[-3000:]
    assert '"copy_engine_ops": 0' not in out
    # reductions read the landed host chunks themselves: no H2D copy in front of them
    assert '"fused_landing_slices": 0' not in out
    # and the sizes below 1 MiB never reach the executor thread
    assert '"small_path_calls": 0' not in out


def test_blocking_cuda_calls_drain_the_executors_first():
    """The interposers of host-blocking CUDA calls, preloaded and switched on, under a program that synchronises and
    reads results back between PCIe-path collectives (the pattern of the reference's deadlock_repro.py)."""
    shim = os.path.join(ROOT, "hylink_b200", "lib", "libhylink_cudashim.so")
    assert os.path.exists(shim), "libhylink_cudashim.so is not built"
    env = {"HYLINK_PCIE_ENABLE": "1", "HYLINK_HOST_BUFFER_SIZE": "256M", "HYLINK_INTERNAL_BUFFER_BYTES": "128M",
           "LD_PRELOAD": shim, "HYLINK_CUDA_BLOCK_SHIM": "1"}
    out = _torchrun(2, ["-m", "hylink_b200.utils.sweep", "--bytes-from", "256K", "--bytes-to", "16M", "--factor", "8", "--check",
                        "--colls", "allreduce,allgather", "--dtypes", "fp32", "--iters", "3", "--path", "pcie", "--no-nccl"], env=env)
    assert '"failures": 0' in out, out[-3000:]
    import json

    done = [json.loads(l) for l in out.splitlines() if l.startswith('{"event": "done"')][0]
    assert done.get("block_shim_drains", 0) > 0, done


def test_forked_collectives_are_correct_and_retune():
    """Every collective forked over NVLink kernels + PCIe schedules, with the feedback controller running."""
    env = {"HYLINK_ORCH_ENABLE": "1", "HYLINK_MIN_MSG_SIZE": "1M", "HYLINK_MIN_MSG_SIZE_8": "1M",
           "HYLINK_HOST_BUFFER_SIZE": "256M", "HYLINK_INTERNAL_BUFFER_BYTES": "128M"}
    out = _torchrun(2, ["-m", "hylink_b200.utils.sweep", "--bytes-from", "2M", "--bytes-to", "128M", "--factor", "8", "--check",
                        "--colls", "allreduce,reducescatter,allgather,alltoall", "--dtypes", "bf16", "--iters", "12",
                        "--path", "split", "--no-nccl"], env=env)
    assert '"failures": 0' in out, out[-3000:]
    import json

    done = [json.loads(l) for l in out.splitlines() if l.startswith('{"event": "done"')][0]
    assert done["stats"]["pcie_bytes"] > 0 and done["stats"]["nvl_bytes"] > 0
    assert 0.0 < done["stats"]["last_alpha"] < 0.5


def test_nccl_symbol_layer_serves_an_unmodified_nccl_program():
    from hylink_b200.utils.nccl_shim_check import real_nccl_path, shim_path

    env = {"LD_PRELOAD": shim_path(), "HYLINK_REAL_NCCL": real_nccl_path()}
    out = _torchrun(2, ["-m", "hylink_b200.utils.nccl_shim_check"], env=env)
    line = [l for l in out.splitlines() if l.startswith("NCCL_SHIM_CHECK")][-1]
    served = int(line.split("served=")[1].split()[0])
    assert served >= 7, line


def test_deterministic_sum_order_against_host_oracles():
    out = _torchrun(2, ["-m", "hylink_b200.utils.determinism", "--bytes-from", "256K", "--bytes-to", "16M"])
    assert '"failures": 0' in out, out[-3000:]


def test_native_perf_tool_threads_and_fork():
    """hl_perf on two GPUs: ranks as threads over the NVLink kernels, ranks as processes over the PCIe path."""
    tool = os.path.join(ROOT, "hylink_b200", "bin", "hl_perf")
    if not os.path.exists(tool):
        from hylink_b200 import _build

        _build.build_core()
        _build.build_tools()
    for args, env in (
        (["--coll", "allreduce", "--ranks", "2", "--mode", "threads", "--path", "nvlink", "--dtype", "bf16",
          "--bytes-from", "4K", "--bytes-to", "64M", "--factor", "16", "--iters", "5"], {}),
        (["--coll", "reducescatter", "--ranks", "2", "--mode", "fork", "--path", "pcie", "--strided",
          "--bytes-from", "1M", "--bytes-to", "1M", "--iters", "3"],
         {"HYLINK_PCIE_ENABLE": "1", "HYLINK_HOST_BUFFER_SIZE": "256M", "HYLINK_INTERNAL_BUFFER_BYTES": "128M"}),
    ):
        p = subprocess.run([tool] + args, env=dict(os.environ, **env), stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                           text=True, timeout=300)
        assert p.returncode == 0 and "Test PASSED." in p.stdout, p.stdout[-3000:]


def test_parallel_schemes_match_dense_math():
    """Tensor/sequence parallel, sharded optimizer, MoE all-to-all, Ulysses / context-parallel attention, GPipe."""
    out = _torchrun(2, ["-m", "hylink_b200.utils.parallel_selftest"])
    assert "PARALLEL SELFTEST PASSED" in out, out[-3000:]


def test_nccl_program_served_without_a_real_nccl():
    """Thread-per-GPU ncclCommInitAll program, group calls, V-variants, split and ncclMemAlloc on the stand-alone personality."""
    e = dict(os.environ, HYLINK_NCCL_STANDALONE="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "hylink_b200.utils.nccl_standalone_check"], cwd=ROOT, env=e, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0 and "NCCL_STANDALONE_CHECK ok" in p.stdout, p.stdout[-4000:]
