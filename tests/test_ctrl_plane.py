"""Control plane without a GPU: shared control block, barrier, mailbox
all-gather and SCM_RIGHTS descriptor passing between real processes, and the
thread flavour (zeroed id)."""
import ctypes as C
import multiprocessing as mp
import threading

import pytest


def _worker(uid, n, r, q):
    from hylink_b200._native import UniqueId, lib

    u = UniqueId()
    C.memmove(C.byref(u), uid, 128)
    rc = lib.hlCtrlSelfTest(u, n, r, 3)
    q.put((r, rc, lib.hlGetLastError().decode()))


@pytest.mark.parametrize("n", [2, 4])
def test_multi_process_rendezvous(n):
    from hylink_b200.parallel.comm import unique_id

    uid = unique_id().ljust(128, b"\0")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(uid, n, r, q)) for r in range(n)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in range(n)]
    for p in ps:
        p.join(30)
    assert all(rc == 0 for _, rc, _ in res), res


def test_single_process_threads():
    from hylink_b200._native import UniqueId, lib

    n, out = 4, {}

    def run(r):
        out[r] = lib.hlCtrlSelfTest(UniqueId(), n, r, 2)

    ts = [threading.Thread(target=run, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
    assert out == {r: 0 for r in range(n)}, (out, lib.hlGetLastError())


def test_missing_rank_times_out_not_hangs():
    """A rank that never joins: the others give up with a timeout result."""
    import os
    import time

    from hylink_b200._native import UniqueId, lib
    from hylink_b200.parallel.comm import unique_id

    os.environ["HYLINK_BARRIER_TIMEOUT_MS"] = "300"
    try:
        u = UniqueId()
        C.memmove(C.byref(u), unique_id().ljust(128, b"\0"), 128)
        t0 = time.time()
        # hlCtrlSelfTest uses its own 20 s limit; go through the communicator instead
        h = C.c_void_p()
        lib.hlCommInitRankDevice.restype = C.c_int
        rc = None
        # a 2-rank communicator where rank 1 never shows up
        from hylink_b200 import _native

        _native.lib.hlConfigReload()
        rc = lib.hlCommInitRankDevice(C.byref(h), 2, u, 0, -2)
        assert rc == 6, (rc, lib.hlGetLastError())  # hlTimeout
        assert time.time() - t0 < 20
    finally:
        del os.environ["HYLINK_BARRIER_TIMEOUT_MS"]
        lib.hlConfigReload()


def test_two_in_process_groups_of_the_same_size_at_once():
    """Ranks as threads of one process, two groups of two created concurrently: every rank must meet its own group
    (ids from hlGetInProcessId carry a group tag behind their leading zero byte)."""
    import ctypes as C
    import threading

    import torch

    from hylink_b200._native import UniqueId, check, lib

    lib.hlGetInProcessId.argtypes = [C.POINTER(UniqueId)]
    ids = [UniqueId(), UniqueId()]
    for u in ids:
        check(lib.hlGetInProcessId(C.byref(u)), "hlGetInProcessId")
    assert C.string_at(C.addressof(ids[0]), 128) != C.string_at(C.addressof(ids[1]), 128)
    results, errors = {}, []

    def rank(group, r):
        try:
            h = C.c_void_p()
            check(lib.hlCommInitRankDevice(C.byref(h), 2, ids[group], r, -2), "init")
            x = torch.full((1000,), float(10 * group + r + 1))
            check(lib.hlAllReduce(x.data_ptr(), x.data_ptr(), 1000, 7, 0, h, None), "allreduce")
            check(lib.hlCommDrain(h), "drain")
            results[(group, r)] = float(x[0])
            lib.hlCommDestroy(h)
        except Exception as ex:  # noqa: BLE001
            errors.append(repr(ex))

    # rank 0 of both groups first, then rank 1 of both: with one open group per size the second rank 0 would
    # displace the first group and the pairs would cross
    th = [threading.Thread(target=rank, args=(g, r)) for r in (0, 1) for g in (0, 1)]
    for t in th:
        t.start()
    for t in th:
        t.join(60)
    assert not errors, errors
    assert results == {(0, 0): 3.0, (0, 1): 3.0, (1, 0): 23.0, (1, 1): 23.0}


def test_reference_environment_names_are_understood():
    """Variables of the reference: aliases where this library has the same knob, a notice where it has none."""
    import os
    import subprocess
    import sys

    code = (
        "import ctypes as C\n"
        "from hylink_b200._native import lib\n"
        "lib.hlConfigValue.restype = C.c_longlong\n"
        "lib.hlConfigValue.argtypes = [C.c_char_p]\n"
        "print({k: lib.hlConfigValue(k.encode()) for k in ('zero_copy', 'small_msg_timeout_ms', 'ipc_close_on_finalize', 'host_buffer_bytes', 'executor_timeout_ms', 'nope')})\n")
    env = dict(os.environ, PCCL_DISABLE_DEVICE_IPC="1", PCCL_SMALL_MSG_FASTPATH_TIMEOUT_MS="1234", PCCL_CUDA_IPC_CLOSE_ON_FINALIZE="0",
               PCCL_HOST_BUFFER_SIZE="64M", PCCL_EXECUTOR_TIMEOUT_MS="5000", PCCL_NCCL_COMPAT_MODE="sp", PCCL_D2D_PUSH="0", HYLINK_LOG_LEVEL="INFO",
               PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = subprocess.run([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-2000:]
    got = eval(p.stdout.strip().splitlines()[-1])
    assert got == {"zero_copy": 0, "small_msg_timeout_ms": 1234, "ipc_close_on_finalize": 0, "host_buffer_bytes": 64 << 20,
                   "executor_timeout_ms": 5000, "nope": -1}
    assert "PCCL_NCCL_COMPAT_MODE=sp is accepted and has no effect here" in p.stderr
    assert "PCCL_D2D_PUSH=0 is accepted and has no effect here" in p.stderr
