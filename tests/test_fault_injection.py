"""Failures made on the host, never on a GPU: a transfer that the executor is told to fail, a rank that is held
back past its peers' deadline, a schedule file cut short. Every rank must come back with an error inside the
deadline (nobody hangs), the communicator must report the latched error, and a fresh communicator must work.
Ranks are real processes on the host-memory device."""
import os
import time

import pytest
import torch

from mp_util import run_ranks

ENV = {"HYLINK_HOST_BUFFER_SIZE": "64M", "HYLINK_INTERNAL_BUFFER_BYTES": "32M", "HYLINK_LOG_LEVEL": "OFF"}


def _comm(rank, n, uid):
    from hylink_b200.parallel.comm import Communicator

    return Communicator(rank, n, uid=uid, device=-2)


def _faulty_then_fresh(rank, n, uid, uid2):
    from hylink_b200 import HylinkError
    from hylink_b200._native import lib

    c = _comm(rank, n, uid)
    x = torch.ones(300000)
    t0 = time.time()
    try:
        c.all_reduce(x)
        c.drain()
        code = 0
    except HylinkError as e:
        code = e.code
    elapsed = time.time() - t0
    latched = c.async_error()
    c.close()
    # the fault is gone: a communicator created afterwards works
    os.environ.pop("HYLINK_FAULT_INJECT", None)
    lib.hlConfigReload()
    c2 = _comm(rank, n, uid2)
    y = torch.full((5000,), float(rank + 1))
    c2.all_reduce(y)
    c2.drain()
    ok = bool((y == n * (n + 1) / 2).all())
    c2.close()
    return code, latched, elapsed, ok


def _second_uid():
    from hylink_b200.parallel.comm import unique_id

    return unique_id().ljust(128, b"\0")


@pytest.mark.parametrize("n", [2, 4])
def test_failed_transfer_on_one_rank_ends_the_collective_everywhere(n):
    env = dict(ENV, HYLINK_FAULT_INJECT="copy_error@2,rank=1", HYLINK_EXECUTOR_TIMEOUT_MS="8000", HYLINK_BARRIER_TIMEOUT_MS="8000")
    res = run_ranks(_faulty_then_fresh, n, _second_uid(), env=env, timeout=120)
    for rank, (code, latched, elapsed, ok) in enumerate(res):
        assert code != 0, f"rank {rank} completed a collective whose transfer failed on rank 1"
        assert code == (4 if rank == 1 else code) and code in (4, 6, 8)   # device error where injected; timeout/remote elsewhere
        assert latched != 0 and elapsed < 20 and ok, (rank, code, latched, elapsed, ok)


def test_rank_held_back_past_the_deadline_times_out_cleanly():
    env = dict(ENV, HYLINK_FAULT_INJECT="stall_ms=4000@1,rank=0", HYLINK_EXECUTOR_TIMEOUT_MS="1000", HYLINK_BARRIER_TIMEOUT_MS="10000")
    res = run_ranks(_faulty_then_fresh, 2, _second_uid(), env=env, timeout=120)
    for rank, (code, latched, elapsed, ok) in enumerate(res):
        assert code in (6, 8), (rank, code)   # the waiting rank times out; the late one finds the failure latched
        assert elapsed < 15 and ok, (rank, elapsed, ok)


def _truncated_schedule(rank, n, uid):
    import ctypes as C

    from hylink_b200 import HylinkError
    from hylink_b200._native import check, lib
    from hylink_b200.utils.schedule import generate

    xml = generate("allreduce", "00")
    cut = xml[: len(xml) // 2]
    c = _comm(rank, n, uid)
    x = torch.ones(4096)
    out = torch.zeros(4096)
    try:
        check(lib.hlSubmitIr(c._h, cut.encode(), x.data_ptr(), out.data_ptr(), 4096, 0, 1, 1, 7, 0, C.c_void_p(0)), "hlSubmitIr")
        verdict = "accepted"
    except HylinkError as e:
        verdict = e.code
    # the refusal happened before anything was queued: the communicator is still usable
    c.all_reduce(x)
    c.drain()
    healthy = bool((x == n).all()) and c.async_error() == 0
    c.close()
    return verdict, healthy


def test_schedule_cut_short_is_refused_before_anything_runs():
    res = run_ranks(_truncated_schedule, 2, env=ENV, timeout=120)
    for verdict, healthy in res:
        assert verdict == 1 and healthy, (verdict, healthy)   # invalid argument; nothing latched
