"""Runs a function on N ranks as separate processes (spawn) and collects results."""
import multiprocessing as mp
import os
import traceback


def _entry(fn, rank, n, uid, args, q, env):
    try:
        os.environ.update(env or {})
        q.put((rank, "ok", fn(rank, n, uid, *args)))
    except BaseException:  # noqa: BLE001
        q.put((rank, "err", traceback.format_exc()))


def run_ranks(fn, n, *args, env=None, timeout=180):
    from hylink_b200.parallel.comm import unique_id

    uid = unique_id().ljust(128, b"\0")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_entry, args=(fn, r, n, uid, args, q, env)) for r in range(n)]
    for p in ps:
        p.start()
    out = {}
    try:
        for _ in range(n):
            r, status, val = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {r} failed:\n{val}")
            out[r] = val
    finally:
        for p in ps:
            p.join(10)
            if p.is_alive():
                p.kill()
    return [out[r] for r in range(n)]
