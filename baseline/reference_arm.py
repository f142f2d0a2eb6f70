"""Reference arm of ``bench.py``: the unmodified reference library, timed on the same cells.

Loads ``baseline/_ref/libpccl.so`` (built by ``baseline/install_reference.py`` from the
reference's own CMake files) and drives it through its public C API exactly as
its own test programs do (pcie-ccl-cuda/tests/coll/test_allreduce.cpp:52-113,
pcie-ccl-cuda/tests/common/test_common.hpp:231-298): single-process mode — a
zeroed ``pcclUniqueId``, one communicator and one host thread per GPU — with the
schedules it ships (``PCCL_IR_PATH``) and its ``PCCL_GPU_NUMA_MAP`` override for
machines whose sysfs has no NUMA node for the GPUs. Nothing of this repository's
library is imported here; PyTorch is used for device buffers, streams and events
only.

The reference's plain API reduces fp32 with sum (pcie-ccl-cuda/src/ir/compiler.hpp:75-89),
so the cells are the same BYTE sizes as the bf16 cells of the other arms. With
one GPU its own C API has no schedule; the one-rank case is served by its NCCL
personality (a device-to-device copy, nccl_hook.cpp:86-98), which is what is
timed then.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import threading
import time
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"

NUMA_MAPS = {2: "0,0", 4: "0,0,1,1", 8: "0,0,1,1,2,2,3,3"}   # patterns 00, 0011, 00112233 of the shipped schedule set


class PcclUniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def bus_factor(coll: str, n: int) -> float:
    if n <= 1:
        return 1.0   # one rank: plain bytes / time
    return 2.0 * (n - 1) / n if coll == "allreduce" else (n - 1) / n


def geomean(xs):
    xs = [x for x in xs if x and x > 0]
    return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else 0.0


def load_library():
    """Returns the loaded reference library, or raises with the loader's own message."""
    if not (REF_DIR / "libpccl.so").exists():
        raise RuntimeError(f"{REF_DIR}/libpccl.so is missing (run baseline/install_reference.py)")
    C.CDLL(str(REF_DIR / "libpccl_kernels.so"), mode=C.RTLD_GLOBAL)
    lib = C.CDLL(str(REF_DIR / "libpccl.so"), mode=C.RTLD_GLOBAL)
    lib.pcclGetErrorString.restype = C.c_char_p
    lib.pcclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, PcclUniqueId, C.c_int]
    for name in ("pcclAllReduce", "pcclAllGather", "pcclReduceScatter"):
        getattr(lib, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.pcclCommDestroy.argtypes = [C.c_void_p]
    return lib


class _Barrier:
    """Thread rendezvous that also carries the first error of any rank to all of them."""

    def __init__(self, n):
        self.bar = threading.Barrier(n)
        self.error = None

    def wait(self):
        try:
            self.bar.wait(timeout=300)
        except threading.BrokenBarrierError:
            if self.error is None:
                self.error = "a rank thread left the run early"
        return self.error is None

    def fail(self, msg):
        if self.error is None:
            self.error = msg
        self.bar.abort()


def _cells(colls, sizes):
    return [(c, s) for c in colls for s in sizes]


def run_multi(n: int, steps: int, warmup: int, colls, sizes, e2e: bool = True) -> dict:
    """n >= 2 GPUs, one thread per GPU in this process. Returns per-cell device times (max over ranks)."""
    import torch

    os.environ.setdefault("PCCL_IR_PATH", str(REF_DIR / "ir"))
    os.environ.setdefault("PCCL_GPU_NUMA_MAP", NUMA_MAPS[n])
    os.environ.setdefault("PCCL_EXECUTOR_TIMEOUT_MS", "60000")
    os.environ.setdefault("PCCL_BARRIER_TIMEOUT_MS", "60000")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")   # pcie-ccl-cuda/README.md:665
    lib = load_library()
    cells = _cells(colls, sizes)
    max_bytes = max(sizes)
    bar = _Barrier(n)
    dev_ms = [[0.0] * len(cells) for _ in range(n)]      # per rank, per cell: mean device ms
    e2e_ms = [[0.0] * len(cells) for _ in range(n)]
    comms = [C.c_void_p() for _ in range(n)]
    # communicators are created one after the other on the calling thread, as the reference's tests do
    for r in range(n):
        torch.cuda.set_device(r)
        torch.zeros(1, device=f"cuda:{r}")
        rc = lib.pcclCommInitRank(C.byref(comms[r]), n, PcclUniqueId(), r)
        if rc != 0:
            raise RuntimeError(f"pcclCommInitRank(rank {r}) -> {lib.pcclGetErrorString(rc).decode()}")

    def submit(coll, send, recv, nbytes, comm, stream):
        count = nbytes // 4
        if coll == "allreduce":
            return lib.pcclAllReduce(send, recv, count, comm, stream)
        if coll == "reducescatter":
            return lib.pcclReduceScatter(send, recv, count // n, comm, stream)
        return lib.pcclAllGather(send, recv, count // n, comm, stream)

    def worker(r):
        try:
            torch.cuda.set_device(r)
            dev = torch.device("cuda", r)
            stream = torch.cuda.Stream(device=dev)
            sptr = C.c_void_p(stream.cuda_stream)
            nslots = 2
            send = [torch.rand(max_bytes // 4, device=dev) * 2 - 1 for _ in range(nslots)]
            recv = [torch.empty(max_bytes // 4, device=dev) for _ in range(nslots)]
            host = torch.empty(max_bytes // 4).pin_memory() if e2e else None
            if host is not None:
                host.uniform_(-1, 1)
            back = torch.empty(1024).pin_memory()
            torch.cuda.synchronize(dev)
            sums = [0.0] * len(cells)
            with torch.cuda.stream(stream):
                for it in range(warmup + steps):
                    for ci, (coll, nbytes) in enumerate(cells):
                        if not bar.wait():
                            return
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        s, d = send[it % nslots], recv[it % nslots]
                        e0.record(stream)
                        rc = submit(coll, C.c_void_p(s.data_ptr()), C.c_void_p(d.data_ptr()), nbytes, comms[r], sptr)
                        e1.record(stream)
                        if rc != 0:
                            bar.fail(f"{coll} {nbytes} B on rank {r} -> {lib.pcclGetErrorString(rc).decode()}")
                            return
                        stream.synchronize()
                        if it >= warmup:
                            sums[ci] += e0.elapsed_time(e1)
                dev_ms[r] = [x / steps for x in sums]
                if e2e:
                    sums = [0.0] * len(cells)
                    for it in range(2 + steps):
                        for ci, (coll, nbytes) in enumerate(cells):
                            in_bytes = nbytes // n if coll == "allgather" else nbytes
                            if not bar.wait():
                                return
                            t0 = time.perf_counter()
                            s, d = send[it % nslots], recv[it % nslots]
                            s[:in_bytes // 4].copy_(host[:in_bytes // 4], non_blocking=True)
                            rc = submit(coll, C.c_void_p(s.data_ptr()), C.c_void_p(d.data_ptr()), nbytes, comms[r], sptr)
                            if rc != 0:
                                bar.fail(f"{coll} {nbytes} B on rank {r} -> {lib.pcclGetErrorString(rc).decode()}")
                                return
                            back.copy_(d[:1024], non_blocking=True)
                            stream.synchronize()
                            if it >= 2:
                                sums[ci] += (time.perf_counter() - t0) * 1e3
                    e2e_ms[r] = [x / steps for x in sums]
            bar.wait()
        except Exception as ex:  # noqa: BLE001 - the message is the result
            bar.fail(f"rank {r}: {type(ex).__name__}: {ex}")

    t_begin = time.perf_counter()
    threads = [threading.Thread(target=worker, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t_begin
    if bar.error:
        raise RuntimeError(bar.error)
    for r in range(n):
        torch.cuda.set_device(r)
        lib.pcclCommDestroy(comms[r])
    lib.pcclFinalize()
    return {"cells": cells, "dev_ms": [max(dev_ms[r][i] for r in range(n)) for i in range(len(cells))],
            "e2e_ms": [max(e2e_ms[r][i] for r in range(n)) for i in range(len(cells))] if e2e else None, "wall_s": wall}


def run_single(steps: int, warmup: int, colls, sizes, e2e: bool = True) -> dict:
    """One GPU: the reference's NCCL personality with a one-rank communicator (device-to-device copy), in a child
    process that loads neither PyTorch nor the real NCCL (see reference_single.py for why)."""
    import json
    import subprocess
    import sys

    cmd = [sys.executable, str(Path(__file__).resolve().parent / "reference_single.py"), str(steps), str(warmup), ",".join(colls),
           ",".join(str(s) for s in sizes)]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    if not lines:
        raise RuntimeError(f"the one-GPU run of the reference ended with exit code {p.returncode}: {p.stderr[-300:]}")
    res = json.loads(lines[-1])
    if "error" in res:
        raise RuntimeError(res["error"])
    res["cells"] = [tuple(c) for c in res["cells"]]
    return res


def probe_multi(n: int) -> None:
    """One small pass of the reference on n GPUs in a CHILD process. The library ends the process with abort() on some
    set-up failures (host pool, schedule lookup); in a child that becomes an error message here instead of the end
    of the caller. Raises RuntimeError with the child's last words when it did not get through."""
    import subprocess
    import sys

    cmd = [sys.executable, str(Path(__file__).resolve()), "--probe", str(n)]
    try:
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    except subprocess.TimeoutExpired:
        raise RuntimeError(f"a one-pass trial of the reference on {n} GPUs did not finish within 300 s") from None
    if p.returncode != 0 or "PROBE OK" not in p.stdout:
        tail = " ".join((p.stderr or p.stdout)[-400:].split())
        raise RuntimeError(f"a one-pass trial of the reference on {n} GPUs ended with exit code {p.returncode}: {tail}")


def run(n: int, steps: int, warmup: int, colls, sizes, e2e: bool = True) -> dict:
    if n == 1:
        return run_single(steps, warmup, colls, sizes, e2e)
    if n not in NUMA_MAPS:
        raise RuntimeError(f"the reference ships no schedule set for {n} GPUs (it has 2, 4 and 8)")
    if os.environ.get("HYLINK_REFERENCE_PROBE", "1") != "0":
        probe_multi(n)
    return run_multi(n, steps, warmup, colls, sizes, e2e)


if __name__ == "__main__":
    import sys

    if len(sys.argv) == 3 and sys.argv[1] == "--probe":
        run_multi(int(sys.argv[2]), 1, 1, ("allreduce", "reducescatter", "allgather"), [1 << 20, 64 << 20], e2e=False)
        print("PROBE OK", flush=True)
