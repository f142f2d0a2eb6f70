"""An NCCL program served by this library alone (no real NCCL underneath).

One process, one communicator per visible GPU from ``ncclCommInitAll``, one host thread per GPU and, for the group
form, one thread that drives all GPUs between ``ncclGroupStart`` and ``ncclGroupEnd`` — the way single-process NCCL
programs are written (multipath-orchestrator/tests/nccl_test/allreduce/allreduce_param.cc:133-150,
pcie-ccl-cuda/tests/dev/test_nccl_compute_overlap.cu:309-327). Run with ``HYLINK_NCCL_STANDALONE=1``::

    HYLINK_NCCL_STANDALONE=1 python -m hylink_b200.utils.nccl_standalone_check [--gpus N]

Prints ``NCCL_STANDALONE_CHECK ok served=<n>`` when every result is right.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys
import threading
from pathlib import Path

import torch

F32, SUM = 7, 0   # ncclFloat32, ncclSum


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=0)
    a = ap.parse_args(argv)
    os.environ["HYLINK_NCCL_STANDALONE"] = "1"
    libdir = Path(__file__).resolve().parent.parent / "lib"
    C.CDLL(str(libdir / "libhylink_b200.so"), mode=C.RTLD_GLOBAL)
    nccl = C.CDLL(str(libdir / "libhylink_nccl.so"))
    n = a.gpus or min(torch.cuda.device_count(), 4)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    nccl.ncclCommInitAll.argtypes = [C.POINTER(vp), i32, C.POINTER(i32)]
    nccl.ncclAllReduce.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    nccl.ncclReduceScatter.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    nccl.ncclReduce.argtypes = [vp, vp, sz, i32, i32, i32, vp, vp]
    nccl.ncclAllGather.argtypes = [vp, vp, sz, i32, vp, vp]
    nccl.ncclAllToAll.argtypes = [vp, vp, sz, i32, vp, vp]
    nccl.ncclBroadcast.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    nccl.ncclSend.argtypes = [vp, sz, i32, i32, vp, vp]
    szp = C.POINTER(sz)
    nccl.ncclAllGatherV.argtypes = [vp, sz, vp, szp, szp, i32, vp, vp]
    nccl.ncclReduceScatterV.argtypes = [vp, szp, szp, vp, sz, i32, i32, vp, vp]
    nccl.ncclCommSplit.argtypes = [vp, i32, i32, C.POINTER(vp), vp]
    nccl.ncclCommCount.argtypes = [vp, C.POINTER(i32)]
    nccl.ncclCommUserRank.argtypes = [vp, C.POINTER(i32)]
    nccl.ncclCommDestroy.argtypes = [vp]
    nccl.ncclMemAlloc.argtypes = [C.POINTER(vp), sz]
    nccl.ncclMemFree.argtypes = [vp]
    nccl.ncclGetErrorString.restype = C.c_char_p
    nccl.ncclGetErrorString.argtypes = [i32]
    nccl.ncclGetLastError.restype = C.c_char_p
    nccl.ncclGetLastError.argtypes = [vp]
    assert nccl.hlNcclShimStandalone() == 1

    def ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {nccl.ncclGetErrorString(rc).decode()} ({nccl.ncclGetLastError(None).decode()})")

    ver = i32()
    ok(nccl.ncclGetVersion(C.byref(ver)), "ncclGetVersion")
    comms = (vp * n)()
    ok(nccl.ncclCommInitAll(comms, n, None), "ncclCommInitAll")
    streams = []
    for r in range(n):
        torch.cuda.set_device(r)
        streams.append(torch.cuda.Stream(device=r))
    count = 1 << 18
    errors = []

    def ptr(t):
        return vp(t.data_ptr())

    def per_rank(r):
        try:
            torch.cuda.set_device(r)
            st = streams[r]
            s = vp(st.cuda_stream)
            c = comms[r]
            with torch.cuda.stream(st):
                x = torch.full((count,), float(r + 1), device=f"cuda:{r}")
                y = torch.zeros_like(x)
                ok(nccl.ncclAllReduce(ptr(x), ptr(y), count, F32, SUM, c, s), "ncclAllReduce")
                st.synchronize()
                assert bool((y == n * (n + 1) / 2).all()), "all-reduce"
                seg = count // n
                part = torch.zeros(seg, device=f"cuda:{r}")
                ok(nccl.ncclReduceScatter(ptr(x), ptr(part), seg, F32, SUM, c, s), "ncclReduceScatter")
                full = torch.zeros(seg * n, device=f"cuda:{r}")
                ok(nccl.ncclAllGather(ptr(x), ptr(full), seg, F32, c, s), "ncclAllGather")
                b = x.clone()
                ok(nccl.ncclBroadcast(ptr(b), ptr(b), count, F32, n - 1, c, s), "ncclBroadcast")
                a2a = torch.zeros(seg * n, device=f"cuda:{r}")
                ok(nccl.ncclAllToAll(ptr(x), ptr(a2a), seg, F32, c, s), "ncclAllToAll")
                red = torch.full((count,), -1.0, device=f"cuda:{r}")
                ok(nccl.ncclReduce(ptr(x), ptr(red), count, F32, SUM, 0, c, s), "ncclReduce")
                st.synchronize()
                assert bool((part == n * (n + 1) / 2).all()), "reduce-scatter"
                assert torch.equal(full, torch.cat([torch.full((seg,), float(q + 1)) for q in range(n)]).to(full.device)), "all-gather"
                assert bool((b == float(n)).all()), "broadcast"
                assert torch.equal(a2a, torch.cat([torch.full((seg,), float(q + 1)) for q in range(n)]).to(full.device)), "all-to-all"
                assert bool((red == (n * (n + 1) / 2 if r == 0 else -1.0)).all()), "reduce"
                # V-variants: equal counts with gaps between the segments (one strided kernel) ...
                gap = seg + 64
                counts = (sz * n)(*([seg] * n))
                displs = (sz * n)(*[q * gap for q in range(n)])
                wide = torch.full((gap * n,), -2.0, device=f"cuda:{r}")
                ok(nccl.ncclAllGatherV(ptr(x), seg, ptr(wide), counts, displs, F32, c, s), "ncclAllGatherV")
                st.synchronize()
                for q in range(n):
                    assert bool((wide[q * gap:q * gap + seg] == float(q + 1)).all()) and bool((wide[q * gap + seg:(q + 1) * gap] == -2.0).all()), "all-gather-v"
                # ... and ragged counts (one call per contributor)
                rag = [1000 + 17 * q for q in range(n)]
                counts = (sz * n)(*rag)
                offs = [sum(rag[:q]) for q in range(n)]
                displs = (sz * n)(*offs)
                wide = torch.zeros(sum(rag), device=f"cuda:{r}")
                ok(nccl.ncclAllGatherV(ptr(x), rag[r], ptr(wide), counts, displs, F32, c, s), "ncclAllGatherV ragged")
                mine = torch.full((rag[r],), -3.0, device=f"cuda:{r}")
                src = torch.full((sum(rag),), float(r + 1), device=f"cuda:{r}")
                ok(nccl.ncclReduceScatterV(ptr(src), counts, displs, ptr(mine), rag[r], F32, SUM, c, s), "ncclReduceScatterV ragged")
                st.synchronize()
                for q in range(n):
                    assert bool((wide[offs[q]:offs[q] + rag[q]] == float(q + 1)).all()), "all-gather-v ragged"
                assert bool((mine == n * (n + 1) / 2).all()), "reduce-scatter-v ragged"
                # sub-communicators by colour
                child = vp()
                ok(nccl.ncclCommSplit(c, r % 2, n - r, C.byref(child), None), "ncclCommSplit")
                cn, cr = i32(), i32()
                ok(nccl.ncclCommCount(child, C.byref(cn)), "ncclCommCount")
                ok(nccl.ncclCommUserRank(child, C.byref(cr)), "ncclCommUserRank")
                members = [q for q in range(n) if q % 2 == r % 2]
                assert cn.value == len(members) and cr.value == sorted(members, reverse=True).index(r), "split ranks"
                z = torch.full((4096,), float(r + 1), device=f"cuda:{r}")
                ok(nccl.ncclAllReduce(ptr(z), ptr(z), 4096, F32, SUM, child, s), "ncclAllReduce on a child")
                st.synchronize()
                assert bool((z == float(sum(q + 1 for q in members))).all()), "child all-reduce"
                ok(nccl.ncclCommDestroy(child), "ncclCommDestroy child")
                # registered memory from ncclMemAlloc: the same collectives, zero-copy
                p = vp()
                ok(nccl.ncclMemAlloc(C.byref(p), count * 4), "ncclMemAlloc")
                from hylink_b200.ops.emu import _tensor_at

                reg = _tensor_at(p.value, count, torch.float32, None)
                reg.fill_(float(r + 1))
                ok(nccl.ncclAllReduce(ptr(reg), ptr(reg), count, F32, SUM, c, s), "ncclAllReduce registered")
                st.synchronize()
                assert bool((reg == n * (n + 1) / 2).all()), "registered all-reduce"
                del reg
                ok(nccl.ncclMemFree(p), "ncclMemFree")
                # point-to-point is refused with a reason
                assert nccl.ncclSend(ptr(x), 16, F32, 0, c, s) == 5 and b"point-to-point" in nccl.ncclGetLastError(None)
        except Exception as ex:  # noqa: BLE001
            errors.append(f"rank {r}: {type(ex).__name__}: {ex}")

    th = [threading.Thread(target=per_rank, args=(r,)) for r in range(n)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    if errors:
        print("\n".join(errors))
        return 1
    # one thread, all GPUs, one group
    xs = []
    for r in range(n):
        torch.cuda.set_device(r)
        xs.append(torch.full((count,), float(r + 1), device=f"cuda:{r}"))
        torch.cuda.synchronize(r)
    ok(nccl.ncclGroupStart(), "ncclGroupStart")
    for r in range(n):
        ok(nccl.ncclAllReduce(ptr(xs[r]), ptr(xs[r]), count, F32, SUM, comms[r], vp(streams[r].cuda_stream)), "grouped ncclAllReduce")
    before = C.c_uint64()
    nccl.hlNcclShimCounters(C.byref(before), None)
    ok(nccl.ncclGroupEnd(), "ncclGroupEnd")
    for r in range(n):
        streams[r].synchronize()
        assert bool((xs[r] == n * (n + 1) / 2).all()), "grouped all-reduce"
    for r in range(n):
        torch.cuda.set_device(r)
        ok(nccl.ncclCommDestroy(comms[r]), "ncclCommDestroy")
    print(f"NCCL_STANDALONE_CHECK ok version={ver.value} gpus={n} served={before.value}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
