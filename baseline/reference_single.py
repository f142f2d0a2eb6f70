"""One-GPU case of the reference arm, in a process of its own that loads neither PyTorch nor NCCL.

The reference's NCCL personality exports the ``nccl*`` names and calls them internally through the dynamic
linker (ncclCommInitAll calls ncclCommInitRank, pcie-ccl-cuda/src/api/nccl_compat/nccl_hook.cpp:742-757). In a
process that has the real NCCL loaded (PyTorch brings it) those internal calls bind to the real library and the
two libraries then hand each other's communicator structures around. So this part runs without PyTorch: device
buffers, streams and events come from the CUDA runtime through ctypes. Prints one JSON object.

    python baseline/reference_single.py <steps> <warmup> <colls,comma> <sizes,comma>
"""
from __future__ import annotations

import ctypes as C
import json
import sys
import time
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


def _cudart():
    for p in ("/usr/local/cuda/lib64/libcudart.so.12", "/usr/local/cuda-12.9/targets/x86_64-linux/lib/libcudart.so.12", "libcudart.so.12"):
        try:
            return C.CDLL(p, mode=C.RTLD_GLOBAL)
        except OSError:
            continue
    raise RuntimeError("libcudart.so.12 not found")


def main() -> int:
    import os

    os.environ.setdefault("PCCL_GPU_NUMA_MAP", "0")   # machines whose sysfs has no NUMA node for the GPU
    steps, warmup = int(sys.argv[1]), int(sys.argv[2])
    colls = sys.argv[3].split(",")
    sizes = [int(s) for s in sys.argv[4].split(",")]
    rt = _cudart()

    def ck(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} -> CUDA error {rc}")

    vp = C.c_void_p
    rt.cudaMalloc.argtypes = [C.POINTER(vp), C.c_size_t]
    rt.cudaMallocHost.argtypes = [C.POINTER(vp), C.c_size_t]
    rt.cudaStreamCreate.argtypes = [C.POINTER(vp)]
    rt.cudaEventCreate.argtypes = [C.POINTER(vp)]
    rt.cudaEventRecord.argtypes = [vp, vp]
    rt.cudaEventElapsedTime.argtypes = [C.POINTER(C.c_float), vp, vp]
    rt.cudaStreamSynchronize.argtypes = [vp]
    rt.cudaMemcpyAsync.argtypes = [vp, vp, C.c_size_t, C.c_int, vp]
    rt.cudaMemset.argtypes = [vp, C.c_int, C.c_size_t]
    ck(rt.cudaSetDevice(0), "cudaSetDevice")
    C.CDLL(str(REF_DIR / "libpccl_kernels.so"), mode=C.RTLD_GLOBAL)
    lib = C.CDLL(str(REF_DIR / "libpccl.so"), mode=C.RTLD_GLOBAL)
    top = max(sizes)
    send, recv = [vp(), vp()], [vp(), vp()]
    for i in range(2):
        ck(rt.cudaMalloc(C.byref(send[i]), top), "cudaMalloc")
        ck(rt.cudaMalloc(C.byref(recv[i]), top), "cudaMalloc")
        ck(rt.cudaMemset(send[i], 0, top), "cudaMemset")
    host, back = vp(), vp()
    ck(rt.cudaMallocHost(C.byref(host), top), "cudaMallocHost")
    ck(rt.cudaMallocHost(C.byref(back), 4096), "cudaMallocHost")
    C.memset(host, 1, top)
    stream = vp()
    ck(rt.cudaStreamCreate(C.byref(stream)), "cudaStreamCreate")
    e0, e1 = vp(), vp()
    ck(rt.cudaEventCreate(C.byref(e0)), "cudaEventCreate")
    ck(rt.cudaEventCreate(C.byref(e1)), "cudaEventCreate")

    comm = vp()
    devs = (C.c_int * 1)(0)
    lib.ncclCommInitAll.argtypes = [C.POINTER(vp), C.c_int, C.POINTER(C.c_int)]
    rc = lib.ncclCommInitAll(C.byref(comm), 1, devs)
    if rc != 0:
        raise RuntimeError(f"ncclCommInitAll(1 device) -> nccl result {rc}")
    f32, nsum = 7, 0   # ncclFloat32, ncclSum
    lib.ncclAllReduce.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.ncclReduceScatter.argtypes = [vp, vp, C.c_size_t, C.c_int, C.c_int, vp, vp]
    lib.ncclAllGather.argtypes = [vp, vp, C.c_size_t, C.c_int, vp, vp]

    def submit(coll, s, d, nbytes):
        cnt = nbytes // 4
        if coll == "allreduce":
            return lib.ncclAllReduce(s, d, cnt, f32, nsum, comm, stream)
        if coll == "reducescatter":
            return lib.ncclReduceScatter(s, d, cnt, f32, nsum, comm, stream)
        return lib.ncclAllGather(s, d, cnt, f32, comm, stream)

    cells = [(c, s) for c in colls for s in sizes]
    dev_sum, e2e_sum = [0.0] * len(cells), [0.0] * len(cells)
    t_begin = time.perf_counter()
    ms = C.c_float()
    for it in range(warmup + steps):
        for ci, (coll, nbytes) in enumerate(cells):
            ck(rt.cudaEventRecord(e0, stream), "cudaEventRecord")
            # all-reduce in place, as torch.distributed.all_reduce (what the other arms time) defines it
            rc = submit(coll, send[it % 2], send[it % 2] if coll == "allreduce" else recv[it % 2], nbytes)
            if rc != 0:
                raise RuntimeError(f"{coll} of {nbytes} bytes -> nccl result {rc}")
            ck(rt.cudaEventRecord(e1, stream), "cudaEventRecord")
            ck(rt.cudaStreamSynchronize(stream), "cudaStreamSynchronize")
            ck(rt.cudaEventElapsedTime(C.byref(ms), e0, e1), "cudaEventElapsedTime")
            if it >= warmup:
                dev_sum[ci] += ms.value
    for it in range(2 + steps):
        for ci, (coll, nbytes) in enumerate(cells):
            t0 = time.perf_counter()
            ck(rt.cudaMemcpyAsync(send[it % 2], host, nbytes, 1, stream), "cudaMemcpyAsync H2D")
            dst = send[it % 2] if coll == "allreduce" else recv[it % 2]
            rc = submit(coll, send[it % 2], dst, nbytes)
            if rc != 0:
                raise RuntimeError(f"{coll} of {nbytes} bytes -> nccl result {rc}")
            ck(rt.cudaMemcpyAsync(back, dst, 4096, 2, stream), "cudaMemcpyAsync D2H")
            ck(rt.cudaStreamSynchronize(stream), "cudaStreamSynchronize")
            if it >= 2:
                e2e_sum[ci] += (time.perf_counter() - t0) * 1e3
    wall = time.perf_counter() - t_begin
    lib.ncclCommDestroy.argtypes = [vp]
    lib.ncclCommDestroy(comm)
    print(json.dumps({"cells": cells, "dev_ms": [x / steps for x in dev_sum], "e2e_ms": [x / steps for x in e2e_sum], "wall_s": wall}))
    return 0


if __name__ == "__main__":
    try:
        sys.exit(main())
    except Exception as ex:  # noqa: BLE001
        print(json.dumps({"error": " ".join(f"{type(ex).__name__}: {ex}".split())}))
        sys.exit(0)
