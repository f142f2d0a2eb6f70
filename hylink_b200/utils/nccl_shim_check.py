"""Checks the drop-in NCCL symbol layer under an unmodified NCCL program.

Run with the shim preloaded, one process per GPU::

    LD_PRELOAD=hylink_b200/lib/libhylink_nccl.so HYLINK_REAL_NCCL=$(python -m hylink_b200.utils.nccl_shim_check --print-real) \
      python -m torch.distributed.run --nproc-per-node 2 -m hylink_b200.utils.nccl_shim_check

The program uses plain ``backend="nccl"``; the collectives must give NCCL's
results while the shim's counters show that they ran on this library, and
send/recv must still work (they pass through to NCCL).
"""
from __future__ import annotations

import ctypes
import os
import sys


def real_nccl_path() -> str:
    """Path of the NCCL library PyTorch itself would load."""
    try:
        import nvidia.nccl as n  # the wheel that ships libnccl.so.2 (a namespace package)

        for base in list(getattr(n, "__path__", [])):
            p = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(p):
                return p
    except ImportError:
        pass
    return "libnccl.so.2"


def shim_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libhylink_nccl.so")


def main() -> int:
    if "--print-real" in sys.argv:
        print(real_nccl_path())
        return 0
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n = 100003
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        t = (torch.arange(n, device=dev) % 7 + rank + 1).to(dtype)
        dist.all_reduce(t)
        want = sum((torch.arange(n, device=dev) % 7 + r + 1) for r in range(world)).to(dtype)
        assert torch.equal(t, want), f"all_reduce {dtype}"
    t = torch.full((n,), float(rank), device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    assert torch.allclose(t, torch.full_like(t, (world - 1) / 2)), "avg"
    out = torch.empty(world * n, device=dev)
    dist.all_gather_into_tensor(out, torch.full((n,), float(rank + 1), device=dev))
    for r in range(world):
        assert torch.all(out[r * n:(r + 1) * n] == r + 1), "all_gather"
    rs = torch.empty(n, device=dev)
    dist.reduce_scatter_tensor(rs, torch.arange(world * n, device=dev, dtype=torch.float32))
    want = torch.arange(rank * n, (rank + 1) * n, device=dev, dtype=torch.float32) * world
    assert torch.equal(rs, want), "reduce_scatter"
    b = torch.full((n,), float(rank), device=dev)
    dist.broadcast(b, src=world - 1)
    assert torch.all(b == world - 1), "broadcast"
    # point-to-point stays on NCCL
    if world >= 2:
        if rank == 0:
            dist.send(torch.full((16,), 42.0, device=dev), dst=1)
        elif rank == 1:
            r = torch.zeros(16, device=dev)
            dist.recv(r, src=0)
            assert torch.all(r == 42.0), "send/recv"
    torch.cuda.synchronize()
    served = passed = -1
    try:
        lib = ctypes.CDLL(shim_path())  # already mapped when preloaded: same instance, same counters
        a, b2 = ctypes.c_uint64(), ctypes.c_uint64()
        lib.hlNcclShimCounters(ctypes.byref(a), ctypes.byref(b2))
        served, passed = a.value, b2.value
    except OSError:
        pass
    dist.barrier()
    if rank == 0:
        print(f"NCCL_SHIM_CHECK served={served} passed_through={passed} preloaded={'libhylink_nccl' in os.environ.get('LD_PRELOAD', '')}",
              flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
