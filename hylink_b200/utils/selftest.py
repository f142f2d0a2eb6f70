"""End-to-end check of the ``hylink`` torch.distributed backend.

Run one process per device (``torchrun --nproc-per-node N -m
hylink_b200.utils.selftest``), or one process per rank on a CPU-only machine
with ``--cpu``: every collective is compared with a locally computed
expectation, then a small DDP model trains a few steps and its parameters are
compared across ranks.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    cpu = "--cpu" in (argv or sys.argv[1:])
    from hylink_b200.parallel import backend_stats, register_backend

    register_backend()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if cpu:
        dev = torch.device("cpu")
        dist.init_process_group("hylink")
    else:
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("hylink", device_id=dev)

    def val(r, n, dtype=torch.float32):
        return (torch.arange(n, dtype=torch.float32) % 13 + r + 1).to(dtype).to(dev)

    n = 10007
    for dtype in (torch.float32, torch.bfloat16) if not cpu else (torch.float32,):
        t = val(rank, n, dtype)
        dist.all_reduce(t)
        want = sum(val(r, n, torch.float32).float() for r in range(world)).to(dtype)
        assert torch.equal(t, want.to(dev)), "all_reduce"
    t = val(rank, n)
    w = dist.all_reduce(t, op=dist.ReduceOp.MAX, async_op=True)
    w.wait()
    assert torch.equal(t, val(world - 1, n)), "all_reduce max"
    t = val(rank, n)
    dist.broadcast(t, src=world - 1)
    assert torch.equal(t, val(world - 1, n)), "broadcast"
    out = torch.empty(world * n, device=dev)
    dist.all_gather_into_tensor(out, val(rank, n))
    for r in range(world):
        assert torch.equal(out[r * n:(r + 1) * n], val(r, n)), "all_gather_into_tensor"
    lst = [torch.empty(n, device=dev) for _ in range(world)]
    dist.all_gather(lst, val(rank, n))
    for r in range(world):
        assert torch.equal(lst[r], val(r, n)), "all_gather"
    full = torch.cat([val(rank, n) * (q + 1) for q in range(world)])
    rs = torch.empty(n, device=dev)
    dist.reduce_scatter_tensor(rs, full)
    want = sum(val(r, n) * (rank + 1) for r in range(world))
    assert torch.allclose(rs, want), "reduce_scatter_tensor"
    if not cpu:
        a2a_in = torch.cat([val(rank, 64) + 100 * q for q in range(world)])
        a2a_out = torch.empty_like(a2a_in)
        dist.all_to_all_single(a2a_out, a2a_in)
        for q in range(world):
            assert torch.equal(a2a_out[q * 64:(q + 1) * 64], val(q, 64) + 100 * rank), "all_to_all_single"
    dist.barrier()

    # DDP: identical parameters on every rank after a few steps
    torch.manual_seed(1234 + rank)  # different init per rank: DDP must broadcast rank 0's
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 8)).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=None if cpu else [dev.index], bucket_cap_mb=1)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    for step in range(4):
        x = torch.randn(32, 64, device=dev)
        loss = ddp(x).square().mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    for g in gathered:
        assert torch.equal(g, gathered[0]), "DDP parameters diverged"
    if rank == 0:
        print("stats", backend_stats())
        print("SELFTEST PASSED", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
