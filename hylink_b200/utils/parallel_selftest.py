"""Checks of the parallelism schemes against single-process math.

Run one process per rank: ``torchrun --nproc-per-node N -m hylink_b200.utils.parallel_selftest`` (GPUs) or with
``--cpu`` on a machine without one. Every scheme computes the same numbers as its dense counterpart on the
gathered data: tensor-parallel and sequence-parallel transformer blocks, the sharded AdamW, the expert-parallel
MoE layer, Ulysses and all-gather context-parallel attention, and a two-stage GPipe schedule.
"""
from __future__ import annotations

import copy
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _close(a, b, tol, what):
    err = (a.float() - b.float()).abs().max().item()
    scale = max(1.0, b.float().abs().max().item())
    assert err <= tol * scale, f"{what}: max error {err:.3e} (scale {scale:.3e})"


def check_tensor_parallel(dev, rank, world, tol):
    from hylink_b200.models.gpt2 import Block, GPT2Config
    from hylink_b200.parallel.tensor_parallel import TPBlock, allreduce_replicated_grads

    torch.manual_seed(7)
    cfg = GPT2Config(n_layer=1, n_head=4 * world, d_model=32 * world, vocab_size=64, n_ctx=64)
    dense = Block(cfg).to(dev)
    b, t = 2, 8 * world
    x = torch.randn(b, t, cfg.d_model, device=dev)
    xd = x.clone().requires_grad_(True)
    yd = dense(xd)
    yd.square().sum().backward()
    for sp in (False, True):
        blk = TPBlock.from_dense(dense, None, sequence_parallel=sp)
        tl = t // world
        xin = (x[:, rank * tl:(rank + 1) * tl] if sp else x).clone().requires_grad_(True)
        y = blk(xin)
        want = yd[:, rank * tl:(rank + 1) * tl] if sp else yd
        _close(y, want.detach(), tol, f"tp block forward (sp={sp})")
        y.square().sum().backward()
        allreduce_replicated_grads(blk)
        gx = xd.grad[:, rank * tl:(rank + 1) * tl] if sp else xd.grad
        _close(xin.grad, gx, tol, f"tp block input gradient (sp={sp})")
        c = 4 * cfg.d_model // world
        _close(blk.fc.weight.grad, dense.fc.weight.grad[rank * c:(rank + 1) * c], tol, f"tp fc weight gradient (sp={sp})")
        _close(blk.out.weight.grad, dense.out.weight.grad[:, rank * c:(rank + 1) * c], tol, f"tp out weight gradient (sp={sp})")
        # without sequence parallelism the replicated parameters see the whole sequence on every rank; with it the
        # partial sums were completed by allreduce_replicated_grads
        _close(blk.ln1.weight.grad, dense.ln1.weight.grad, tol, f"tp ln1 gradient (sp={sp})")
        _close(blk.out.bias.grad, dense.out.bias.grad, tol, f"tp out bias gradient (sp={sp})")


def check_sharded_adamw(dev, rank, world, tol):
    from hylink_b200.parallel.zero import ShardedAdamW

    torch.manual_seed(11)
    model = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 7)).to(dev)
    ref = copy.deepcopy(model)
    opt = ShardedAdamW(model.parameters(), lr=1e-2, weight_decay=0.1, master_fp32=False)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.1)
    for step in range(3):
        xs = [torch.randn(5, 24, generator=torch.Generator().manual_seed(100 * step + q)).to(dev) for q in range(world)]
        opt.zero_grad()
        model(xs[rank]).square().mean().backward()
        opt.step()
        ropt.zero_grad()
        sum(ref(xq).square().mean() for xq in xs).div(world).backward()   # the mean over ranks of the per-rank losses
        ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        _close(p, q, tol, "sharded AdamW parameters after 3 steps")
    assert opt.state_bytes_per_rank() <= (sum(p.numel() for p in ref.parameters()) // world + 8) * 8


def check_moe(dev, rank, world, tol):
    from hylink_b200.parallel.moe import ExpertParallelMLP

    torch.manual_seed(13)  # same router on every rank; experts differ per rank below
    d, hdim, epr, cap, tokens = 16, 32, 2, 6, 20
    layer = ExpertParallelMLP(d, hdim, experts_per_rank=epr, capacity=cap).to(dev)
    with torch.no_grad():
        g = torch.Generator().manual_seed(1000 + rank)
        layer.w1.copy_(torch.randn(epr, d, hdim, generator=g) * 0.3)
        layer.w2.copy_(torch.randn(epr, hdim, d, generator=g) * 0.3)
    w1 = torch.empty(world * epr, d, hdim, device=dev)
    w2 = torch.empty(world * epr, hdim, d, device=dev)
    dist.all_gather_into_tensor(w1, layer.w1.data.contiguous())
    dist.all_gather_into_tensor(w2, layer.w2.data.contiguous())
    x = torch.randn(tokens, d, generator=torch.Generator().manual_seed(50 + rank)).to(dev).requires_grad_(True)
    y = layer(x)
    xr = x.detach().clone().requires_grad_(True)
    yr = layer.dense_reference(xr, w1, w2)
    _close(y, yr.detach(), tol, "moe forward")
    y.square().sum().backward()
    yr.square().sum().backward()
    _close(x.grad, xr.grad, tol, "moe input gradient")


def check_attention(dev, rank, world, tol):
    from hylink_b200.parallel.sequence_parallel import allgather_kv_attention, ring_attention, ulysses_attention

    torch.manual_seed(17)
    b, t, h, e = 2, 6 * world, 2 * world, 8
    full = [torch.randn(b, t, h, e, device=dev) for _ in range(3)]
    fr = [z.clone().requires_grad_(True) for z in full]
    want = F.scaled_dot_product_attention(*(z.transpose(1, 2) for z in fr), is_causal=True).transpose(1, 2)
    want.square().sum().backward()
    tl = t // world
    sl = slice(rank * tl, (rank + 1) * tl)
    for name, fn in (("ulysses", ulysses_attention), ("allgather-kv", allgather_kv_attention), ("ring", ring_attention)):
        loc = [z[:, sl].clone().requires_grad_(True) for z in full]
        got = fn(*loc, group=None, causal=True)
        _close(got, want[:, sl].detach(), tol, f"{name} attention forward")
        got.square().sum().backward()
        for i, nm in enumerate("qkv"):
            _close(loc[i].grad, fr[i].grad[:, sl], tol, f"{name} attention d{nm}")


def check_pipeline(dev, rank, world, tol):
    from hylink_b200.parallel.pipeline import GPipeStage

    torch.manual_seed(19)
    stages = [torch.nn.Sequential(torch.nn.Linear(12, 12), torch.nn.Tanh()).to(dev) for _ in range(world)]
    mbs = [torch.randn(3, 12, generator=torch.Generator().manual_seed(200 + i)).to(dev) for i in range(4)]
    tgts = [torch.randn(3, 12, generator=torch.Generator().manual_seed(300 + i)).to(dev) for i in range(4)]
    ref = copy.deepcopy(stages)
    total = 0
    for xm, tm in zip(mbs, tgts):
        y = xm
        for s in ref:
            y = s(y)
        total = total + F.mse_loss(y, tm) / len(mbs)
    total.backward()
    st = GPipeStage(stages[rank], rank, world, act_shape=(3, 12), device=dev)
    loss = st.run(mbs if rank == 0 else [None] * len(mbs), loss_fn=F.mse_loss, targets=tgts)
    if rank == world - 1:
        _close(loss, total.detach(), tol, "pipeline loss")
    for p, q in zip(stages[rank].parameters(), ref[rank].parameters()):
        _close(p.grad, q.grad, tol, "pipeline stage gradients")


def main(argv=None) -> int:
    args = argv if argv is not None else sys.argv[1:]
    cpu = "--cpu" in args
    from hylink_b200.parallel import register_backend

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
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    tol = 2e-5 if cpu else 2e-4
    for name, fn in (("tensor/sequence parallel block", check_tensor_parallel), ("sharded AdamW", check_sharded_adamw),
                     ("expert-parallel MoE", check_moe), ("sequence-parallel attention", check_attention),
                     ("GPipe schedule", check_pipeline)):
        fn(dev, rank, world, tol)
        dist.barrier()
        if rank == 0:
            print(f"ok: {name}", flush=True)
    if rank == 0:
        print("PARALLEL SELFTEST PASSED", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
