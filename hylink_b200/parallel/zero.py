"""Optimizer-state and gradient sharding (the ZeRO / FSDP traffic pattern):
reduce-scatter of the gradients, an optimizer step on the local shard only,
all-gather of the updated parameters.

The reference lists ZeRO/FSDP as a consumer of its reduce-scatter and
all-gather (it ships neither); this module is that consumer for the
``torch.distributed`` backend of this library. All parameters live in ONE flat
buffer padded to a multiple of the group size, so a step is exactly one
reduce-scatter and one all-gather whatever the number of tensors, and the
parameters of the model are views into the buffer (no copies around the
collectives).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class ShardedAdamW:
    """AdamW whose moments (and, optionally, fp32 master weights) exist only for this rank's 1/n of the parameters."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 group=None, master_fp32: bool = True):
        self.group = group
        self.n, self.r = dist.get_world_size(group), dist.get_rank(group)
        self.params = [p for p in params if p.requires_grad]
        assert self.params, "no parameters"
        dev, dt = self.params[0].device, self.params[0].dtype
        assert all(p.dtype == dt and p.device == dev for p in self.params), "one dtype and device per optimizer"
        total = sum(p.numel() for p in self.params)
        # every shard a multiple of 8 elements: 16-byte packets on the wire for 16-bit types
        self.shard = -(-total // (self.n * 8)) * 8
        self.flat = torch.zeros(self.shard * self.n, dtype=dt, device=dev)
        self.flat_grad = torch.zeros_like(self.flat)
        off = 0
        for p in self.params:
            k = p.numel()
            self.flat[off:off + k].copy_(p.data.reshape(-1))
            p.data = self.flat[off:off + k].view_as(p.data)       # the model now computes on views of the flat buffer
            p.grad = self.flat_grad[off:off + k].view_as(p.data)  # and accumulates gradients straight into the flat one
            off += k
        self.total = total
        mine = self.flat[self.r * self.shard:(self.r + 1) * self.shard]
        self.master = mine.float().clone() if (master_fp32 and dt != torch.float32) else None
        self.m = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.grad_shard = torch.empty(self.shard, dtype=dt, device=dev)
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.t = 0

    def zero_grad(self) -> None:
        self.flat_grad.zero_()

    @torch.no_grad()
    def step(self) -> None:
        """Mean-reduce gradients to their owners, update the owned shard, gather the new parameters."""
        dist.reduce_scatter_tensor(self.grad_shard, self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
        g = self.grad_shard.float().div_(self.n)
        self.t += 1
        b1, b2 = self.betas
        mine = self.flat[self.r * self.shard:(self.r + 1) * self.shard]
        w = self.master if self.master is not None else mine.float()
        w.mul_(1 - self.lr * self.wd)
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        step = self.lr / (1 - b1 ** self.t)
        denom = (self.v / (1 - b2 ** self.t)).sqrt_().add_(self.eps)
        w.addcdiv_(self.m, denom, value=-step)
        mine.copy_(w)
        dist.all_gather_into_tensor(self.flat, mine.clone(), group=self.group)

    def state_bytes_per_rank(self) -> int:
        return (self.m.numel() + self.v.numel() + (self.master.numel() if self.master is not None else 0)) * 4
