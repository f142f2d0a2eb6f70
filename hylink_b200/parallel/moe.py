"""Expert parallelism: a mixture-of-experts MLP whose tokens travel to their
expert's rank and back with two all-to-all calls.

The reference carries all-to-all as a primitive (native and strided:
pcie-ccl-cuda/include/pccl/pccl.h:47-51,107-110; orchestrated in
multipath-orchestrator/libampccl/hook/nccl_hook.cc:564-599) without a layer that
uses it; this is that layer. Routing is top-1 with a fixed capacity per
(source rank, expert), so every all-to-all moves equal splits — the form the
all-to-all kernels of this library implement. Tokens beyond an expert's
capacity pass through unchanged (their residual path), as in capacity-factor
MoE implementations.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all over dimension 0; its own transpose in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def all_to_all(x: torch.Tensor, group=None) -> torch.Tensor:
    """Differentiable equal-split all-to-all: chunk q of dimension 0 goes to rank q."""
    return _AllToAll.apply(x, group)


class ExpertParallelMLP(nn.Module):
    """``experts_per_rank`` GELU MLPs on every rank; ``n * experts_per_rank`` experts in total."""

    def __init__(self, d_model: int, d_hidden: int, experts_per_rank: int = 1, capacity: int = 64, group=None):
        super().__init__()
        self.group = group
        self.n, self.r = dist.get_world_size(group), dist.get_rank(group)
        self.epr, self.cap = experts_per_rank, capacity
        self.n_experts = self.n * experts_per_rank
        self.router = nn.Linear(d_model, self.n_experts, bias=False)
        self.w1 = nn.Parameter(torch.randn(experts_per_rank, d_model, d_hidden) * 0.02)
        self.w2 = nn.Parameter(torch.randn(experts_per_rank, d_hidden, d_model) * 0.02)

    def forward(self, x):
        """x: [tokens, d_model] (this rank's tokens). Returns the same shape."""
        t, d = x.shape
        probs = F.softmax(self.router(x).float(), dim=-1)
        gate, expert = probs.max(dim=-1)                                   # top-1
        # position of every token in its expert's queue on THIS rank (arrival order), capacity cut
        onehot = F.one_hot(expert, self.n_experts)
        pos = (onehot.cumsum(0) - 1).gather(1, expert[:, None]).squeeze(1)
        keep = pos < self.cap
        slot = expert * self.cap + pos                                     # row in the dispatch buffer
        send = x.new_zeros(self.n_experts * self.cap, d)
        send = send.index_add(0, slot[keep], x[keep])                      # differentiable scatter
        # rows are ordered (destination rank, local expert, slot): equal splits of epr*cap rows per rank
        recv = all_to_all(send, self.group)                                # [(source rank, local expert, slot), d]
        h = recv.view(self.n, self.epr, self.cap, d).transpose(0, 1).reshape(self.epr, self.n * self.cap, d)
        h = torch.bmm(F.gelu(torch.bmm(h, self.w1.to(h.dtype)), approximate="tanh"), self.w2.to(h.dtype))
        back = h.view(self.epr, self.n, self.cap, d).transpose(0, 1).reshape(self.n_experts * self.cap, d)
        got = all_to_all(back, self.group)                                 # same row layout as `send`
        y = x.clone()
        y[keep] = x[keep] + gate[keep, None].to(x.dtype) * got[slot[keep]]
        return y

    def dense_reference(self, x, all_w1, all_w2):
        """The same layer computed without communication from all experts' weights (for tests)."""
        probs = F.softmax(self.router(x).float(), dim=-1)
        gate, expert = probs.max(dim=-1)
        onehot = F.one_hot(expert, self.n_experts)
        pos = (onehot.cumsum(0) - 1).gather(1, expert[:, None]).squeeze(1)
        keep = pos < self.cap
        y = x.clone()
        for e in range(self.n_experts):
            m = keep & (expert == e)
            if m.any():
                h = F.gelu(x[m] @ all_w1[e].to(x.dtype), approximate="tanh") @ all_w2[e].to(x.dtype)
                y[m] = x[m] + gate[m, None].to(x.dtype) * h
        return y
