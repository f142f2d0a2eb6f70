"""Tensor parallelism and Megatron-style sequence parallelism over the process
group's collectives.

The reference implements no parallelism itself; it is exercised by Megatron
with tensor parallel size 4, optionally with ``--sequence-parallel``
(pcie-ccl-cuda/README.md:640-663, pcie-ccl-cuda/torch_dist_smoke/run_megatron.sh:19-41).
These layers produce exactly that traffic on this library's backend:

* tensor parallel: one all-reduce of the activations after every row-parallel
  linear in the forward pass and one all-reduce of the input gradient before
  every column-parallel linear in the backward pass;
* sequence parallel: the activations between blocks are sharded along the
  sequence; the all-reduce pair becomes an all-gather (before the column
  linear) and a reduce-scatter (after the row linear), mirrored in backward.

``TPBlock`` is the transformer block of :mod:`hylink_b200.models.gpt2` with its
attention heads and MLP columns split over the group; ``TPBlock.from_dense``
cuts a rank's shard out of a dense block, which is how the tests check the
parallel block against the dense one.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _world(group) -> int:
    return dist.get_world_size(group)


class _CopyToRegion(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient backward (entry of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRegion(torch.autograd.Function):
    """All-reduce forward, identity backward (exit of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _gather_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[b, t/n, d] on every rank -> [b, t, d]; the sequence is sharded in rank order."""
    n = _world(group)
    xt = x.transpose(0, 1).contiguous()  # [t/n, b, d]: the gathered dimension must be the outermost one
    out = torch.empty((n * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, xt, group=group)
    return out.transpose(0, 1).contiguous()


def _scatter_sum_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[b, t, d] partial sums on every rank -> this rank's [b, t/n, d] slice of the total."""
    n = _world(group)
    xt = x.transpose(0, 1).contiguous()
    out = torch.empty((xt.shape[0] // n,) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, xt, group=group)
    return out.transpose(0, 1).contiguous()


class _GatherSeq(torch.autograd.Function):
    """All-gather along the sequence forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _scatter_sum_seq(g, ctx.group), None


class _ScatterSumSeq(torch.autograd.Function):
    """Reduce-scatter along the sequence forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _scatter_sum_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.group), None


class ColumnParallelLinear(nn.Module):
    """``y_r = x W_r^T + b_r`` with the output features split over the group."""

    def __init__(self, in_features: int, out_features: int, group=None, sequence_parallel: bool = False, bias: bool = True):
        super().__init__()
        self.group = group
        self.sequence_parallel = sequence_parallel
        n = _world(group)
        assert out_features % n == 0, "output features must divide by the group size"
        self.weight = nn.Parameter(torch.empty(out_features // n, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features // n)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        x = _GatherSeq.apply(x, self.group) if self.sequence_parallel else _CopyToRegion.apply(x, self.group)
        return F.linear(x, self.weight, self.bias)


class RowParallelLinear(nn.Module):
    """``y = sum_r x_r W_r^T + b`` with the input features split over the group."""

    def __init__(self, in_features: int, out_features: int, group=None, sequence_parallel: bool = False, bias: bool = True):
        super().__init__()
        self.group = group
        self.sequence_parallel = sequence_parallel
        n = _world(group)
        assert in_features % n == 0, "input features must divide by the group size"
        self.weight = nn.Parameter(torch.empty(out_features, in_features // n))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        y = F.linear(x, self.weight)
        y = _ScatterSumSeq.apply(y, self.group) if self.sequence_parallel else _ReduceFromRegion.apply(y, self.group)
        return y if self.bias is None else y + self.bias


class TPBlock(nn.Module):
    """Pre-LayerNorm transformer block with heads and MLP columns split over the group.

    With ``sequence_parallel`` the block's input and output are this rank's
    slice ``[b, t/n, d]`` of the sequence; LayerNorm, residuals and biases of
    the row-parallel linears then work on the slice only.
    """

    def __init__(self, d_model: int, n_head: int, group=None, sequence_parallel: bool = False):
        super().__init__()
        n = _world(group)
        assert n_head % n == 0, "heads must divide by the group size"
        self.group, self.sp = group, sequence_parallel
        self.heads_local, self.head_dim = n_head // n, d_model // n_head
        self.ln1 = nn.LayerNorm(d_model)
        self.qkv = ColumnParallelLinear(d_model, 3 * d_model, group, sequence_parallel)
        self.proj = RowParallelLinear(d_model, d_model, group, sequence_parallel)
        self.ln2 = nn.LayerNorm(d_model)
        self.fc = ColumnParallelLinear(d_model, 4 * d_model, group, sequence_parallel)
        self.out = RowParallelLinear(4 * d_model, d_model, group, sequence_parallel)

    def forward(self, x):
        h = self.qkv(self.ln1(x))  # [b, t, 3 * heads_local * head_dim], full sequence
        b, t, _ = h.shape
        q, k, v = h.view(b, t, 3, self.heads_local, self.head_dim).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, self.heads_local * self.head_dim))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))

    @staticmethod
    def from_dense(dense, group=None, sequence_parallel: bool = False) -> "TPBlock":
        """This rank's shard of a dense block (:class:`hylink_b200.models.gpt2.Block`)."""
        n, r = _world(group), dist.get_rank(group)
        d = dense.proj.weight.shape[0]
        blk = TPBlock(d, dense.n_head, group, sequence_parallel).to(dense.proj.weight.device, dense.proj.weight.dtype)
        hl, hd = blk.heads_local, blk.head_dim
        with torch.no_grad():
            for name in ("ln1", "ln2"):
                getattr(blk, name).load_state_dict(getattr(dense, name).state_dict())
            # dense qkv rows are ordered (which of q/k/v, head, head_dim): keep this rank's heads of each of the three
            w = dense.qkv.weight.view(3, dense.n_head, hd, d)[:, r * hl:(r + 1) * hl]
            blk.qkv.weight.copy_(w.reshape(3 * hl * hd, d))
            blk.qkv.bias.copy_(dense.qkv.bias.view(3, dense.n_head, hd)[:, r * hl:(r + 1) * hl].reshape(-1))
            blk.proj.weight.copy_(dense.proj.weight[:, r * hl * hd:(r + 1) * hl * hd])
            blk.proj.bias.copy_(dense.proj.bias)
            c = 4 * d // n
            blk.fc.weight.copy_(dense.fc.weight[r * c:(r + 1) * c])
            blk.fc.bias.copy_(dense.fc.bias[r * c:(r + 1) * c])
            blk.out.weight.copy_(dense.out.weight[:, r * c:(r + 1) * c])
            blk.out.bias.copy_(dense.out.bias)
        return blk


def allreduce_replicated_grads(module: nn.Module, group=None) -> None:
    """Sum the gradients of parameters that are replicated but saw only a slice of the sequence.

    Under sequence parallelism LayerNorm weights and the biases of row-parallel
    linears are applied to this rank's tokens only, so their gradients are
    partial sums; one all-reduce per such parameter completes them.
    """
    for m in module.modules():
        if isinstance(m, TPBlock) and m.sp:
            for p in (m.ln1.weight, m.ln1.bias, m.ln2.weight, m.ln2.bias, m.proj.bias, m.out.bias):
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=group)
