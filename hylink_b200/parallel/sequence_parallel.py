"""Long-context attention over a sequence that is sharded across ranks.

Two schemes, both absent from the reference (it has no attention code and no
ring schedule) but built from collectives it does carry:

* :func:`ulysses_attention` — all-to-all switches the sharding from sequence
  to heads, every rank runs ordinary attention on whole sequences of its
  heads, a second all-to-all switches back. Traffic: two all-to-alls of the
  activations per call, independent of the group size.
* :func:`allgather_kv_attention` — context parallelism by gathering K and V:
  every rank keeps its queries, all-gathers keys and values, and applies the
  causal mask for its own slice of positions. Traffic: one all-gather of K
  and V (reduce-scatter of their gradients in backward).

Ring-style point-to-point schedules stay on NCCL send/recv
(:mod:`hylink_b200.parallel.p2p`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .moe import all_to_all


def _seq_to_heads(x: torch.Tensor, group) -> torch.Tensor:
    """[b, t/n, h, e] -> [b, t, h/n, e]."""
    n = dist.get_world_size(group)
    b, tl, h, e = x.shape
    # chunk q of dim 0 goes to rank q: put the destination (head group) first
    send = x.view(b, tl, n, h // n, e).permute(2, 1, 0, 3, 4).contiguous()      # [n(dst), t/n, b, h/n, e]
    recv = all_to_all(send.view(n * tl, b, h // n, e), group)                    # [n(src) * t/n, b, h/n, e] = whole sequence
    return recv.permute(1, 0, 2, 3).contiguous()                                 # [b, t, h/n, e]


def _heads_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[b, t, h/n, e] -> [b, t/n, h, e]."""
    n = dist.get_world_size(group)
    b, t, hl, e = x.shape
    send = x.permute(1, 0, 2, 3).contiguous()                                    # [t = n(dst) * t/n, b, h/n, e]
    recv = all_to_all(send, group)                                               # [n(src head group) * t/n, b, h/n, e]
    return recv.view(n, t // n, b, hl, e).permute(2, 1, 0, 3, 4).reshape(b, t // n, n * hl, e)


def ulysses_attention(q, k, v, group=None, causal: bool = True):
    """q, k, v: [b, t/n, heads, head_dim], sequence sharded in rank order. Returns the same layout."""
    qh, kh, vh = (_seq_to_heads(z, group).transpose(1, 2) for z in (q, k, v))    # [b, h/n, t, e]
    a = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal)
    return _heads_to_seq(a.transpose(1, 2).contiguous(), group)


class _GatherTime(torch.autograd.Function):
    """All-gather along dimension 0 forward, reduce-scatter (sum) backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        x = x.contiguous()
        out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = torch.empty((g.shape[0] // n,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None


def allgather_kv_attention(q, k, v, group=None, causal: bool = True):
    """q, k, v: [b, t/n, heads, head_dim], sequence sharded in rank order. Returns the same layout."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    b, tl, h, e = q.shape
    kf = _GatherTime.apply(k.transpose(0, 1), group).transpose(0, 1)             # [b, t, h, e]
    vf = _GatherTime.apply(v.transpose(0, 1), group).transpose(0, 1)
    mask = None
    if causal:
        qpos = torch.arange(r * tl, (r + 1) * tl, device=q.device)[:, None]
        mask = qpos >= torch.arange(n * tl, device=q.device)[None, :]
    a = F.scaled_dot_product_attention(q.transpose(1, 2), kf.transpose(1, 2), vf.transpose(1, 2), attn_mask=mask)
    return a.transpose(1, 2).contiguous()
