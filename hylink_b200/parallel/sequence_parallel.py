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

* :func:`ring_attention` — context parallelism with a ring schedule: the K/V
  blocks travel once around the ring (n - 1 point-to-point shifts on the NCCL
  side group of :mod:`hylink_b200.parallel.p2p`, next to this library's
  collectives), every rank attends its queries to the block it currently
  holds and merges the partial results with a running log-sum-exp, so no rank
  ever holds more than two K/V blocks. Blocks that lie entirely in the causal
  future are not computed. Traffic: (n - 1)/n of K and V per rank, like the
  all-gather, but in n - 1 steps that overlap with the block computations.
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


class _RingShift(torch.autograd.Function):
    """Sends a tensor to the next rank of the ring and returns what the previous rank sent; gradients go the other way."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _shift(x, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _shift(g, ctx.group, -1), None


def _shift(x: torch.Tensor, group, direction: int) -> torch.Tensor:
    from . import p2p

    n, r = dist.get_world_size(group), dist.get_rank(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty_like(x)
    dst, src = (r + direction) % n, (r - direction) % n
    if group is not None:
        dst, src = dist.get_global_rank(group, dst), dist.get_global_rank(group, src)
    for req in p2p.batch_isend_irecv([("send", x, dst), ("recv", out, src)]):
        req.wait()
    return out


def ring_attention(q, k, v, group=None, causal: bool = True):
    """q, k, v: [b, t/n, heads, head_dim], sequence sharded in rank order. Returns the same layout.

    Step s works on the K/V block that started on rank (r - s) mod n while the next shift is already in flight."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    b, tl, h, e = q.shape
    scale = e ** -0.5
    qh = q.transpose(1, 2)                                           # [b, h, tl, e]
    kv = torch.stack((k, v))                                         # one message per shift
    out = None
    lse = None
    tri = torch.ones(tl, tl, dtype=torch.bool, device=q.device).tril() if causal else None
    for s_ in range(n):
        owner = (r - s_) % n
        nxt = _RingShift.apply(kv, group) if s_ + 1 < n else None    # issued before this block's math
        if not causal or owner <= r:
            kh, vh = kv[0].transpose(1, 2), kv[1].transpose(1, 2)
            scores = torch.matmul(qh, kh.transpose(-1, -2)) * scale  # [b, h, tl, tl]
            if causal and owner == r:
                scores = scores.masked_fill(~tri, float("-inf"))
            blk_lse = torch.logsumexp(scores.float(), dim=-1)        # [b, h, tl]
            blk_out = torch.matmul(torch.exp(scores.float() - blk_lse[..., None]).to(vh.dtype), vh)
            if out is None:
                out, lse = blk_out.float(), blk_lse
            else:
                new = torch.logaddexp(lse, blk_lse)
                out = out * torch.exp(lse - new)[..., None] + blk_out.float() * torch.exp(blk_lse - new)[..., None]
                lse = new
        if nxt is None:
            # Every rank must run every shift's backward (its neighbours wait for it there), also the ranks whose
            # last blocks lie in the causal future and never enter the math: tie the end of the chain to the result.
            out = out + kv.float().sum() * 0.0
        kv = nxt
    return out.to(q.dtype).transpose(1, 2).contiguous()
