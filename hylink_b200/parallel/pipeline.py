"""Pipeline parallelism: a GPipe schedule (all forward micro-batches, then all
backward ones) whose stage-to-stage traffic is point-to-point send/recv.

Send/recv is deliberately NOT served by this library's collective kernels: like
the reference (multipath-orchestrator/libampccl/hook/nccl_hook.cc:637-646), it
leaves them to the vendor library, on a side process group and its own stream,
so that pipeline traffic overlaps with the collectives of the other parallel
dimensions (see :mod:`hylink_b200.parallel.p2p`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import p2p


class GPipeStage:
    """One stage of a linear pipeline; stage ``s`` runs on rank ``s`` of the group."""

    def __init__(self, module: torch.nn.Module, stage: int, n_stages: int, act_shape, act_dtype=torch.float32, device=None):
        self.module, self.stage, self.n = module, stage, n_stages
        self.shape, self.dtype = tuple(act_shape), act_dtype
        self.device = device if device is not None else next(module.parameters()).device

    def run(self, micro_batches, loss_fn=None, targets=None):
        """Forward and backward over all micro-batches.

        ``micro_batches``: inputs (first stage only; other stages pass their count as a list of ``None``).
        ``loss_fn(output, target)`` and ``targets`` are used by the last stage. Returns the mean loss on the
        last stage, ``None`` elsewhere. Parameter gradients are accumulated in ``.grad`` as usual.
        """
        first, last = self.stage == 0, self.stage == self.n - 1
        saved_in, saved_out, losses = [], [], []
        for i, mb in enumerate(micro_batches):
            if first:
                x = mb
            else:
                x = torch.empty(self.shape, dtype=self.dtype, device=self.device)
                p2p.recv(x, self.stage - 1)
                x.requires_grad_(True)
            y = self.module(x)
            if last:
                loss = loss_fn(y, targets[i]) / len(micro_batches)
                losses.append(loss.detach())
                saved_out.append(loss)
            else:
                p2p.send(y.detach().contiguous(), self.stage + 1)
                saved_out.append(y)
            saved_in.append(x)
        for i in range(len(micro_batches)):
            if last:
                saved_out[i].backward()
            else:
                g = torch.empty_like(saved_out[i])
                p2p.recv(g, self.stage + 1)
                saved_out[i].backward(g)
            if not first:
                p2p.send(saved_in[i].grad.contiguous(), self.stage - 1)
        return torch.stack(losses).sum() if last else None
