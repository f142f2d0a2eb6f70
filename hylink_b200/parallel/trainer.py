"""A small data-parallel trainer on the ``hylink`` backend.

``DDPTrainer`` is the user-facing entry for the benchmark workload: it wraps
the model in ``DistributedDataParallel`` over this library's process group
(25 MB gradient buckets by default), owns a fused AdamW, and exposes
``step(tokens)`` which takes a pinned host batch, copies it to the device,
runs forward / backward (gradient all-reduces overlap the backward pass on the
backend's own stream) / optimizer, and returns the loss as a Python float.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP


def init_distributed(backend: str = "hylink"):
    """Initialise ``torch.distributed`` from torchrun's environment (or as a single rank)."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if backend == "hylink":
        from .backend import register_backend

        register_backend()
    if not dist.is_initialized():
        dist.init_process_group(backend, rank=rank, world_size=world, device_id=dev)
    return rank, world, dev


class DDPTrainer:
    def __init__(self, model: torch.nn.Module, device: torch.device, lr: float = 3e-4, bucket_cap_mb: int = 25,
                 dtype: torch.dtype = torch.bfloat16, cta_budget: int | None = None):
        self.device = device
        # gradient all-reduces overlap the backward pass: they get a CTA budget (the GEMMs keep the other SMs)
        self._old_budget = None
        if dist.get_backend() == "hylink":
            from .backend import set_cta_budget

            if cta_budget is None:
                cta_budget = int(os.environ.get("HYLINK_DDP_CTA_BUDGET", "32"))
            self._old_budget = set_cta_budget(cta_budget)
        self.model = model.to(device=device, dtype=dtype)
        self.registered_buckets = False
        self._pool = None
        self._steps = 0
        pool = None
        if dist.get_backend() == "hylink" and dist.get_world_size() > 1 and os.environ.get("HYLINK_DDP_REGISTERED", "1") != "0":
            # Gradient buckets in registered memory: the bucket all-reduces then run zero-copy, in place in every
            # rank's bucket (multimem load-reduce / store through NVSwitch), on a few SMs beside the backward GEMMs.
            try:
                from .backend import registered_mem_pool

                dist.barrier()                       # the group's communicator (and its allocator) exists after this
                pool = registered_mem_pool()
            except Exception as ex:  # noqa: BLE001 - an older PyTorch without pluggable pools: buckets are staged
                print(f"hylink: gradient buckets stay unregistered ({type(ex).__name__}: {ex})", flush=True)
        if pool is not None:
            with torch.cuda.use_mem_pool(pool):
                self.ddp = DDP(self.model, device_ids=[device.index], bucket_cap_mb=bucket_cap_mb, gradient_as_bucket_view=True,
                               static_graph=False)
            self.registered_buckets = True
            self._pool = pool
        else:
            self.ddp = DDP(self.model, device_ids=[device.index], bucket_cap_mb=bucket_cap_mb, gradient_as_bucket_view=True,
                           static_graph=False)
        self.opt = torch.optim.AdamW(self.ddp.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self._dev_batch = None

    def close(self) -> None:
        """Gives the process group its previous CTA budget back."""
        if self._old_budget is not None:
            from .backend import set_cta_budget

            set_cta_budget(self._old_budget)
            self._old_budget = None

    def step_device(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimisation step on device-resident tokens; returns the loss tensor (no host sync)."""
        if self._pool is not None and self._steps == 1:
            # DDP re-buckets its gradients once, before the second forward pass, in the order they became ready:
            # do that here, under the registered pool, so that the new buckets are registered too.
            with torch.cuda.use_mem_pool(self._pool):
                if self.ddp.reducer._rebuild_buckets():
                    self.ddp._has_rebuilt_buckets = True
        self._steps += 1
        loss = self.ddp(idx, targets)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return loss

    def step(self, tokens: torch.Tensor) -> float:
        """``tokens``: pinned host tensor [batch, seq + 1] of token ids. Returns the loss."""
        if self._dev_batch is None or self._dev_batch.shape != tokens.shape:
            self._dev_batch = torch.empty(tokens.shape, dtype=tokens.dtype, device=self.device)
        self._dev_batch.copy_(tokens, non_blocking=True)
        loss = self.step_device(self._dev_batch[:, :-1], self._dev_batch[:, 1:])
        self._loss_host.copy_(loss.detach().float().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(self._loss_host[0])
