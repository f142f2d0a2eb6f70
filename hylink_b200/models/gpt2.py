"""GPT-2 (the benchmark workload): decoder-only transformer with learned
positions, pre-LayerNorm blocks, GELU MLP and a tied output head.

``GPT2Config.medium()`` is the configuration the headline benchmark names:
24 layers, d_model 1024, 16 heads, vocabulary 50257, context 1024. Weights are
random-initialised (no checkpoints are available offline); the model exists so
that the collective library can be measured under a real DDP training step,
with gradient buckets overlapping the backward pass.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    vocab_size: int = 50257
    n_ctx: int = 1024
    dropout: float = 0.0

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, n_head=4, d_model=128, vocab_size=1024, n_ctx=128)

    @staticmethod
    def by_name(name: str) -> "GPT2Config":
        return {"gpt2-medium": GPT2Config.medium, "medium": GPT2Config.medium, "tiny": GPT2Config.tiny,
                "gpt2-small": lambda: GPT2Config(n_layer=12, n_head=12, d_model=768)}[name]()


class Block(nn.Module):
    def __init__(self, c: GPT2Config):
        super().__init__()
        self.ln1 = nn.LayerNorm(c.d_model)
        self.qkv = nn.Linear(c.d_model, 3 * c.d_model)
        self.proj = nn.Linear(c.d_model, c.d_model)
        self.ln2 = nn.LayerNorm(c.d_model)
        self.fc = nn.Linear(c.d_model, 4 * c.d_model)
        self.out = nn.Linear(4 * c.d_model, c.d_model)
        self.n_head = c.n_head

    def forward(self, x):
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.n_head, d // self.n_head).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, d))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, c: GPT2Config):
        super().__init__()
        self.config = c
        self.wte = nn.Embedding(c.vocab_size, c.d_model)
        self.wpe = nn.Embedding(c.n_ctx, c.d_model)
        self.blocks = nn.ModuleList([Block(c) for _ in range(c.n_layer)])
        self.ln_f = nn.LayerNorm(c.d_model)
        self.apply(self._init)
        for blk in self.blocks:  # scaled init of the residual projections
            for p in (blk.proj.weight, blk.out.weight):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * c.n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        b, t = idx.shape
        pos = torch.arange(t, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        x = self.ln_f(x)
        logits = F.linear(x, self.wte.weight)  # tied head
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def smoke_step() -> float:
    """One tiny forward + backward + fused all-reduce of the gradients on cuda:0."""
    from ..ops import EmuGroup

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    model = GPT2(GPT2Config.tiny()).to(dev, torch.bfloat16)
    idx = torch.randint(0, 1024, (2, 64), device=dev)
    loss = model(idx, idx)
    loss.backward()
    # the gradients of two emulated ranks go through the NVLink all-reduce kernel
    flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    g = EmuGroup(2, stage_bytes=16 << 20)
    ins = [flat.clone(), flat.clone()]
    outs = [torch.empty_like(flat), torch.empty_like(flat)]
    g.run("all_reduce", ins, outs, flat.numel(), scale=0.5, algo="twoshot")
    torch.cuda.synchronize()
    assert torch.equal(outs[0], ((flat.float() + flat.float()) * 0.5).to(torch.bfloat16))
    g.close()
    return float(loss.detach())
