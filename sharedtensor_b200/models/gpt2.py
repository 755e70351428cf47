"""GPT-2 small (12 layers, d_model 768, 12 heads, context 1024, vocabulary 50257, 124 M parameters).

bf16 compute over fp32 master weights: the masters live in a table-synced shared arena
(:func:`sharedtensor_b200.createOrFetchTable`), the module's parameters are bf16 views of one flat buffer that is
refreshed from the arena by the fused snapshot-and-cast kernel before every step.  The transformer itself is
written with PyTorch operators (library GEMMs and attention); only the synchronisation path is this
framework's own code.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    vocab: int = 50257
    ctx: int = 1024
    d_model: int = 768
    n_head: int = 12
    n_layer: int = 12

    @classmethod
    def tiny(cls) -> "GPT2Config":
        return cls(vocab=257, ctx=64, d_model=64, n_head=4, n_layer=2)


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
        self.cfg = c
        self.wte = nn.Embedding(c.vocab, c.d_model)
        self.wpe = nn.Embedding(c.ctx, c.d_model)
        self.blocks = nn.ModuleList(Block(c) for _ in range(c.n_layer))
        self.ln_f = nn.LayerNorm(c.d_model)
        self.apply(self._init)
        for blk in self.blocks:  # scaled init of the residual projections, as in GPT-2
            for lin in (blk.proj, blk.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * c.n_layer))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, tokens):
        b, t = tokens.shape
        x = self.wte(tokens) + self.wpe(torch.arange(t, device=tokens.device))
        for blk in self.blocks:
            x = blk(x)
        return F.linear(self.ln_f(x), self.wte.weight)  # tied output embedding

    def loss(self, tokens, targets):
        logits = self(tokens)
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
