"""char-RNN: 2-layer LSTM, hidden 512, vocabulary 65, all parameters (about 3.3 M fp32) in one flat tensor.

The reference's README lists a char-rnn example as a TODO (README.md:37); this is the model that example would
train.  Forward and backward use PyTorch's LSTM; what this framework adds is the flat parameter buffer whose
views the module uses, so that ``copyToTensor`` / ``pushUpdate`` move the whole model in one call.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class CharRNN(nn.Module):
    def __init__(self, vocab: int = 65, hidden: int = 512, layers: int = 2):
        super().__init__()
        self.vocab, self.hidden, self.layers = vocab, hidden, layers
        self.embed = nn.Embedding(vocab, vocab)
        self.lstm = nn.LSTM(vocab, hidden, num_layers=layers, batch_first=True)
        self.head = nn.Linear(hidden, vocab)
        self.embed.weight.data.copy_(torch.eye(vocab))  # one-hot inputs, as in char-rnn
        self.embed.weight.requires_grad_(False)

    def forward(self, tokens: torch.Tensor, state=None):
        x = self.embed(tokens)
        y, state = self.lstm(x, state)
        return self.head(y), state

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        logits, _ = self(tokens)
        return F.cross_entropy(logits.reshape(-1, self.vocab), targets.reshape(-1))


def flatten_parameters(module: nn.Module, align: int = 1, dtype: torch.dtype = torch.float32):
    """Moves every trainable parameter of ``module`` into one flat buffer and makes the parameters views of it.
    Returns ``(flat, offsets)``; offsets are multiples of ``align``."""
    params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
    offsets, off = {}, 0
    for n, p in params:
        offsets[n] = off
        off += (p.numel() + align - 1) // align * align
    device = params[0][1].device
    flat = torch.zeros(max(off, 1), dtype=dtype, device=device)
    for n, p in params:
        view = flat[offsets[n]: offsets[n] + p.numel()].view(p.shape)
        view.copy_(p.data)
        p.data = view
    return flat, offsets


def flat_gradient(module: nn.Module, offsets: dict, numel: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Gathers the gradients into a flat buffer with the layout of :func:`flatten_parameters`."""
    params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
    g = out if out is not None else torch.zeros(numel, dtype=torch.float32, device=params[0][1].device)
    for n, p in params:
        if p.grad is not None:
            g[offsets[n]: offsets[n] + p.numel()].copy_(p.grad.reshape(-1))
    return g
