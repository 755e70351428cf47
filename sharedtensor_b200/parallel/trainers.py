"""Data-parallel trainers.

``AsyncTrainer`` is the product: every rank trains on its own data and shares progress through a shared tensor
(the reference's loop, README.md:15-19: ``copyToTensor`` -> learn -> ``addFromTensor(new - current)``).
``SyncTrainer`` is the baseline it is measured against: gradients averaged with an NCCL all-reduce every step.
Both record (wall-clock seconds, loss) pairs and the time spent in synchronisation calls on the training stream.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.char_rnn import flatten_parameters


@dataclass
class TrainLog:
    wall: list = field(default_factory=list)
    loss: list = field(default_factory=list)
    tokens: int = 0
    seconds: float = 0.0
    sync_seconds: float = 0.0   # copyToTensor + push (async) or all-reduce + update (sync), as seen by the training stream

    @property
    def tokens_per_s(self) -> float:
        return self.tokens / self.seconds if self.seconds else 0.0

    def summary(self) -> dict:
        return {"tokens_per_s": self.tokens_per_s, "seconds": self.seconds, "exposed_sync_s": self.sync_seconds,
                "exposed_sync_frac": self.sync_seconds / self.seconds if self.seconds else 0.0,
                "first_loss": self.loss[0] if self.loss else None, "last_loss": self.loss[-1] if self.loss else None}


def _grad_views(module: torch.nn.Module, offsets: dict, gflat: torch.Tensor) -> None:
    """Points every parameter's .grad at its slice of one flat gradient buffer."""
    for n, p in module.named_parameters():
        if p.requires_grad:
            p.grad = gflat[offsets[n]: offsets[n] + p.numel()].view(p.shape)


class _Base:
    def __init__(self, model: torch.nn.Module, lr: float, align: int = 32, param_dtype: torch.dtype = torch.float32):
        self.model = model
        self.lr = lr
        self.dtype = param_dtype
        if param_dtype != torch.float32:
            model.to(param_dtype)
        self.flat, self.offsets = flatten_parameters(model, align=align, dtype=param_dtype)
        self.gflat = torch.zeros_like(self.flat)
        _grad_views(model, self.offsets, self.gflat)
        self.device = self.flat.device
        self.log = TrainLog()

    def _timed(self, fn) -> None:
        if self.device.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            self._events.append((e0, e1))
        else:
            t0 = time.perf_counter()
            fn()
            self.log.sync_seconds += time.perf_counter() - t0

    def run(self, batches, steps: int, log_every: int = 10) -> TrainLog:
        self._events = []
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        for step in range(steps):
            tokens, targets = next(batches)
            self._timed(self.pull)
            self.gflat.zero_()
            loss = self.model.loss(tokens, targets)
            loss.backward()
            self._timed(self.push)
            self.log.tokens += tokens.numel()
            if step % log_every == 0 or step == steps - 1:
                self.log.loss.append(float(loss.detach()))
                self.log.wall.append(time.perf_counter() - t0)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            self.log.sync_seconds += sum(a.elapsed_time(b) for a, b in self._events) / 1e3
        self.log.seconds = time.perf_counter() - t0
        return self.log

    def pull(self) -> None:
        raise NotImplementedError

    def push(self) -> None:
        raise NotImplementedError


class AsyncTrainer(_Base):
    """SGD on a shared tensor: ``w <- shared`` (one snapshot kernel), backward, ``shared += -lr * g`` (one add kernel).
    With bf16 parameters the shared tensor holds fp32 masters: the snapshot casts, the add consumes bf16 gradients."""

    def __init__(self, model, shared, lr: float, param_dtype: torch.dtype = torch.float32, align: int = 32,
                 rounds_per_step: int = 0):
        """``rounds_per_step`` > 0 is for a shared tensor created with ``engine="manual"``: the trainer then queues
        that many sync rounds behind every update (on the comm stream, overlapping the next forward pass) instead of
        leaving the rounds to a free-running engine thread.  One round per step is enough to keep up: what a round
        could not send stays in the residual and goes out with the next one."""
        super().__init__(model, lr, align=align, param_dtype=param_dtype)
        self.shared = shared
        self.rounds_per_step = rounds_per_step
        if shared.numel != self.flat.numel():
            raise ValueError("Not the right size!")

    def pull(self) -> None:
        if self.dtype == torch.bfloat16:
            self.shared.copyToTensorBF16(self.flat)
        else:
            self.shared.copyToTensor(self.flat)

    def push(self) -> None:
        if self.dtype == torch.bfloat16:
            self.shared.addScaledBF16(self.gflat, -self.lr)
        else:
            self.gflat.mul_(-self.lr)
            self.shared.addFromTensor(self.gflat)
        if self.rounds_per_step > 0:
            self.shared.step(self.rounds_per_step)


class SyncTrainer(_Base):
    """Synchronous data parallelism: gradients are averaged over the process group every step (NCCL on GPUs)."""

    def __init__(self, model, lr: float, param_dtype: torch.dtype = torch.float32, align: int = 32, group=None):
        super().__init__(model, lr, align=align, param_dtype=param_dtype)
        self.master = self.flat.float().clone() if param_dtype != torch.float32 else None
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 1:  # every rank starts from rank 0's weights
            dist.broadcast(self.flat, 0, group=group)
            if self.master is not None:
                self.master.copy_(self.flat)

    def pull(self) -> None:
        pass

    def push(self) -> None:
        if self.world > 1:
            dist.all_reduce(self.gflat, group=self.group)
        if self.master is not None:
            self.master.add_(self.gflat.float(), alpha=-self.lr / self.world)
            self.flat.copy_(self.master)
        else:
            self.flat.add_(self.gflat, alpha=-self.lr / self.world)


def random_token_batches(vocab: int, batch: int, seq: int, device, seed: int):
    """Synthetic data: uniform random token ids; the target is the next token of the same random stream."""
    g = torch.Generator(device=device).manual_seed(seed)
    while True:
        x = torch.randint(0, vocab, (batch, seq + 1), generator=g, device=device)
        yield x[:, :-1].contiguous(), x[:, 1:].contiguous()


def structured_token_batches(vocab: int, batch: int, seq: int, device, seed: int, period: int = 7, active: int = 512):
    """Learnable synthetic data: token t+1 = (token t + step) mod m with a per-sequence step in 1..period, so a
    model has to look at the previous two tokens; m = min(vocab, active), so that a large vocabulary first has to
    be narrowed down to the tokens that occur (a loss of ln m) and the arithmetic comes on top.  Used to compare async
    and sync loss curves on something that can actually be learnt (uniform-random tokens cannot)."""
    g = torch.Generator(device=device).manual_seed(seed)
    ar = torch.arange(seq + 1, device=device)
    m = min(vocab, active)
    while True:
        start = torch.randint(0, m, (batch, 1), generator=g, device=device)
        step = torch.randint(1, period + 1, (batch, 1), generator=g, device=device)
        x = (start + step * ar) % m
        yield x[:, :-1].contiguous(), x[:, 1:].contiguous()
