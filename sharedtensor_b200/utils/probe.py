"""Replica-convergence latency on device clocks.

One rank (the origin) adds an update and stamps its GPU's ``%globaltimer`` behind the add; every rank runs a probe
kernel over a sample of its replica until the squared error against the expected values is within tolerance, and
that kernel stamps its own GPU's clock the first time it is.  The clocks of different GPUs are related through the
host's monotonic clock, which all ranks of one machine share: a one-thread kernel is bracketed by two host clock
reads, and the launch with the tightest bracket gives ``gpu clock - host clock`` to within half the bracket.
(The reference has no notion of time at all; it never reports when an update has arrived.)
"""
from __future__ import annotations

import time

import torch


class ConvergenceProbe:
    def __init__(self, cu, device: torch.device):
        self.cu = cu
        self.dev = device
        self.stamps = torch.zeros(4, dtype=torch.int64, device=device)      # [0] converged at, [1] origin's add landed at
        self.stamps_host = torch.zeros(4, dtype=torch.int64).pin_memory()
        self.scratch = torch.zeros(2, dtype=torch.float64, device=device)
        self.err = torch.zeros(1, dtype=torch.float64, device=device)
        self.offset_ns = 0.0
        self.bracket_ns = 0.0
        self.launches = 0

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.dev).cuda_stream

    def calibrate(self, tries: int = 200) -> tuple[float, float]:
        """Measures ``gpu clock - host monotonic clock`` for this rank's GPU; returns (offset, bracket width) in ns."""
        best = None
        for _ in range(tries):
            torch.cuda.synchronize(self.dev)
            t0 = time.monotonic_ns()
            self.cu.stamp(self.stamps.data_ptr(), self._stream())
            torch.cuda.synchronize(self.dev)
            t1 = time.monotonic_ns()
            self.stamps_host.copy_(self.stamps)
            if best is None or t1 - t0 < best[1]:
                best = (int(self.stamps_host[0]) - (t0 + t1) / 2.0, float(t1 - t0))
        self.offset_ns, self.bracket_ns = best
        return best

    def arm(self) -> None:
        self.stamps.zero_()

    def stamp_origin(self) -> None:
        """Call on the origin right after its ``addFromTensor``, on the same stream."""
        self.cu.stamp(self.stamps.data_ptr() + 8, self._stream())

    def wait(self, values_ptr: int, stride: int, expect: torch.Tensor, threshold: float, timeout_s: float = 5.0) -> tuple[float, float]:
        """Polls until the sampled squared error is at most `threshold`.  Returns (time of convergence, time the
        origin's add landed or 0), both in ns on the host's clock (inf if the wait ran out)."""
        t0 = time.perf_counter()
        s = self._stream()
        while True:
            for _ in range(4):
                self.cu.probe_converged(values_ptr, stride, expect.data_ptr(), expect.numel(), threshold, self.scratch.data_ptr(),
                                        self.stamps.data_ptr(), self.err.data_ptr(), s)
            self.launches += 4
            self.stamps_host.copy_(self.stamps, non_blocking=True)
            torch.cuda.synchronize(self.dev)
            if int(self.stamps_host[0]) != 0 or time.perf_counter() - t0 > timeout_s:
                break
        conv = float(self.stamps_host[0]) - self.offset_ns if int(self.stamps_host[0]) != 0 else float("inf")
        landed = float(self.stamps_host[1]) - self.offset_ns if int(self.stamps_host[1]) != 0 else 0.0
        return conv, landed
