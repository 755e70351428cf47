"""Public API: ``createOrFetch``, ``SharedTensor``.

Mirrors the reference's Lua module (src/sharedtensor.c:346-477): ``createOrFetch(host, port, tensor)``
returns an object with ``copyToTensor`` and ``addFromTensor``.  Additions: ``pushUpdate(new, old)``
(the fused ``addFromTensor(new - old)`` of the README's training loop), ``stats``, ``flush``,
``state_dict`` / ``load_state_dict`` and an explicit ``close`` (the reference kills the process when
a connected tensor is garbage collected, 421-430).
"""
from __future__ import annotations

import logging
from typing import Any

import torch

from .utils.config import Config

log = logging.getLogger("sharedtensor")


class _Range:
    """An NVTX range around an API call (``Config.nvtx`` / ``SHAREDTENSOR_NVTX=1``), so that a timeline shows where
    the training loop talks to the shared tensor.  Costs nothing when switched off."""

    __slots__ = ("on",)

    def __init__(self, on: bool, name: str):
        self.on = on and torch.cuda.is_available()
        if self.on:
            torch.cuda.nvtx.range_push(name)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()
        return False


def _check(t: torch.Tensor, n: int, device: torch.device, what: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what}: expected a torch.Tensor, got {type(t).__name__}")
    if t.dtype != torch.float32:
        raise TypeError(f"{what}: expected torch.float32, got {t.dtype}")
    if t.numel() != n:
        raise ValueError("Not the right size!")  # the reference's message, src/sharedtensor.c:335
    if t.device.type != device.type or (device.type == "cuda" and t.device.index != device.index):
        raise ValueError(f"{what}: tensor lives on {t.device}, the shared tensor on {device}")
    if not t.is_contiguous():
        raise ValueError(f"{what}: tensor must be contiguous")
    return t


class SharedTensor:
    """One replica of a shared flat fp32 vector.  Create it with :func:`createOrFetch`."""

    def __init__(self, backend: Any, n: int, shape: torch.Size, cfg: Config):
        self._b = backend
        self._n = n
        self._shape = shape
        self.cfg = cfg
        self._closed = False

    # --- reference API ---------------------------------------------------------------------
    def copyToTensor(self, t: torch.Tensor) -> torch.Tensor:
        """``t <- values`` (src/sharedtensor.c:435-446).  Per-element consistent snapshot."""
        with _Range(self.cfg.nvtx, "sharedtensor.copyToTensor"):
            self._b.copy_to(_check(t, self._n, self._b.device, "copyToTensor"))
        return t

    def addFromTensor(self, delta: torch.Tensor) -> None:
        """``values += delta`` locally; the change reaches every other replica asynchronously
        (src/sharedtensor.c:334-344, 448-453)."""
        with _Range(self.cfg.nvtx, "sharedtensor.addFromTensor"):
            self._b.add(_check(delta, self._n, self._b.device, "addFromTensor"))

    # --- additions -------------------------------------------------------------------------
    def pushUpdate(self, new: torch.Tensor, old: torch.Tensor) -> None:
        """``values += new - old`` in one pass (the README's ``addFromTensor(new:csub(current))``)."""
        dev = self._b.device
        with _Range(self.cfg.nvtx, "sharedtensor.pushUpdate"):
            self._b.sub_add(_check(new, self._n, dev, "pushUpdate(new)"), _check(old, self._n, dev, "pushUpdate(old)"))

    def copyToTensorBF16(self, t: torch.Tensor) -> torch.Tensor:
        """``t <- bf16(values)`` in one pass (GPU replicas; bf16 compute over fp32 master weights)."""
        if t.dtype != torch.bfloat16 or t.numel() != self._n or not t.is_contiguous():
            raise ValueError("copyToTensorBF16 needs a contiguous bfloat16 tensor of the shared size")
        if hasattr(self._b, "copy_to_bf16"):
            self._b.copy_to_bf16(t)
        else:
            tmp = torch.empty(self._n, dtype=torch.float32, device=self._b.device)
            self._b.copy_to(tmp)
            t.copy_(tmp)
        return t

    def addScaledBF16(self, g: torch.Tensor, alpha: float) -> None:
        """``values += alpha * g`` for a bfloat16 ``g`` (an SGD step on bf16 gradients fused with the add)."""
        if g.dtype != torch.bfloat16 or g.numel() != self._n or not g.is_contiguous():
            raise ValueError("addScaledBF16 needs a contiguous bfloat16 tensor of the shared size")
        if hasattr(self._b, "add_scaled_bf16"):
            self._b.add_scaled_bf16(g, float(alpha))
        else:
            self._b.add((g.to(torch.float32) * alpha).to(self._b.device))

    def step(self, rounds: int = 1) -> None:
        """Runs ``rounds`` sync rounds now (only needed with ``engine='manual'``)."""
        if hasattr(self._b, "step"):
            self._b.step(rounds)

    def flush(self, timeout: float = 30.0) -> bool:
        """Waits until this replica has nothing left to send and nothing arriving."""
        with _Range(self.cfg.nvtx, "sharedtensor.flush"):
            return self._b.flush(timeout)

    def stats(self) -> dict:
        s = self._b.stats()
        s["config"] = self.cfg.asdict()
        return s

    def events(self) -> list:
        """Membership events of this replica, oldest first (CPU replicas: joined, master, adopted, edge_lost, rejoined,
        took_over; each with a wall-clock time in milliseconds and a detail string)."""
        return list(self._b.stats().get("events", []))

    def trace(self) -> list:
        """Per-round records kept on the device (GPU replicas): when each of the last 64 rounds ended on the GPU's
        clock, how many tiles it had to look at and how many frames had been sent by then."""
        return self._b.trace() if hasattr(self._b, "trace") else []

    def state_dict(self) -> dict:
        """The replica's values as a CPU tensor (see ``utils.checkpoint`` for why mirrors are not part of the state)."""
        return self._b.state_dict()

    def load_state_dict(self, state: dict) -> None:
        """Overwrites the local values; the difference propagates like any other update."""
        v = state["values"].to(dtype=torch.float32).contiguous()
        if v.numel() != self._n:
            raise ValueError("Not the right size!")
        self._b.load_values(v)

    @property
    def is_master(self) -> bool:
        return self._b.is_master()

    @property
    def numel(self) -> int:
        return self._n

    @property
    def shape(self) -> torch.Size:
        return self._shape

    @property
    def device(self) -> torch.device:
        return self._b.device

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self._b.close()

    def __enter__(self) -> "SharedTensor":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


def createOrFetch(host: str, port: int, tensor: torch.Tensor, **options: Any) -> SharedTensor:
    """Connects to the shared tensor served at ``host:port``; if nobody answers, founds it with the
    values of ``tensor`` (src/sharedtensor.c:347-391).  For a joiner only the element count of
    ``tensor`` matters.  Returns once the replica holds the shared state.

    ``options`` are the fields of :class:`sharedtensor_b200.utils.Config`.
    """
    cfg = Config.from_env_and_kwargs(**options)
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("createOrFetch needs a torch.Tensor")
    if tensor.dtype != torch.float32:
        raise TypeError(f"createOrFetch needs a torch.float32 tensor, got {tensor.dtype}")
    n = tensor.numel()
    flat = tensor.detach().contiguous().view(-1)
    on_gpu = flat.is_cuda
    transport = cfg.transport
    if transport == "auto":
        transport = "gpu" if on_gpu else "tcp"
    if transport == "gpu" and not on_gpu:
        raise ValueError("transport='gpu' needs a CUDA tensor")
    if transport == "gpu" and cfg.topology == "mesh":
        from .parallel.gpu_backend import GpuMeshBackend

        backend = GpuMeshBackend(n, cfg, flat.device)
    elif transport == "gpu":
        from .parallel.gpu_backend import GpuBackend

        backend = GpuBackend(n, cfg, flat.device)
    else:
        if on_gpu:
            from .parallel.gpu_backend import GpuTcpBackend

            backend = GpuTcpBackend(n, cfg, flat.device)
        else:
            from .parallel.cpu_backend import CpuBackend

            backend = CpuBackend(n, cfg)
    backend.start(host, int(port), flat)
    st = SharedTensor(backend, n, tensor.shape, cfg)
    if not backend.wait_ready(cfg.ready_timeout_s):
        st.close()
        raise TimeoutError(f"shared tensor at {host}:{port}: state did not arrive within {cfg.ready_timeout_s}s")
    return st
