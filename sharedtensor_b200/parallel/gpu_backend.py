"""GPU replica backend: device-resident values, peer-memory rings to same-host neighbours.

Thin wrapper over the C++ ``GpuNode`` (membership + upgrade to peer memory) and ``GpuReplica`` (kernels,
engine thread).  Nothing here touches the data path.
"""
from __future__ import annotations

import struct

import torch

from .. import _native
from ..utils.config import Config

_SLOTS = {"up": 0, "left": 1, "right": 2}


def _gpu_config(cfg: Config):
    cu = _native.cuda()
    g = cu.GpuConfig()
    g.block = cfg.block
    g.ring_slots = cfg.ring_slots
    g.min_exp = cfg.min_exp
    g.rel_bits = cfg.rel_bits
    g.comm_ctas = cfg.comm_ctas
    g.shareable = True
    g.rounds_in_flight = cfg.rounds_in_flight
    g.idle_sleep_us = cfg.idle_sleep_us
    g.round_interval_us = cfg.round_interval_us
    g.bits = cfg.bits
    g.sweeps = cfg.sweeps_per_launch
    g.poll_deadline_us = cfg.poll_deadline_us
    g.yield_to_updates = cfg.yield_to_updates
    g.comm_high_priority = cfg.comm_high_priority
    return g


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class GpuBackend:
    def __init__(self, n: int, cfg: Config, device: torch.device):
        if not torch.cuda.is_available():
            raise RuntimeError("the GPU transport needs a CUDA device")
        if cfg.tcp_bits != 1:
            raise ValueError("tcp_bits=8 is a frame format of CPU replicas; the TCP edges of a GPU replica speak the reference's frames")
        cu = _native.cuda()
        self.n = n
        self.cfg = cfg
        self.device = torch.device("cuda", device.index if device.index is not None else torch.cuda.current_device())
        opt = cu.GpuNodeOptions()
        opt.rejoin = cfg.rejoin
        opt.rejoin_backoff_ms = cfg.rejoin_backoff_ms
        opt.listen_backlog = cfg.listen_backlog
        opt.start_engine = cfg.engine == "thread"
        self.node = cu.GpuNode(self.device.index, n, _gpu_config(cfg), opt)
        self.rep = self.node.replica()

    def start(self, host: str, port: int, init: torch.Tensor | None) -> None:
        self.node.start(host, port, init.data_ptr() if init is not None else 0, _stream(self.device))

    def wait_ready(self, timeout_s: float) -> bool:
        return self.node.wait_ready(int(timeout_s * 1000))

    def add(self, delta: torch.Tensor) -> None:
        self.rep.add(delta.data_ptr(), _stream(self.device))

    def sub_add(self, new: torch.Tensor, old: torch.Tensor) -> None:
        self.rep.sub_add(new.data_ptr(), old.data_ptr(), _stream(self.device))

    def add_scaled_bf16(self, g: torch.Tensor, alpha: float) -> None:
        self.rep.add_scaled_bf16(g.data_ptr(), alpha, _stream(self.device))

    def copy_to(self, out: torch.Tensor) -> None:
        self.rep.snapshot(out.data_ptr(), _stream(self.device))

    def copy_to_bf16(self, out: torch.Tensor) -> None:
        self.rep.snapshot_bf16(out.data_ptr(), _stream(self.device))

    def step(self, rounds: int = 1) -> None:
        """Runs sync rounds from the caller's thread (``engine='manual'``)."""
        for _ in range(rounds):
            self.rep.round()

    def flush(self, timeout_s: float) -> bool:
        import time

        names = _native.cuda().status_names()
        i_work, i_pend = names.index("last_work_count"), names.index("pending_tiles")
        t0 = time.time()
        quiet = 0
        while time.time() - t0 < timeout_s:
            if not self.rep.engine_running():
                self.rep.round()
            st = self.rep.status()
            if st[i_work] == 0 and st[i_pend] == 0:
                quiet += 1
                if quiet >= 3:
                    return True
            else:
                quiet = 0
            time.sleep(0.0005)
        return False

    def stats(self) -> dict:
        s = self.node.stats()
        s["backend"] = "gpu/p2p"
        return s

    def trace(self) -> list[dict]:
        """The last rounds as recorded on the device: GPU clock (ns), round number, tiles listed, frames sent so far."""
        cu = _native.cuda()
        st = self.rep.status()
        base, ne, nw = cu.STATUS_WORDS, cu.TRACE_ENTRIES, cu.TRACE_WORDS
        recs = [st[base + i * nw: base + (i + 1) * nw] for i in range(ne)]
        recs = [{"gpu_time_ns": r[0], "round": r[1], "tiles": r[2], "frames_sent": r[3]} for r in recs if r[0]]
        return sorted(recs, key=lambda r: r["round"])

    def is_master(self) -> bool:
        return self.node.is_master()

    def state_dict(self) -> dict:
        out = torch.empty(self.n, device=self.device)
        self.copy_to(out)
        torch.cuda.synchronize(self.device)
        return {"values": out.cpu()}

    def load_values(self, values: torch.Tensor) -> None:
        v = values.to(self.device)
        cur = torch.empty(self.n, device=self.device)
        self.copy_to(cur)
        self.sub_add(v, cur)  # the difference propagates like any other update
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        self.node.close()

    def inject_sever(self, slot: str) -> None:
        self.node.inject_sever(_SLOTS[slot])


class GpuMeshBackend(GpuBackend):
    """Fixed, fully connected group of GPU replicas on one host (``topology='mesh'``): one hop, no forwarding."""

    def __init__(self, n: int, cfg: Config, device: torch.device):
        import os

        if not torch.cuda.is_available():
            raise RuntimeError("the GPU transport needs a CUDA device")
        cu = _native.cuda()
        self.n = n
        self.cfg = cfg
        self.device = torch.device("cuda", device.index if device.index is not None else torch.cuda.current_device())
        self.rank = cfg.group_rank if cfg.group_rank >= 0 else int(os.environ.get("RANK", "0"))
        self.world = cfg.group_size if cfg.group_size > 0 else int(os.environ.get("WORLD_SIZE", "1"))
        self.node = cu.GpuMeshNode(self.device.index, n, _gpu_config(cfg), self.rank, self.world, cfg.engine == "thread")
        self.rep = self.node.replica()

    def start(self, host: str, port: int, init: torch.Tensor | None) -> None:
        self.node.start(host, port, init.data_ptr() if (init is not None and self.rank == 0) else 0, _stream(self.device),
                        int(self.cfg.ready_timeout_s * 1000))

    def wait_ready(self, timeout_s: float) -> bool:
        return True  # start() returns once the common initial state is in place

    def is_master(self) -> bool:
        return self.rank == 0

    def stats(self) -> dict:
        names = _native.cuda().status_names()
        st = self.rep.status()
        dev = {k: v for k, v in zip(names, st)}
        for k in dev:  # the residual maxima are kept as float bit patterns (they are updated with an integer max)
            if k.startswith("residual_max"):
                dev[k] = struct.unpack("<f", struct.pack("<I", dev[k] & 0xFFFFFFFF))[0]
        return {"backend": "gpu/p2p-mesh", "master": self.rank == 0, "ready": True, "n": self.n, "rank": self.rank,
                "group_size": self.world, "members_alive": self.node.members_alive(), "dropped": self.node.dropped(),
                "launches": self.rep.launches(), "device": dev, "edges": {}}

    def inject_sever(self, slot: str) -> None:
        raise NotImplementedError("mesh groups have no tree slots")


class GpuTcpBackend:
    """CUDA tensors over TCP edges (cross-host, or below a CPU/reference parent): the replica is kept by
    the CPU node and user tensors are staged through pinned host memory."""

    def __init__(self, n: int, cfg: Config, device: torch.device):
        from .cpu_backend import CpuBackend

        self.n = n
        self.cfg = cfg
        self.device = torch.device("cuda", device.index if device.index is not None else torch.cuda.current_device())
        self.cpu = CpuBackend(n, cfg)
        self.stage = torch.empty(n, dtype=torch.float32).pin_memory()
        self.stage2 = torch.empty(n, dtype=torch.float32).pin_memory()

    def start(self, host, port, init):
        if init is not None:
            self.stage.copy_(init)
        self.cpu.start(host, port, self.stage if init is not None else None)

    def wait_ready(self, t):
        return self.cpu.wait_ready(t)

    def add(self, delta):
        self.stage.copy_(delta)
        self.cpu.add(self.stage)

    def sub_add(self, new, old):
        self.stage.copy_(new)
        self.stage2.copy_(old)
        self.cpu.sub_add(self.stage, self.stage2)

    def copy_to(self, out):
        self.cpu.copy_to(self.stage)
        out.copy_(self.stage)

    def flush(self, t):
        return self.cpu.flush(t)

    def stats(self):
        s = self.cpu.stats()
        s["backend"] = "gpu-staged/tcp"
        return s

    def is_master(self):
        return self.cpu.is_master()

    def state_dict(self):
        return self.cpu.state_dict()

    def load_values(self, v):
        self.cpu.load_values(v.cpu().contiguous())

    def close(self):
        self.cpu.close()
