"""CPU replica backend: host memory, TCP edges, reference wire format.

Thin wrapper over the C++ ``CpuNode``; nothing here touches the data path.
"""
from __future__ import annotations

import torch

from .. import _native
from ..utils.config import Config


def _node_config(cfg: Config):
    core = _native.core()
    nc = core.NodeConfig()
    nc.tcp_block = cfg.tcp_block
    nc.tcp_bits = cfg.tcp_bits
    nc.gate_min_exp = cfg.min_exp
    nc.gate_rel_bits = cfg.rel_bits
    nc.min_scale_abs = cfg.min_scale_abs
    nc.min_scale_rel = cfg.min_scale_rel
    nc.max_frames_per_s = cfg.max_frames_per_s
    nc.idle_keepalive_ms = cfg.idle_keepalive_ms
    nc.listen_backlog = cfg.listen_backlog
    nc.ready_mode = 0 if cfg.ready_mode == "first_frame" else 1
    nc.ready_bits = cfg.ready_bits
    nc.ready_timeout_ms = int(cfg.ready_timeout_s * 1000)
    nc.rejoin = cfg.rejoin
    nc.rejoin_backoff_ms = cfg.rejoin_backoff_ms
    return nc


class CpuBackend:
    device = torch.device("cpu")

    def __init__(self, n: int, cfg: Config):
        self.n = n
        self.cfg = cfg
        self.node = _native.core().CpuNode(n, _node_config(cfg))

    def start(self, host: str, port: int, init: torch.Tensor | None) -> None:
        self.node.start(host, port, init.data_ptr() if init is not None else 0)

    def wait_ready(self, timeout_s: float) -> bool:
        return self.node.wait_ready(int(timeout_s * 1000))

    def add(self, delta: torch.Tensor) -> None:
        self.node.add(delta.data_ptr(), delta.numel())

    def sub_add(self, new: torch.Tensor, old: torch.Tensor) -> None:
        self.node.sub_add(new.data_ptr(), old.data_ptr(), new.numel())

    def copy_to(self, out: torch.Tensor) -> None:
        self.node.copy_to(out.data_ptr(), out.numel())

    def flush(self, timeout_s: float) -> bool:
        return self.node.flush(int(timeout_s * 1000), 50)

    def stats(self) -> dict:
        s = self.node.stats()
        s["backend"] = "cpu/tcp"
        return s

    def is_master(self) -> bool:
        return self.node.is_master()

    def state_dict(self) -> dict:
        st = self.node.export_state()
        return {k: torch.frombuffer(bytearray(v), dtype=torch.float32).clone() for k, v in st.items()}

    def load_values(self, values: torch.Tensor) -> None:
        self.node.import_values(values.data_ptr(), values.numel())

    def close(self) -> None:
        self.node.close()

    # host-side fault injection used by the tests
    def inject_drop_frames(self, slot: str, k: int) -> None:
        self.node.inject_drop_frames({"up": 0, "left": 1, "right": 2}[slot], k)

    def inject_sever(self, slot: str) -> None:
        self.node.inject_sever({"up": 0, "left": 1, "right": 2}[slot])
