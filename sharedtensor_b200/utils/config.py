"""Configuration of a shared tensor.

The reference has no configuration beyond the three arguments of ``createOrFetch`` and a handful of
hard-coded constants (listen backlog 5 at src/sharedtensor.c:323, a one-second idle sleep at 163,
fan-out 2 in the struct at 31-33, the scale rule at 158-159).  Here every such constant is a field
of one dataclass, validated once, overridable per call (keyword arguments of ``createOrFetch``) and
per process (``SHAREDTENSOR_<FIELD>`` environment variables), and echoed back by ``stats()``.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass
from typing import Any

_TRUE = {"1", "true", "yes", "on"}


@dataclass
class Config:
    # --- where the replica lives and how edges are carried -------------------------------------
    transport: str = "auto"          # auto | gpu | tcp   (auto: gpu for CUDA tensors, tcp for CPU tensors)
    topology: str = "tree"           # tree (reference semantics, dynamic join) | mesh (fixed group over NVSwitch)
    group_rank: int = -1             # mesh only: this member's rank (default: $RANK)
    group_size: int = 0              # mesh only: number of members (default: $WORLD_SIZE)
    # --- quantiser ------------------------------------------------------------------------------
    scale_mode: str = "block32"      # GPU edges: block32 .. block4096
    tcp_scale_mode: str = "tensor"   # TCP edges: tensor (reference wire format) | block32 .. block4096
    tcp_bits: int = 1                # TCP edges of CPU tensors in a block mode: 1 (sign frames) | 8 (one frame delivers an update to < 1 %)
    min_exp: int = -60               # blocks whose scale exponent is below this stay silent
    rel_bits: int = 22               # ... or this many bits below the block's own value RMS
    min_scale_abs: float = 0.0       # tensor mode cut-offs
    min_scale_rel: float = 2.0 ** -22
    # --- GPU engine -----------------------------------------------------------------------------
    ring_slots: int = 4              # frames in flight per edge direction
    bits: int = 8                    # bits per element of a GPU frame: 1 (sign frames, the reference's) | 2 | 4 | 8
    sweeps_per_launch: int = 0       # passes over the tensor per launch of the round kernel (0: one; more saves launches but delays a fresh update)
    engine: str = "thread"           # thread: free-running rounds on a comm stream | manual: caller drives step()
    comm_ctas: int = 0               # CTAs of the round kernel (0 = one per SM)
    rounds_in_flight: int = 2        # how far the engine thread runs ahead of the GPU
    idle_sleep_us: int = 1000        # longest engine pause while nothing moves (backs off from 10 us; doorbells end it)
    round_interval_us: int = 0       # pause after every busy round: caps the round rate (a rate limit for GPU edges)
    poll_deadline_us: int = 1000     # upper bound of every wait inside the round kernel
    yield_to_updates: bool = True    # a running round kernel gives up its SMs when addFromTensor has an update ready
    comm_high_priority: bool = False # comm stream at the highest stream priority (then rounds do not yield to updates)
    use_multimem: bool = False       # reserved: NVLS store fan-out is not built (plain peer stores only)
    nvtx: bool = False               # NVTX ranges around the API calls (copyToTensor, addFromTensor, pushUpdate, flush)
    # --- TCP edges ------------------------------------------------------------------------------
    max_frames_per_s: float = 0.0    # rate cap per edge (README.md:31 of the reference lists this as a TODO)
    idle_keepalive_ms: int = 0
    listen_backlog: int = 5
    # --- membership -----------------------------------------------------------------------------
    ready_mode: str = "converged"    # first_frame (reference) | converged
    ready_bits: int = 12
    ready_timeout_s: float = 30.0
    rejoin: bool = True              # re-run the join walk when the up edge is lost
    rejoin_backoff_ms: int = 200

    def __post_init__(self) -> None:
        self.validate()

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _block_of(mode: str) -> int:
        if mode == "tensor":
            return 0
        if not mode.startswith("block"):
            raise ValueError(f"unknown scale mode {mode!r}")
        b = int(mode[5:])
        if b < 32 or b > 4096 or b & (b - 1):
            raise ValueError(f"block size must be a power of two in 32..4096, got {b}")
        return b

    @property
    def block(self) -> int:
        return self._block_of(self.scale_mode)

    @property
    def tcp_block(self) -> int:
        return self._block_of(self.tcp_scale_mode)

    def validate(self) -> None:
        if self.transport not in ("auto", "gpu", "tcp"):
            raise ValueError(f"transport must be auto, gpu or tcp, got {self.transport!r}")
        if self.topology not in ("tree", "mesh"):
            raise ValueError(f"topology must be tree or mesh, got {self.topology!r}")
        if self.block == 0:
            raise ValueError("GPU edges need a block scale mode (block32..block4096)")
        self.tcp_block  # validates
        if self.tcp_bits not in (1, 8):
            raise ValueError("tcp_bits must be 1 or 8")
        if self.tcp_bits == 8 and self.tcp_block == 0:
            raise ValueError("tcp_bits=8 needs tcp_scale_mode block32..block4096 (the tensor mode is the reference's wire format)")
        if self.engine not in ("thread", "manual"):
            raise ValueError(f"engine must be thread or manual, got {self.engine!r}")
        if self.ready_mode not in ("first_frame", "converged"):
            raise ValueError(f"ready_mode must be first_frame or converged, got {self.ready_mode!r}")
        if not 2 <= self.ring_slots <= 64 or self.ring_slots & (self.ring_slots - 1):
            raise ValueError("ring_slots must be a power of two in 2..64")
        if self.rel_bits < 1 or self.rel_bits > 60:
            raise ValueError("rel_bits must be in 1..60")
        if self.use_multimem:
            raise ValueError("use_multimem: the NVLS store path is not built; leave it False")
        if self.bits not in (1, 2, 4, 8):
            raise ValueError("bits must be 1, 2, 4 or 8")
        if not 0 <= self.sweeps_per_launch <= 64:
            raise ValueError("sweeps_per_launch must be in 0..64")
        if not 1 <= self.poll_deadline_us <= 2_000_000:
            raise ValueError("poll_deadline_us must be in 1..2000000")
        if self.rounds_in_flight < 1:
            raise ValueError("rounds_in_flight must be >= 1")

    # ------------------------------------------------------------------------------------------
    @classmethod
    def from_env_and_kwargs(cls, **kwargs: Any) -> "Config":
        values: dict[str, Any] = {}
        for f in dataclasses.fields(cls):
            env = os.environ.get("SHAREDTENSOR_" + f.name.upper())
            if env is None:
                continue
            if f.type in ("bool", bool):
                values[f.name] = env.strip().lower() in _TRUE
            elif f.type in ("int", int):
                values[f.name] = int(env)
            elif f.type in ("float", float):
                values[f.name] = float(env)
            else:
                values[f.name] = env
        unknown = set(kwargs) - {f.name for f in dataclasses.fields(cls)}
        if unknown:
            raise TypeError(f"unknown shared tensor option(s): {sorted(unknown)}")
        values.update(kwargs)
        return cls(**values)

    def asdict(self) -> dict[str, Any]:
        return dataclasses.asdict(self)
