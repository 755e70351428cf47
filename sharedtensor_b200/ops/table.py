"""Table sync: a set of named tensors shared as one flat arena, each with its own magnitude.

The reference lists this as a TODO ("Support 'table sync' so that a table of tensors all get synched, but
tensors can have different magnitudes", README.md:41).  Here every tensor starts on a scale-block boundary of the
arena, so no quantiser block ever mixes two tensors and each tensor is effectively scaled on its own; a
segmented reduction kernel reports per-tensor energies and RMS exponents.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..api import SharedTensor, createOrFetch


class TableLayout:
    """Offsets of named tensors inside a flat fp32 arena; every tensor starts on a multiple of ``align``."""

    def __init__(self, shapes: Mapping[str, torch.Size], align: int):
        self.align = align
        self.names = list(shapes)
        self.shapes = {k: torch.Size(v) for k, v in shapes.items()}
        self.offsets: dict[str, int] = {}
        off = 0
        for k in self.names:
            self.offsets[k] = off
            n = self.shapes[k].numel()
            off += (n + align - 1) // align * align
        self.numel = max(off, 1)

    def views(self, flat: torch.Tensor) -> dict[str, torch.Tensor]:
        return {k: flat[self.offsets[k]: self.offsets[k] + self.shapes[k].numel()].view(self.shapes[k]) for k in self.names}

    def pack(self, tensors: Mapping[str, torch.Tensor], out: torch.Tensor | None = None) -> torch.Tensor:
        first = next(iter(tensors.values()))
        flat = out if out is not None else torch.zeros(self.numel, dtype=torch.float32, device=first.device)
        for k, v in self.views(flat).items():
            v.copy_(tensors[k])
        return flat

    def segment_offsets(self) -> list[int]:
        """n_seg + 1 boundaries of the padded segments (a segment's padding belongs to it and is zero)."""
        return [self.offsets[k] for k in self.names] + [self.numel]


class SharedTable:
    """A table of tensors kept in sync as one shared arena.  Create it with :func:`createOrFetchTable`."""

    def __init__(self, shared: SharedTensor, layout: TableLayout):
        self.shared = shared
        self.layout = layout
        self._scratch: torch.Tensor | None = None

    # ---- dict-of-tensors interface
    def copyToTensors(self, out: Mapping[str, torch.Tensor]) -> None:
        flat = self._flat()
        self.shared.copyToTensor(flat)
        for k, v in self.layout.views(flat).items():
            out[k].copy_(v)

    def addFromTensors(self, deltas: Mapping[str, torch.Tensor]) -> None:
        flat = self._flat()
        flat.zero_()
        self.layout.pack(deltas, flat)
        self.shared.addFromTensor(flat)

    # ---- flat interface (no packing: keep parameters as views of one arena, see ``views``)
    def new_flat(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return torch.zeros(self.layout.numel, dtype=dtype, device=self.shared.device)

    def views(self, flat: torch.Tensor) -> dict[str, torch.Tensor]:
        return self.layout.views(flat)

    def copyToFlat(self, flat: torch.Tensor) -> torch.Tensor:
        return self.shared.copyToTensor(flat)

    def copyToFlatBF16(self, flat: torch.Tensor) -> torch.Tensor:
        return self.shared.copyToTensorBF16(flat)

    def addFromFlat(self, flat: torch.Tensor) -> None:
        self.shared.addFromTensor(flat)

    def pushUpdateFlat(self, new: torch.Tensor, old: torch.Tensor) -> None:
        self.shared.pushUpdate(new, old)

    # ---- per-tensor magnitudes
    def scales(self, flat: torch.Tensor | None = None) -> dict[str, dict]:
        """Per-tensor sum of squares and floor(log2(rms)) of the current values (or of ``flat``)."""
        src = flat
        if src is None:
            src = self._flat()
            self.shared.copyToTensor(src)
        offs = self.layout.segment_offsets()
        n_seg = len(self.layout.names)
        if src.is_cuda:
            from .. import _native

            cu = _native.cuda()
            dev = src.device
            off_d = torch.tensor(offs, dtype=torch.int64, device=dev)
            scratch = torch.empty(cu.table_scales_scratch_doubles(n_seg, self.layout.numel), dtype=torch.float64, device=dev)
            sums = torch.empty(n_seg, dtype=torch.float64, device=dev)
            exps = torch.empty(n_seg, dtype=torch.int8, device=dev)
            cu.table_scales(src.data_ptr(), off_d.data_ptr(), n_seg, self.layout.numel, scratch.data_ptr(), sums.data_ptr(),
                            exps.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
            sums_l, exps_l = sums.cpu().tolist(), exps.cpu().tolist()
        else:
            import math

            from .. import _native

            sums_l = _native.core().segment_sumsq(src.data_ptr(), offs)
            exps_l = []
            for k, s in zip(self.layout.names, sums_l):
                cnt = offs[self.layout.names.index(k) + 1] - self.layout.offsets[k]
                exps_l.append(math.floor(math.log2(math.sqrt(s / cnt))) if s > 0 and cnt else -128)
        return {k: {"sumsq": s, "rms_exp": e} for k, s, e in zip(self.layout.names, sums_l, exps_l)}

    def _flat(self) -> torch.Tensor:
        if self._scratch is None:
            self._scratch = self.new_flat()
        return self._scratch

    def stats(self) -> dict:
        return self.shared.stats()

    def flush(self, timeout: float = 30.0) -> bool:
        return self.shared.flush(timeout)

    def close(self) -> None:
        self.shared.close()


def createOrFetchTable(host: str, port: int, tensors: Mapping[str, torch.Tensor], **options) -> SharedTable:
    """Like :func:`createOrFetch` for a dict of fp32 tensors.  Peers must pass the same names and shapes in the same
    order (like the reference, nothing about the layout travels over the wire)."""
    from ..utils.config import Config

    cfg = Config.from_env_and_kwargs(**options)
    first = next(iter(tensors.values()))
    on_gpu = first.is_cuda
    if not on_gpu and "tcp_scale_mode" not in options:
        options["tcp_scale_mode"] = "block32"  # one scale for the whole arena would mix the tensors' magnitudes
        cfg = Config.from_env_and_kwargs(**options)
    align = cfg.block if on_gpu else max(cfg.tcp_block, 32)
    layout = TableLayout({k: v.shape for k, v in tensors.items()}, align)
    flat = layout.pack(tensors)
    shared = createOrFetch(host, port, flat, **options)
    return SharedTable(shared, layout)
