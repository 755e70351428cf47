#!/usr/bin/env python
"""Runs every hot kernel a few times on a small case (arrays larger than L2, a few hundred MB in total) so that
a profiler can capture them, and prints CUDA-event timings of the same launches.

    python benchmarks/profile_kernels.py [--elements 33554432] [--links 1] [--frames 3]
    ncu --set full --clock-control none -k regex:round_main -s 2 -c 1 -o out python benchmarks/profile_kernels.py

Kernels, in launch order after two warm-up iterations: add (addFromTensor), sub_add (pushUpdate), snapshot fp32,
snapshot bf16, add_scaled_bf16, table_scales (3 kernels), round_begin / round_main / round_publish on the hub
of a star of `links` edges (all replicas on one GPU, wired to each other in-process).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from sharedtensor_b200 import _native  # noqa: E402
from sharedtensor_b200.parallel.local_wiring import connect_local  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=int, default=32 * 1024 * 1024)
    ap.add_argument("--links", type=int, default=1)
    ap.add_argument("--frames", type=int, default=3)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--hub-mode", default="both", choices=["both", "rx", "tx"],
                    help="what the timed hub round does: receive and send, receive only, send only")
    args = ap.parse_args()
    cu = _native.cuda()
    n = args.elements
    s = torch.cuda.current_stream().cuda_stream
    cfg = cu.GpuConfig()
    cfg.frames_per_round = args.frames
    cfg.ring_slots = 8
    hub = cu.GpuReplica(0, n, cfg)
    leaves = [cu.GpuReplica(0, n, cfg) for _ in range(args.links)]
    for leaf in leaves:
        connect_local(hub, leaf)
    init = torch.randn(n, device="cuda")
    d = torch.randn(n, device="cuda") * 1e-3
    new, old = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    out = torch.empty(n, device="cuda")
    out16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    g16 = (torch.randn(n, device="cuda") * 1e-3).to(torch.bfloat16)
    sizes = [n // 8, n // 2, n - n // 8 - n // 2]
    offs = torch.tensor([0, sizes[0], sizes[0] + sizes[1], n], dtype=torch.int64, device="cuda")
    scratch = torch.empty(cu.table_scales_scratch_doubles(3, n), dtype=torch.float64, device="cuda")
    sums = torch.empty(3, dtype=torch.float64, device="cuda")
    exps = torch.empty(3, dtype=torch.int8, device="cuda")
    hub.load_values(init.data_ptr(), s)
    cs = hub.comm_stream()
    ext = torch.cuda.ExternalStream(cs)
    times: dict[str, list] = {}

    def timed(name, fn, stream=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = stream if stream is not None else torch.cuda.current_stream()
        torch.cuda.synchronize()
        e0.record(st)
        fn()
        e1.record(st)
        torch.cuda.synchronize()
        times.setdefault(name, []).append(e0.elapsed_time(e1))

    for it in range(args.iters):
        timed("add", lambda: hub.add(d.data_ptr(), cs), ext)
        timed("sub_add", lambda: hub.sub_add(new.data_ptr(), old.data_ptr(), cs), ext)
        timed("snapshot_f32", lambda: hub.snapshot(out.data_ptr(), s))
        timed("snapshot_bf16", lambda: hub.snapshot_bf16(out16.data_ptr(), s))
        timed("add_scaled_bf16", lambda: hub.add_scaled_bf16(g16.data_ptr(), -1e-3, cs), ext)
        timed("table_scales", lambda: cu.table_scales(hub.values_ptr(), offs.data_ptr(), 3, n, scratch.data_ptr(), sums.data_ptr(),
                                                      exps.data_ptr(), s))
        for leaf in leaves:  # the leaves have something to say to the hub as well
            leaf.add(d.data_ptr(), leaf.comm_stream())
            leaf.round()
            leaf.sync()
        timed("round(hub)", lambda: hub.round(args.hub_mode != "tx", args.hub_mode != "rx"), ext)
    med = {k: sorted(v)[len(v) // 2] for k, v in times.items()}
    alg = {"add": 12 * n, "sub_add": 16 * n, "snapshot_f32": 8 * n, "snapshot_bf16": 6 * n, "add_scaled_bf16": 10 * n,
           "table_scales": 4 * n, "round(hub)": (8 + 8 * args.links) * n}
    peaks_file = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
    rep = {k: {"ms": round(v, 4), "algorithmic_GBs": round(alg[k] / v / 1e6, 1), "frac_of_measured_hbm": round(alg[k] / v / 1e6 / hbm, 3)}
           for k, v in med.items()}
    print(json.dumps({"elements": n, "links": args.links, "frames_per_round": args.frames, "kernels": rep,
                      "hub_status": dict(zip(cu.status_names(), hub.status()[:12]))}))


if __name__ == "__main__":
    main()
