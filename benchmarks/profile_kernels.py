#!/usr/bin/env python
"""Runs every hot kernel a few times on a small case (arrays larger than L2) so that a profiler can capture them,
and prints CUDA-event timings of the same launches.

    python benchmarks/profile_kernels.py [--elements 33554432] [--links 1 | --mesh 8] [--bits 8] [--shape 0]
    ncu --set full --clock-control none -k regex:round_kernel -s 2 -c 1 -o out python benchmarks/profile_kernels.py

Kernels, in launch order after the warm-up iterations: add (addFromTensor), sub_add (pushUpdate), snapshot fp32,
snapshot bf16, add_scaled_bf16, table_scales (3 kernels), and the round kernel on the hub of a star of `links`
edges, or on member 0 of a fully connected group of `mesh` members (one link, mesh-1 rings in, mesh-1 rings out:
the shape the headline benchmark runs).  All replicas live on one GPU and are wired to each other in-process;
the timed round both receives a frame on every ring and sends one.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from sharedtensor_b200 import _native  # noqa: E402
from sharedtensor_b200.parallel.local_wiring import connect_local, connect_mesh  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=int, default=32 * 1024 * 1024)
    ap.add_argument("--links", type=int, default=1)
    ap.add_argument("--mesh", type=int, default=0, help="members of a fully connected group instead of a star")
    ap.add_argument("--bits", type=int, default=8)
    ap.add_argument("--block", type=int, default=32)
    ap.add_argument("--shape", type=int, default=-1, help="CTA make-up of the round kernel (default: the library's)")
    ap.add_argument("--chunk", type=int, default=0)
    ap.add_argument("--ctas", type=int, default=0, help="CTAs of the round kernel (0: one per SM)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--only-round", action="store_true")
    ap.add_argument("--hub-quiet", action="store_true",
                    help="the hub makes no update of its own: its tiles carry no change mark, so a pass only receives")
    ap.add_argument("--hub-mode", default="both", choices=["both", "rx", "tx"],
                    help="what the timed round does: receive and send, receive only, send only")
    args = ap.parse_args()
    cu = _native.cuda()
    n = args.elements
    s = torch.cuda.current_stream().cuda_stream
    cfg = cu.GpuConfig()
    cfg.bits = args.bits
    cfg.block = args.block
    cfg.ring_slots = 2
    if args.shape >= 0:
        cfg.shape = args.shape
    cfg.chunk_tiles = args.chunk
    cfg.comm_ctas = args.ctas
    hub = cu.GpuReplica(0, n, cfg)
    if args.mesh:
        others = [cu.GpuReplica(0, n, cfg) for _ in range(args.mesh - 1)]
        connect_mesh([hub] + others)
        n_rings = args.mesh - 1
        n_links = 1
    else:
        others = [cu.GpuReplica(0, n, cfg) for _ in range(args.links)]
        for leaf in others:
            connect_local(hub, leaf)
        n_rings = args.links
        n_links = args.links
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
    if args.mesh:
        for r in [hub] + others:
            r.load_values(init.data_ptr(), s)
            r.copy_mirror_from_values(0)
    torch.cuda.synchronize()
    ext = torch.cuda.ExternalStream(hub.comm_stream())
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
        if not args.only_round:
            timed("add", lambda: hub.add(d.data_ptr(), s))
            timed("sub_add", lambda: hub.sub_add(new.data_ptr(), old.data_ptr(), s))
            timed("snapshot_f32", lambda: hub.snapshot(out.data_ptr(), s))
            timed("snapshot_bf16", lambda: hub.snapshot_bf16(out16.data_ptr(), s))
            timed("add_scaled_bf16", lambda: hub.add_scaled_bf16(g16.data_ptr(), -1e-3, s))
            timed("table_scales", lambda: cu.table_scales(hub.values_ptr(), offs.data_ptr(), 3, n, scratch.data_ptr(), sums.data_ptr(),
                                                          exps.data_ptr(), s))
        elif not args.hub_quiet:
            hub.add(d.data_ptr(), s)
        for leaf in others:  # the others have something to say to the hub as well
            leaf.add(d.data_ptr(), s)
            torch.cuda.synchronize()
            leaf.round()
            leaf.sync()
        torch.cuda.synchronize()
        timed("round(hub)", lambda: hub.round(args.hub_mode != "tx", args.hub_mode != "rx"), ext)
    med = {k: sorted(v)[len(v) // 2] for k, v in times.items()}
    pb = args.bits * 512 + max(16, 4096 // args.block)
    # values read and written back (the reduce-add of what arrived), every mirror read and written, the frames read; the
    # frames written go to the peers' memory (here, with every replica on one GPU, they land in this GPU's memory too and
    # are not counted)
    round_bytes = 8 * n + 8 * n_links * n + n_rings * (n // 4096) * pb
    alg = {"add": 12 * n, "sub_add": 16 * n, "snapshot_f32": 8 * n, "snapshot_bf16": 6 * n, "add_scaled_bf16": 10 * n,
           "table_scales": 4 * n, "round(hub)": round_bytes}
    peaks_file = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_file.read_text())["hbm_gbs"] if peaks_file.exists() else 6650.0
    rep = {k: {"ms": round(v, 4), "algorithmic_GBs": round(alg[k] / v / 1e6, 1), "frac_of_measured_hbm": round(alg[k] / v / 1e6 / hbm, 3)}
           for k, v in med.items()}
    print(json.dumps({"elements": n, "links": n_links, "rings": n_rings, "mesh": args.mesh, "bits": args.bits, "shape": cfg.shape,
                      "kernels": rep, "hub_status": dict(zip(cu.status_names(), hub.status()[:12]))}))


if __name__ == "__main__":
    main()
