#!/usr/bin/env python
"""Baseline B: synchronous data parallelism by NCCL all-reduce of the uncompressed fp32 delta.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \
        baseline/nccl_allreduce.py [--elements 100000000] [--steps 50]

Same workload as bench.py (every rank produces one N(0,1e-3) delta per step at a 0.5-2 ms cadence), but the ranks
advance in lock step: delta -> all-reduce(sum) -> replica += sum.  One step applies `world` updates to every replica
exactly.  Prints one JSON line with updates/s and the all-reduce bus bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=int, default=100_000_000)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from sharedtensor_b200 import _native

    cu = _native.cuda()
    n = args.elements
    g = torch.Generator(device=dev).manual_seed(7)
    replica = torch.randn(n, generator=g, device=dev)
    g.manual_seed(1000 + rank)
    delta = torch.randn(n, generator=g, device=dev) * 1e-3
    buf = torch.empty_like(delta)
    rng = torch.Generator().manual_seed(99 + rank)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        u = float(torch.rand(1, generator=rng))
        cu.delay(int((0.5 + 1.5 * u) * 1e6), stream)
        buf.copy_(delta)
        if world > 1:
            dist.all_reduce(buf)
        replica.add_(buf)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    secs = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
    if world > 1:
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
    # all-reduce alone, for the bus bandwidth
    ar_ms = None
    if world > 1:
        ts = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dist.all_reduce(buf)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ar_ms = float(t)
    if rank == 0:
        s = float(secs)
        out = {"baseline": "nccl fp32 all-reduce", "n_gpus": world, "elements": n, "steps": args.steps,
               "updates_per_s": world * args.steps / s, "ms_per_step": s * 1e3 / args.steps, "allreduce_ms": ar_ms,
               "allreduce_busbw_GBs": (4 * n * 2 * (world - 1) / world / (ar_ms * 1e-3) / 1e9) if ar_ms else None}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
