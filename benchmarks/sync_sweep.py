#!/usr/bin/env python
"""Sync bandwidth / latency sweep over tensor sizes (1 Ki .. 1 Gi fp32 elements, powers of 4).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29500 \
        benchmarks/sync_sweep.py [--max-log4 15] [--out sweep.json]

For every size and the N ranks of one box it measures, with deltas ~ N(0,1):
  * the compressed path of this framework: device time of one sync round under load (max over ranks), the
    HBM bytes that round moves per rank and the packed bytes it puts on each edge, and the time until one
    update has reached every replica to 1 % (engine free-running), taken from GPU clock stamps: the origin's
    behind its add, every replica's when its probe kernel first finds the error within tolerance;
  * the baseline: an NCCL all-reduce of the uncompressed fp32 delta followed by the local add.
It prints one JSON object per size on rank 0 and a summary table at the end.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import sharedtensor  # noqa: E402
from sharedtensor_b200 import _native  # noqa: E402

TOL = 1e-2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-log4", type=int, default=5)    # 4^5 = 1 Ki
    ap.add_argument("--max-log4", type=int, default=15)   # 4^15 = 1 Gi
    ap.add_argument("--probes", type=int, default=24)
    ap.add_argument("--topology", default="tree", choices=["tree", "mesh"])
    ap.add_argument("--bits", type=int, default=0, help="bits per element of a frame (0: the library's default)")
    ap.add_argument("--rounds", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cu = _native.cuda()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nccl = dist.new_group(backend="nccl") if world > 1 else None
    stream = torch.cuda.current_stream().cuda_stream
    base_port = int(os.environ.get("MASTER_PORT", "29500")) + 100
    peaks = {}
    pk = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm = peaks.get("hbm_gbs", 6650.0)

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()

    def allmax(x):
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    from sharedtensor_b200.utils.probe import ConvergenceProbe
    probe = ConvergenceProbe(cu, dev)
    probe.calibrate()
    kw = {"bits": args.bits} if args.bits else {}
    rows = []
    for i, k in enumerate(range(args.min_log4, args.max_log4 + 1)):
        n = 4 ** k
        g = torch.Generator(device=dev).manual_seed(5)
        init = torch.randn(n, generator=g, device=dev)
        deltas = []
        for r in range(world):
            g.manual_seed(100 + r)
            deltas.append(torch.randn(n, generator=g, device=dev))
        # ---- our path
        st = None
        if args.topology == "mesh":
            st = sharedtensor.createOrFetch("127.0.0.1", base_port + i, init if rank == 0 else torch.empty(n, device=dev),
                                            topology="mesh", group_rank=rank, group_size=world, **kw)
            barrier()
        else:
            for r in range(world):
                if r == rank:
                    st = sharedtensor.createOrFetch("127.0.0.1", base_port + i, init if rank == 0 else torch.empty(n, device=dev), **kw)
                barrier()
        rep = st._b.rep
        out = torch.empty(n, device=dev)
        stride = max(1, n >> 17)               # the probe looks at up to 128 Ki elements: a heavier one slows the kernels it watches
        expect_s = init[::stride].clone()
        lat = []
        for pr in range(args.probes + 2):
            origin = pr % world
            expect_s += deltas[origin][::stride]
            thr = float((deltas[origin][::stride].double() ** 2).sum()) * TOL * TOL
            probe.arm()
            barrier()
            if rank == origin:
                st.addFromTensor(deltas[origin])
                probe.stamp_origin()
            t_conv, t_landed = probe.wait(rep.values_ptr(), stride, expect_s, thr, timeout_s=10.0)
            t_add = allmax(t_landed if rank == origin else -1e30)
            if pr >= 2:                           # the first two probes warm the path up
                lat.append(allmax(t_conv - t_add) / 1e9)
        # device time of a round under load: stop the engine thread and drive rounds by hand
        rep.stop_engine()
        barrier()
        cs = torch.cuda.ExternalStream(rep.comm_stream())
        times = []
        for j in range(args.rounds):
            rep.add(deltas[rank].data_ptr(), rep.comm_stream())
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(cs)
            rep.round()
            e1.record(cs)
            rep.sync()
            times.append(e0.elapsed_time(e1))
            if j % 4 == 3:
                barrier()
        times = sorted(times[3:])
        round_ms = allmax(times[len(times) // 2])
        links = 1 if args.topology == "mesh" else sum(1 for e in st.stats()["edges"].values() if e["state"] == "connected")
        max_links = int(allmax(float(links)))
        barrier()
        st.close()
        barrier()
        # ---- baseline: NCCL all-reduce of the fp32 delta + local add
        ar_ms = None
        if nccl is not None:
            buf = deltas[rank].clone()
            for _ in range(3):
                dist.all_reduce(buf, group=nccl)
            torch.cuda.synchronize()
            ts = []
            for _ in range(10):
                buf.copy_(deltas[rank])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                dist.all_reduce(buf, group=nccl)
                out.add_(buf)
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ar_ms = allmax(sorted(ts)[len(ts) // 2])
        lat_ms = sorted(x * 1e3 for x in lat)
        bits = st.cfg.bits
        hbm_bytes = (8 + 8 * max_links) * n  # values + one mirror per link, read and written
        edge_bytes = n * bits / 8 + n / 32   # one frame with block-32 scales per round and edge direction
        row = {"elements": n, "n_gpus": world, "topology": args.topology, "frame_bits": bits, "round_ms": round_ms, "links_max": max_links,
               "round_hbm_GBs": hbm_bytes / round_ms / 1e6, "round_hbm_frac_of_measured": hbm_bytes / round_ms / 1e6 / hbm,
               "edge_bytes_per_round": edge_bytes, "edge_GBs": edge_bytes / round_ms / 1e6,
               "nvlink_roofline_ms": edge_bytes / 770e9 * 1e3, "hbm_roofline_ms": hbm_bytes / (hbm * 1e9) * 1e3,
               "latency_ms_p50": lat_ms[len(lat_ms) // 2], "latency_ms_max": lat_ms[-1], "latency_probes": len(lat_ms),
               "latency_clock": "GPU clock stamps related through the host's monotonic clock",
               "nccl_allreduce_add_ms": ar_ms}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        del init, deltas, expect_s, out
        torch.cuda.empty_cache()
    if rank == 0 and args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
