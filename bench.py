#!/usr/bin/env python
"""Headline benchmark: applied updates/s (and replica-convergence latency) of a shared 100M-element fp32
tensor, each rank adding N(0,1e-3) deltas at a randomised 0.5-2 ms cadence.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 50 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference over loopback TCP, same workload

One step of a rank = wait its cadence interval (a device-side delay kernel standing in for the compute
between updates) + ``addFromTensor(delta)``.  The engine propagates in the background.  A timed region
starts after a barrier and ends, on every rank, when its replica holds initial + the sum of ALL ranks'
updates so far to within 1 % (relative L2 of the region's updates, checked on a strided sample of the
replica by a device kernel); its time is the maximum over ranks.  The region of ``--steps`` updates per
rank is run ``--repeats`` times and value = world_size * steps / (median region time).  Rank 0 prints one
JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_ELEMENTS = 100_000_000
INIT_STD, DELTA_STD = 1.0, 1e-3
CADENCE_MS = (0.5, 2.0)
POOL = 4                 # distinct deltas per rank, cycled
SAMPLE_STRIDE = 64       # convergence is decided on every 64th element (the full tensor is compared once at the end)
POLL_EVERY = 16          # ... and polled on every 16th of those: a poll that reads 50 MB beside the sync kernels slows them down
TOL = 1e-2               # "applied": outstanding error below 1 % of the update's norm


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="how often the region of --steps updates is timed (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--elements", type=int, default=N_ELEMENTS)
    ap.add_argument("--probes", type=int, default=200, help="single-update latency probes after the timed regions")
    ap.add_argument("--topology", default="auto", choices=["auto", "tree", "mesh"],
                    help="auto: the fixed fully connected group when the ranks are known up front (N > 1 under "
                         "torch.distributed.run), else the join tree; the other one is measured too and reported under "
                         "other_topology")
    ap.add_argument("--bits", type=int, default=0, help="bits per element of a GPU frame (0: the library's default)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the comparison run on the other topology")
    ap.add_argument("--no-full-check", action="store_true")
    ap.add_argument("--ref-time-cap", type=float, default=120.0, help="wall-clock cap of the reference arm's wait, seconds")
    return ap.parse_args()


def resolve_topology(args, world: int) -> None:
    if args.topology == "auto":
        args.topology = "mesh" if world > 1 else "tree"


def env_rank():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def shared_config(n: int, world: int) -> dict:
    """The part of the record both arms print word for word."""
    return {"model": "shared parameter vector, 100M fp32 elements ~ N(0,1)", "elements": n, "global_batch": world, "seq_len": None,
            "parallelism": f"async-dp{world}", "delta": "N(0,1e-3) fp32", "cadence_ms": list(CADENCE_MS),
            "applied_when": f"rel-L2 of outstanding update <= {TOL} on every replica",
            "l2": "inputs larger than L2 (400 MB per array)"}


def pct(sorted_vals: list, q: float):
    if not sorted_vals:
        return None
    return sorted_vals[min(len(sorted_vals) - 1, int(q * len(sorted_vals)))]


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) from a thread while the benchmark runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int, period_s: float = 0.01):
        self.gpu = gpu_index
        self.period = period_s
        self.sm: list[float] = []
        self.power: list[float] = []
        self.reasons: set[str] = set()
        self.smax = None
        self._stop = threading.Event()
        self.thread = None
        self.err = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # no NVML: report that instead of numbers
            self.err = f"NVML unavailable: {e}"
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop.set()
        if self.thread:
            self.thread.join(timeout=2)
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.smax, "reasons": [self.err or "no samples"], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.smax, "reasons": sorted(self.reasons),
                "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None}


# ======================================================================================================
# our arm
# ======================================================================================================
def seed_of(rank: int, p: int) -> int:
    return 1_000_003 * (rank + 1) + p


def run_ours(args) -> dict | None:
    import torch
    import torch.distributed as dist

    import sharedtensor
    from sharedtensor_b200 import _native

    rank, local_rank, world = env_rank()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N>1")
    resolve_topology(args, world)
    # host threads and pinned buffers on the socket next to this rank's GPU (matters once 8 ranks copy at once)
    from sharedtensor_b200.utils.affinity import bind_to_gpu
    cpus = bind_to_gpu(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cu = _native.cuda()
    # Host-side coordination only (barriers, max/sum of a few scalars) goes through gloo: a barrier kernel
    # spinning on the GPU while a neighbour is still mapping memory would stall the driver calls it needs.
    if world > 1:
        dist.init_process_group("gloo")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def allreduce(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def allmax(x: float) -> float:
        return allreduce(x, dist.ReduceOp.MAX) if world > 1 else x

    def allsum(x: float) -> float:
        return allreduce(x, dist.ReduceOp.SUM) if world > 1 else x

    def allgather(x: float) -> list:
        if world == 1:
            return [x]
        t = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(t, torch.tensor([x], dtype=torch.float64))
        return [float(v.item()) for v in t]

    n = args.elements
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev)

    def randn_seeded(seed: int, std: float) -> torch.Tensor:
        gen.manual_seed(seed)
        return torch.randn(n, generator=gen, device=dev, dtype=torch.float32) * std

    # ---- synthetic data: the shared initial state and every rank's delta pool (samples of all, full tensors of ours)
    init = randn_seeded(7, INIT_STD)
    pool, pool_s = [], {}
    for r in range(world):
        for p in range(POOL):
            d = randn_seeded(seed_of(r, p), DELTA_STD)
            pool_s[(r, p)] = d[::SAMPLE_STRIDE].clone()
            if r == rank:
                pool.append(d)
            del d
    n_s = pool_s[(0, 0)].numel()
    rng_cad = torch.Generator().manual_seed(99 + rank)
    pinned = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)] if not args.no_e2e else []
    # end-to-end path: two device staging buffers and a copy stream, so that the host->device copy of step j+1 runs
    # while step j is added, sent and read back (what a data loader does); every copy is inside the timed region
    staging = [torch.empty(n, device=dev) for _ in range(2)] if not args.no_e2e else []
    copy_stream = torch.cuda.Stream(device=dev)

    from sharedtensor_b200.utils.probe import ConvergenceProbe
    probe = ConvergenceProbe(cu, dev)

    def measure(topology: str, headline: bool, port: int) -> dict:
        expect_s = init[::SAMPLE_STRIDE].clone()
        counts: dict = {}    # how often every (rank, pool index) has been added since the start
        kw = {"bits": args.bits} if args.bits else {}
        st = None
        if topology == "mesh":
            st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.empty(n, device=dev), topology="mesh",
                                            group_rank=rank, group_size=world, **kw)
            barrier()
        else:
            # the tree: ranks join one after the other so that the shape is the reference's (left, right, redirect ...)
            for r in range(world):
                if r == rank:
                    st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.empty(n, device=dev), **kw)
                barrier()
        assert st is not None
        rep = st._b.rep
        err_buf = torch.zeros(2, dtype=torch.float64, device=dev)
        err_host = torch.zeros(2, dtype=torch.float64).pin_memory()
        extra_launches = 0

        def sampled_err2(light: torch.Tensor | None = None) -> float:
            nonlocal extra_launches
            err_buf.zero_()
            if light is not None:
                cu.sample_sqerr(rep.values_ptr(), SAMPLE_STRIDE * POLL_EVERY, light.data_ptr(), light.numel(), err_buf.data_ptr(), stream)
            else:
                cu.sample_sqerr(rep.values_ptr(), SAMPLE_STRIDE, expect_s.data_ptr(), n_s, err_buf.data_ptr(), stream)
            err_host.copy_(err_buf, non_blocking=True)
            torch.cuda.synchronize()
            extra_launches += 2
            return float(err_host[0])

        def add_expected(r: int, p: int, times: int = 1):
            expect_s.add_(pool_s[(r, p)], alpha=float(times))
            counts[(r, p)] = counts.get((r, p), 0) + times

        def cadences_ns(steps: int) -> list:
            """The pauses before the updates of one region: uniform over the cadence range, stratified (one value from
            each of `steps` equal slices, in this rank's random order), so that every region offers the same load and
            regions differ by what the system does, not by the draw."""
            u = (torch.randperm(steps, generator=rng_cad).double() + 0.5) / steps
            return [int((CADENCE_MS[0] + float(x) * (CADENCE_MS[1] - CADENCE_MS[0])) * 1e6) for x in u]

        def run_steps(k0: int, steps: int, e2e: bool, pool_mod: int = POOL) -> dict:
            """Issues `steps` updates on this rank (all ranks do the same), waits until the replica holds everybody's.
            Times are device times of this rank (CUDA events on the launching stream)."""
            nonlocal extra_launches
            # what everybody is about to add
            total = torch.zeros_like(expect_s)
            for r in range(world):
                for j in range(steps):
                    total.add_(pool_s[(r, (k0 + j) % pool_mod)])
                    counts[(r, (k0 + j) % pool_mod)] = counts.get((r, (k0 + j) % pool_mod), 0) + 1
            expect_s.add_(total)
            upd2 = float((total.double() ** 2).sum())
            upd2_light = float((total[::POLL_EVERY].double() ** 2).sum())
            expect_light = expect_s[::POLL_EVERY].contiguous()
            del total
            d2h = 0
            barrier()
            e0, e_adds, e1 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            main_stream = torch.cuda.current_stream()
            h2d_done = [torch.cuda.Event() for _ in range(2)]
            buf_free = [torch.cuda.Event() for _ in range(2)]
            step_done = torch.cuda.Event()
            copy_ev = []

            def issue_h2d(j: int) -> None:
                b = j % 2
                with torch.cuda.stream(copy_stream):
                    if j >= 2:
                        copy_stream.wait_event(buf_free[b])       # the add of step j-2 has read this buffer
                    else:
                        copy_stream.wait_stream(main_stream)      # not before the timed region starts
                    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    c0.record(copy_stream)
                    staging[b].copy_(pinned[(k0 + j) % pool_mod], non_blocking=True)   # pinned host -> device
                    c1.record(copy_stream)
                    copy_ev.append((c0, c1))
                    h2d_done[b].record(copy_stream)

            if e2e:
                issue_h2d(0)
            cads = cadences_ns(steps)
            for j in range(steps):
                p = (k0 + j) % pool_mod
                cu.delay(cads[j], stream)
                extra_launches += 1
                if e2e:
                    if j + 1 < steps:
                        issue_h2d(j + 1)
                    main_stream.wait_event(h2d_done[j % 2])       # this step's input has arrived
                    st.addFromTensor(staging[j % 2])
                    buf_free[j % 2].record(main_stream)
                    err_buf.zero_()
                    cu.sample_sqerr(rep.values_ptr(), SAMPLE_STRIDE, expect_s.data_ptr(), n_s, err_buf.data_ptr(), stream)
                    err_host.copy_(err_buf, non_blocking=True)                   # this step's result: device -> host
                    step_done.record(main_stream)
                    step_done.synchronize()                       # the host reads the result of every step
                    extra_launches += 2
                    d2h += 16
                else:
                    st.addFromTensor(pool[p])
            e_adds.record()
            deadline = time.time() + 60.0
            rel = float("inf")
            while time.time() < deadline:
                # polled on the light sample; the decision is taken on the full one
                if upd2_light > 0 and (sampled_err2(expect_light) / upd2_light) ** 0.5 > TOL:
                    continue
                e2 = sampled_err2()
                rel = (e2 / upd2) ** 0.5 if upd2 > 0 else 0.0
                if rel <= TOL:
                    break
            e1.record()
            torch.cuda.synchronize()
            out = {"secs": e0.elapsed_time(e1) / 1e3, "secs_adds": e0.elapsed_time(e_adds) / 1e3, "rel": rel, "d2h": d2h}
            if copy_ev:
                out["h2d_gbs"] = statistics.median(4 * n / (a.elapsed_time(b) * 1e6) for a, b in copy_ev)
            return out

        # ---- warm-up (untimed), timed regions, end-to-end region
        k = 0
        if args.warmup:
            run_steps(k, args.warmup, False)
            k += args.warmup
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = rep.launches()
        x0 = extra_launches
        regions = []
        for _ in range(max(1, args.repeats)):
            r = run_steps(k, args.steps, False)
            k += args.steps
            regions.append({"secs": allmax(r["secs"]), "secs_adds": allmax(r["secs_adds"]), "rel": allmax(r["rel"])})
        launches = int(allsum(float(rep.launches() - l0 + extra_launches - x0)))
        clocks = sampler.stop() if rank == 0 else {}
        e2e = None
        if headline and not args.no_e2e:
            k_e2e = max(3, min(args.steps, 10))
            for i, h in enumerate(pinned):
                h.copy_(pool[i % POOL])
            r2 = run_steps(0, k_e2e, True, pool_mod=len(pinned))
            s2 = allmax(r2["secs"])
            e2e = {"value": world * k_e2e / s2, "unit": "updates/s", "steps": k_e2e, "h2d_bytes_per_step": 4 * n,
                   "d2h_bytes_per_step": r2["d2h"] // k_e2e, "final_rel_err": allmax(r2["rel"]),
                   "h2d_gbs_per_rank": [round(v, 2) for v in allgather(r2.get("h2d_gbs", 0.0))],
                   "note": "every step copies its 400 MB delta from pinned host memory; the rate of that copy bounds the value"}

        # ---- single-update convergence latency on device clocks: the origin stamps its GPU's clock behind its add, every
        # rank's probe kernel stamps its own GPU's clock when the sampled error first passes the tolerance; clocks of
        # different GPUs are related through the host's monotonic clock.
        lat_ms = []
        offsets = None
        if world > 1 and args.probes > 0:
            probe.launches = 0
            off, width = probe.calibrate()
            offs = allgather(off)
            widths = allgather(float(width))
            offsets = {"gpu_minus_host_ns": [round(o) for o in offs], "bracket_ns": [round(w) for w in widths]}
            for i in range(args.probes):
                origin, p = i % world, i % POOL
                add_expected(origin, p)
                thr = float((pool_s[(origin, p)][::POLL_EVERY].double() ** 2).sum()) * TOL * TOL
                expect_light = expect_s[::POLL_EVERY].contiguous()
                probe.arm()
                barrier()
                if rank == origin:
                    st.addFromTensor(pool[p])
                    probe.stamp_origin()
                t_conv, t_landed = probe.wait(rep.values_ptr(), SAMPLE_STRIDE * POLL_EVERY, expect_light, thr)
                t_add = allmax(t_landed if rank == origin else -1e30)
                lat_ms.append(allmax(t_conv - t_add) / 1e6)
            extra_launches += probe.launches

        # ---- every element of every replica against the exact sum (the polling above looks at every 64th)
        full_rel = None
        if world > 1 and headline and not args.no_full_check:
            barrier()
            st.flush(30.0)
            barrier()
            st.flush(30.0)
            barrier()
            expect = init.clone()
            for (r, p), c in sorted(counts.items()):
                expect.add_(randn_seeded(seed_of(r, p), DELTA_STD), alpha=float(c))
            got = torch.empty(n, device=dev)
            st.copyToTensor(got)
            torch.cuda.synchronize()
            upd = (expect - init).double().norm().item()
            full_rel = allmax(float((got - expect).double().norm().item() / max(upd, 1e-30)))
            del expect, got
        stats = st.stats()
        barrier()
        st.close()
        barrier()
        return {"regions": regions, "launches": launches, "clocks": clocks, "e2e": e2e, "lat_ms": lat_ms, "stats": stats,
                "offsets": offsets, "full_rel": full_rel, "cfg_bits": st.cfg.bits, "cfg_block": st.cfg.block}

    def summarise(regions: list) -> dict:
        secs = sorted(r["secs"] for r in regions)
        med = statistics.median(secs)
        steady = statistics.median(r["secs_adds"] for r in regions)
        return {"value": world * args.steps / med, "ms_per_step": med * 1e3 / args.steps,
                "value_min": world * args.steps / secs[-1], "value_max": world * args.steps / secs[0],
                "steady_updates_per_s": world * args.steps / steady, "final_rel_err": max(r["rel"] for r in regions)}

    base_port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    main = measure(args.topology, True, base_port)
    # the other topology of the same GPUs, for comparison (a mesh group is one hop wide, a tree up to five)
    other = None
    if world > 1 and not args.no_extra:
        other_name = "mesh" if args.topology == "tree" else "tree"
        o = measure(other_name, False, base_port + 40)
        ol = sorted(o["lat_ms"])
        other = {"topology": other_name, **summarise(o["regions"]), "repeats": len(o["regions"]), "steps": args.steps,
                 "latency_ms": {"p50": pct(ol, 0.5), "p99": pct(ol, 0.99), "probes": len(ol)}}
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    lat = sorted(main["lat_ms"])
    summ = summarise(main["regions"])
    out = {
        "metric": "applied_updates_per_s", "value": summ["value"], "unit": "updates/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "repeats": len(main["regions"]), "ms_per_step": summ["ms_per_step"],
        "value_min": summ["value_min"], "value_max": summ["value_max"], "steady_updates_per_s": summ["steady_updates_per_s"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "ours",
        "config": shared_config(n, world),
        "arm_config": {"transport": f"{args.topology} over NVLink peer memory", "scale_block": main["cfg_block"],
                       "frame_bits": main["cfg_bits"], "host_cpus_bound": len(cpus),
                       "value_is": "median over `repeats` regions of `steps` updates per rank, each timed on the device "
                                   "(CUDA events) from a barrier until the replica holds every rank's updates; max over ranks",
                       "steady_updates_per_s_is": "the same without the final wait for convergence (until the last add was issued)",
                       "e2e_pipeline": "host->device copy of step j+1 overlaps step j (two staging buffers, copy stream); "
                                       "the host waits for and reads every step's result"},
        "final_rel_err": summ["final_rel_err"], "full_check_rel_err": main["full_rel"], "gpu_launches": main["launches"],
        "clocks": main["clocks"],
        "latency_ms": {"p50": pct(lat, 0.5), "p99": pct(lat, 0.99), "probes": len(lat),
                       "clock": "GPU %globaltimer stamps (origin: behind its add; every rank: when its probe kernel first finds the "
                                "error on every 1024th element within tolerance), related through the host's monotonic clock; max over ranks",
                       "clock_offsets": main["offsets"]},
        "device_status": main["stats"].get("device"),
    }
    if main["e2e"]:
        out["e2e"] = main["e2e"]
    if other:
        out["other_topology"] = other
    return out


# ======================================================================================================
# reference arm: the unmodified reference (one CPU process per rank, loopback TCP), same workload
# ======================================================================================================
def run_reference(args) -> dict | None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT / "baseline"))
    import build_ref
    from ref_worker import RefWorker

    rank, local_rank, world = env_rank()
    lib = build_ref.build()
    if lib is None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference source not found (baseline/_ref/sharedtensor.c missing)"}))
        return None
    if world > 1:
        dist.init_process_group("gloo")

    def barrier():
        if world > 1:
            dist.barrier()

    def allmax(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n = args.elements
    threads = max(1, (os.cpu_count() or 8) // max(world, 1) // 2)

    def randn_seeded(seed: int, std: float) -> torch.Tensor:
        g = torch.Generator().manual_seed(seed)
        return torch.randn(n, generator=g, dtype=torch.float32) * std

    # expected values on the sample (every rank regenerates every rank's seeded deltas, as the worker does)
    expect_s = randn_seeded(7, INIT_STD)[::SAMPLE_STRIDE].clone()
    pool_s = {}
    for r in range(world):
        for p in range(POOL):
            pool_s[(r, p)] = randn_seeded(seed_of(r, p), DELTA_STD)[::SAMPLE_STRIDE].clone()
    port = int(os.environ.get("MASTER_PORT", "29500")) + 23
    w = RefWorker(n, threads=threads)
    tmp = f"/tmp/ref_sample_{os.getpid()}.pt"
    try:
        for r in range(world):
            if r == rank:
                if rank == 0:
                    w.call(op="create", host="127.0.0.1", port=port, n=n, seed=7, std=INIT_STD)
                else:
                    w.call(op="create", host="127.0.0.1", port=port, n=n)
            barrier()
        w.call(op="pool", seeds=[seed_of(rank, p) for p in range(POOL)], std=DELTA_STD)
        rng = torch.Generator().manual_seed(99 + rank)

        def rel_err(upd2: float) -> float:
            w.call(op="sample", stride=SAMPLE_STRIDE, path=tmp)
            s = torch.load(tmp)
            return float(((s - expect_s).double() ** 2).sum() / upd2) ** 0.5 if upd2 > 0 else 0.0

        def run_steps(k0: int, steps: int, cap: float, e2e: bool = False):
            """Like the other arm's region.  e2e: every step also reads a 16-byte result (a digest of the replica) back
            through copyToTensor, the only read the reference's API has; its deltas are in host memory to begin with."""
            total = torch.zeros_like(expect_s)
            for r in range(world):
                for j in range(steps):
                    total.add_(pool_s[(r, (k0 + j) % POOL)])
            expect_s.add_(total)
            upd2 = float((total.double() ** 2).sum())
            barrier()
            t0 = time.perf_counter()
            cad = (torch.randperm(steps, generator=rng).double() + 0.5) / steps   # stratified, as in the other arm
            for j in range(steps):
                time.sleep((CADENCE_MS[0] + float(cad[j]) * (CADENCE_MS[1] - CADENCE_MS[0])) / 1e3)
                w.call(op="add_pool", seed=seed_of(rank, (k0 + j) % POOL))
                if e2e:
                    w.call(op="digest", stride=SAMPLE_STRIDE)
            t_adds = time.perf_counter() - t0
            rel, converged = float("inf"), False
            while True:
                rel = rel_err(upd2)
                if rel <= TOL:
                    converged = True
                    break
                if time.perf_counter() - t0 > cap:
                    break
            return time.perf_counter() - t0, rel, converged, t_adds

        k = 0
        if args.warmup:
            run_steps(k, args.warmup, args.ref_time_cap / 2)
            k += args.warmup
        regions = []
        repeats = max(1, args.repeats)
        budget_end = time.perf_counter() + 1.5 * args.ref_time_cap     # all repeats together stay within this
        for i in range(repeats):
            secs, rel, conv, t_adds = run_steps(k, args.steps, args.ref_time_cap)
            k += args.steps
            regions.append({"secs": allmax(secs), "rel": allmax(rel), "conv": allmax(0.0 if conv else 1.0) == 0.0, "secs_adds": allmax(t_adds)})
            stop = allmax(1.0 if (not regions[-1]["conv"] or time.perf_counter() + regions[-1]["secs"] > budget_end) else 0.0)
            if stop > 0:
                break   # a region that ran into the cap (or no time left for another one): no point in repeating it
        e2e = None
        if not args.no_e2e:
            k_e2e = max(3, min(args.steps, 10))
            secs2, rel2, conv2, _ = run_steps(k, k_e2e, args.ref_time_cap / 2, e2e=True)
            secs2 = allmax(secs2)
            e2e = {"value": world * k_e2e / secs2, "unit": "updates/s", "steps": k_e2e, "h2d_bytes_per_step": 4 * n,
                   "d2h_bytes_per_step": 16, "final_rel_err": allmax(rel2), "converged": allmax(0.0 if conv2 else 1.0) == 0.0,
                   "note": "the reference's replica lives in host memory: every step hands addFromTensor a 400 MB delta in host memory "
                           "and reads a 16-byte digest of copyToTensor's output; no device is involved"}
        barrier()
    finally:
        w.kill()
        if os.path.exists(tmp):
            os.remove(tmp)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    secs = sorted(r["secs"] for r in regions)
    med = statistics.median(secs)
    conv_all = all(r["conv"] for r in regions)
    return {
        "metric": "applied_updates_per_s", "value": world * args.steps / med, "unit": "updates/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "repeats": len(regions), "ms_per_step": med * 1e3 / args.steps,
        "value_min": world * args.steps / secs[-1], "value_max": world * args.steps / secs[0],
        "steady_updates_per_s": world * args.steps / statistics.median(r["secs_adds"] for r in regions),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "converged": conv_all, "final_rel_err": max(r["rel"] for r in regions),
        "note": None if conv_all else f"replicas had not reached {TOL} relative error when the {args.ref_time_cap:.0f}s cap ended the wait; "
                                      "value is an upper bound",
        "config": shared_config(n, world),
        "arm_config": {"transport": "reference: CPU processes, binary tree over loopback TCP", "timing": "host wall clock (no device)",
                       "repeats_note": "a region that runs into the wall-clock cap is not repeated"},
        "gpu_launches": 0,
        **({"e2e": e2e} if e2e else {}),
    }


def main():
    args = parse_args()
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
