#!/usr/bin/env python
"""Headline benchmark: applied updates/s (and replica-convergence latency) of a shared 100M-element fp32
tensor, each rank adding N(0,1e-3) deltas at a randomised 0.5-2 ms cadence.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 50 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference over loopback TCP, same workload

One step of a rank = wait its cadence interval (a device-side delay kernel standing in for the compute
between updates) + ``addFromTensor(delta)``.  The engine propagates in the background.  The timed region
starts after a barrier and ends, on every rank, when its replica holds initial + the sum of ALL ranks'
timed updates to within 1 % (relative L2 of the outstanding update, checked on a strided sample of the
replica by a device kernel); the reported time is the maximum over ranks and
value = world_size * steps / time.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
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
SAMPLE_STRIDE = 64       # convergence is checked on every 64th element
TOL = 1e-2               # "applied": outstanding error below 1 % of the update's norm


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--elements", type=int, default=N_ELEMENTS)
    ap.add_argument("--probes", type=int, default=24, help="single-update latency probes after the timed region")
    ap.add_argument("--topology", default="auto", choices=["auto", "tree", "mesh"],
                    help="auto: the fixed fully connected group when the ranks are known up front (N > 1 under "
                         "torch.distributed.run), else the join tree; the other one is measured too and reported under "
                         "other_topology")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the comparison run on the other topology")
    ap.add_argument("--ref-time-cap", type=float, default=120.0, help="wall-clock cap of the reference arm's wait, seconds")
    return ap.parse_args()


def resolve_topology(args, world: int) -> None:
    if args.topology == "auto":
        args.topology = "mesh" if world > 1 else "tree"


def env_rank():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) from a thread while the benchmark runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int, period_s: float = 0.02):
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

    def allmax(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    n = args.elements
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev)

    def randn_seeded(seed: int, std: float) -> torch.Tensor:
        gen.manual_seed(seed)
        return torch.randn(n, generator=gen, device=dev, dtype=torch.float32) * std

    # ---- synthetic data: the shared initial state and every rank's delta pool (samples of all, full tensors of ours)
    init = randn_seeded(7, INIT_STD)
    expect_s = init[::SAMPLE_STRIDE].clone()
    pool, pool_s = [], {}
    for r in range(world):
        for p in range(POOL):
            d = randn_seeded(seed_of(r, p), DELTA_STD)
            pool_s[(r, p)] = d[::SAMPLE_STRIDE].clone()
            if r == rank:
                pool.append(d)
            del d
    n_s = expect_s.numel()
    rng_cad = torch.Generator().manual_seed(99 + rank)
    pinned = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)] if not args.no_e2e else []
    for i, h in enumerate(pinned):
        h.copy_(pool[i % POOL])
    # end-to-end path: two device staging buffers and a copy stream, so that the host->device copy of step j+1 runs
    # while step j is added, sent and read back (what a data loader does); every copy is inside the timed region
    staging = [torch.empty(n, device=dev) for _ in range(2)] if not args.no_e2e else []
    copy_stream = torch.cuda.Stream(device=dev)

    def measure(topology: str, with_e2e: bool, port: int) -> dict:
        nonlocal expect_s
        expect_s = init[::SAMPLE_STRIDE].clone()
        # ---- the tree: ranks join one after the other so that the shape is the reference's (left, right, redirect ...)
        st = None
        if topology == "mesh":
            st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.empty(n, device=dev), topology="mesh",
                                            group_rank=rank, group_size=world)
            barrier()
        else:
            for r in range(world):
                if r == rank:
                    st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.empty(n, device=dev))
                barrier()
        assert st is not None
        rep = st._b.rep
        err_buf = torch.zeros(2, dtype=torch.float64, device=dev)
        err_host = torch.zeros(2, dtype=torch.float64).pin_memory()
        extra_launches = 0

        def sampled_err2() -> float:
            nonlocal extra_launches
            err_buf.zero_()
            cu.sample_sqerr(rep.values_ptr(), SAMPLE_STRIDE, expect_s.data_ptr(), n_s, err_buf.data_ptr(), stream)
            err_host.copy_(err_buf, non_blocking=True)
            torch.cuda.synchronize()
            extra_launches += 2
            return float(err_host[0])

        def add_expected(r: int, p: int, times: int = 1):
            expect_s.add_(pool_s[(r, p)], alpha=float(times))

        def cadence_ns() -> int:
            u = float(torch.rand(1, generator=rng_cad))
            return int((CADENCE_MS[0] + u * (CADENCE_MS[1] - CADENCE_MS[0])) * 1e6)

        def run_steps(k0: int, steps: int, e2e: bool, pool_mod: int = POOL) -> tuple[float, float, int]:
            """Issues `steps` updates on this rank (all ranks do the same), waits until the replica holds everybody's;
            returns (seconds to local convergence, final relative error, bytes read back)."""
            nonlocal extra_launches
            # what everybody is about to add
            upd2 = 0.0
            total = torch.zeros_like(expect_s)
            for r in range(world):
                for j in range(steps):
                    total.add_(pool_s[(r, (k0 + j) % pool_mod)])
            expect_s.add_(total)
            upd2 = float((total.double() ** 2).sum())
            del total
            d2h = 0
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            main_stream = torch.cuda.current_stream()
            h2d_done = [torch.cuda.Event() for _ in range(2)]
            buf_free = [torch.cuda.Event() for _ in range(2)]
            step_done = torch.cuda.Event()

            def issue_h2d(j: int) -> None:
                b = j % 2
                with torch.cuda.stream(copy_stream):
                    if j >= 2:
                        copy_stream.wait_event(buf_free[b])       # the add of step j-2 has read this buffer
                    else:
                        copy_stream.wait_stream(main_stream)      # not before the timed region starts
                    staging[b].copy_(pinned[(k0 + j) % pool_mod], non_blocking=True)   # pinned host -> device
                    h2d_done[b].record(copy_stream)

            if e2e:
                issue_h2d(0)
            for j in range(steps):
                p = (k0 + j) % pool_mod
                cu.delay(cadence_ns(), stream)
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
            deadline = time.time() + 60.0
            rel = float("inf")
            while time.time() < deadline:
                e2 = sampled_err2()
                rel = (e2 / upd2) ** 0.5 if upd2 > 0 else 0.0
                if rel <= TOL:
                    break
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / 1e3, rel, d2h

        # ---- warm-up (untimed), timed region, end-to-end region
        if args.warmup:
            run_steps(0, args.warmup, False)
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = rep.launches()
        x0 = extra_launches
        secs, rel, _ = run_steps(args.warmup, args.steps, False)
        launches = int(allsum(float(rep.launches() - l0 + extra_launches - x0)))
        secs = allmax(secs)
        rel = allmax(rel)
        clocks = sampler.stop() if rank == 0 else {}
        e2e = None
        if with_e2e:
            k_e2e = max(3, min(args.steps, 10))
            if pinned:
                for i, h in enumerate(pinned):
                    h.copy_(pool[i % POOL])
            s2, rel2, d2h = run_steps(args.warmup + args.steps, k_e2e, True, pool_mod=len(pinned))
            s2 = allmax(s2)
            e2e = {"value": world * k_e2e / s2, "unit": "updates/s", "steps": k_e2e, "h2d_bytes_per_step": 4 * n,
                   "d2h_bytes_per_step": d2h // k_e2e, "final_rel_err": allmax(rel2)}

        # ---- single-update convergence latency: one rank adds, everybody measures until its replica has it
        lat = []
        for i in range(args.probes if world > 1 else 0):
            origin, p = i % world, i % POOL
            add_expected(origin, p)
            upd2 = float((pool_s[(origin, p)].double() ** 2).sum())
            barrier()
            t0 = time.perf_counter()
            if rank == origin:
                st.addFromTensor(pool[p])
            while True:
                e2 = sampled_err2()
                if (e2 / upd2) ** 0.5 <= TOL or time.perf_counter() - t0 > 5.0:
                    break
            lat.append(allmax(time.perf_counter() - t0))
        stats = st.stats()
        barrier()
        st.close()
        barrier()
        return {"secs": secs, "rel": rel, "launches": launches, "clocks": clocks, "e2e": e2e, "lat": lat, "stats": stats}
    base_port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    main = measure(args.topology, not args.no_e2e, base_port)
    # the other topology of the same GPUs, for comparison (a mesh group is one hop wide, a tree up to five)
    other = None
    if world > 1 and not args.no_extra:
        other_name = "mesh" if args.topology == "tree" else "tree"
        o = measure(other_name, False, base_port + 40)
        ol = sorted(x * 1e3 for x in o["lat"])
        other = {"topology": other_name, "value": world * args.steps / o["secs"], "ms_per_step": o["secs"] * 1e3 / args.steps,
                 "final_rel_err": o["rel"], "latency_ms": {"p50": ol[len(ol) // 2] if ol else None,
                                                           "p99": ol[min(len(ol) - 1, int(0.99 * len(ol)))] if ol else None}}
    secs, rel, launches, clocks, e2e, lat, stats = (main[k] for k in ("secs", "rel", "launches", "clocks", "e2e", "lat", "stats"))
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    lat_ms = sorted(x * 1e3 for x in lat)
    out = {
        "metric": "applied_updates_per_s", "value": world * args.steps / secs, "unit": "updates/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3 / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "shared parameter vector, 100M fp32 elements ~ N(0,1)", "elements": n, "global_batch": world,
                   "seq_len": None, "parallelism": f"async-dp{world} ({args.topology} over NVLink peer memory)",
                   "delta": "N(0,1e-3) fp32", "cadence_ms": list(CADENCE_MS), "scale_block": 32,
                   "applied_when": f"rel-L2 of outstanding update <= {TOL} on every replica",
                   "l2": "inputs larger than L2 (400 MB per array)",
                   "host_cpus_bound": len(cpus),
                   "e2e_pipeline": "host->device copy of step j+1 overlaps step j (two staging buffers, copy stream); "
                                   "the host waits for and reads every step's result"},
        "final_rel_err": rel, "gpu_launches": launches, "clocks": clocks,
        "latency_ms": {"p50": lat_ms[len(lat_ms) // 2] if lat_ms else None,
                       "p99": lat_ms[min(len(lat_ms) - 1, int(0.99 * len(lat_ms)))] if lat_ms else None,
                       "probes": len(lat_ms), "clock": "host wall clock after a barrier, max over ranks"},
        "device_status": stats.get("device"),
    }
    if e2e:
        out["e2e"] = e2e
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

        def run_steps(k0: int, steps: int, cap: float):
            total = torch.zeros_like(expect_s)
            for r in range(world):
                for j in range(steps):
                    total.add_(pool_s[(r, (k0 + j) % POOL)])
            expect_s.add_(total)
            upd2 = float((total.double() ** 2).sum())
            barrier()
            t0 = time.perf_counter()
            for j in range(steps):
                u = float(torch.rand(1, generator=rng))
                time.sleep((CADENCE_MS[0] + u * (CADENCE_MS[1] - CADENCE_MS[0])) / 1e3)
                w.call(op="add_pool", seed=seed_of(rank, (k0 + j) % POOL))
            rel, converged = float("inf"), False
            while True:
                rel = rel_err(upd2)
                if rel <= TOL:
                    converged = True
                    break
                if time.perf_counter() - t0 > cap:
                    break
            return time.perf_counter() - t0, rel, converged

        if args.warmup:
            run_steps(0, args.warmup, args.ref_time_cap / 2)
        secs, rel, conv = run_steps(args.warmup, args.steps, args.ref_time_cap)
        secs = allmax(secs)
        rel = allmax(rel)
        conv_all = allmax(0.0 if conv else 1.0) == 0.0
        barrier()
    finally:
        w.kill()
        if os.path.exists(tmp):
            os.remove(tmp)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    return {
        "metric": "applied_updates_per_s", "value": world * args.steps / secs, "unit": "updates/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3 / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "converged": conv_all, "final_rel_err": rel,
        "note": None if conv_all else f"replicas had not reached {TOL} relative error when the {args.ref_time_cap:.0f}s cap ended the wait; "
                                      "value is an upper bound",
        "config": {"model": "shared parameter vector, 100M fp32 elements ~ N(0,1)", "elements": n, "global_batch": world, "seq_len": None,
                   "parallelism": f"async-dp{world} (reference: CPU processes, binary tree over loopback TCP)", "delta": "N(0,1e-3) fp32",
                   "cadence_ms": list(CADENCE_MS), "applied_when": f"rel-L2 of outstanding update <= {TOL} on every replica"},
        "gpu_launches": 0,
    }


def main():
    args = parse_args()
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
