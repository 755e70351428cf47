"""CPU tensors over loopback TCP — the reference's own ground (src/sharedtensor.c is CPU-only): two replicas in one
process, replica A adds K updates of N(0, 1e-3), the clock stops when replica B holds all of them to 1 % (relative
L2 of what is still outstanding).  Prints one JSON line.

    python benchmarks/cpu_tcp.py --elements 100000000 --steps 10
"""
from __future__ import annotations

import argparse
import json
import socket
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import sharedtensor  # noqa: E402


SAMPLE = 64


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=float, default=1e8)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--tol", type=float, default=0.01)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--tcp-scale-mode", default="tensor",
                    help="tensor = the reference's wire format (one scale per frame); block32 ... block4096 = one exponent "
                         "byte per block, between nodes of this framework only")
    ap.add_argument("--tcp-bits", type=int, default=1,
                    help="bits per element of a frame in a block mode: 1 = sign frames, 8 = integer frames (one frame delivers "
                         "an update to under 1 %%)")
    args = ap.parse_args()
    n = int(args.elements)
    kw = {"tcp_scale_mode": args.tcp_scale_mode, "tcp_bits": args.tcp_bits}
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    torch.manual_seed(0)
    init = torch.randn(n)
    a = sharedtensor.createOrFetch("127.0.0.1", port, init.clone(), **kw)
    t0 = time.perf_counter()
    b = sharedtensor.createOrFetch("127.0.0.1", port, torch.zeros(n), **kw)
    out = torch.empty(n)
    b.flush(args.timeout)
    join_s = time.perf_counter() - t0
    deltas = [torch.randn(n) * 1e-3 for _ in range(2)]
    expect = torch.empty(n)

    def run(steps: int) -> tuple[float, float]:
        a.flush(args.timeout)
        b.flush(args.timeout)
        a.copyToTensor(expect)
        total = torch.zeros(n)
        for j in range(steps):  # what is about to be added, summed before the clock starts
            total += deltas[j % 2]
        # the check looks at every 64th element (like bench.py's device-side check): a full-tensor norm per poll
        # would take longer than a frame and keep the replica's lock busy
        es, outstanding = (expect + total)[::SAMPLE].clone(), float(total[::SAMPLE].norm())
        t0 = time.perf_counter()
        for j in range(steps):
            a.addFromTensor(deltas[j % 2])
        rel = float("inf")
        while time.perf_counter() - t0 < args.timeout:
            b.copyToTensor(out)
            rel = float((out[::SAMPLE] - es).norm()) / outstanding
            if rel <= args.tol:
                break
            time.sleep(0.01)
        return time.perf_counter() - t0, rel

    run(args.warmup)
    secs, rel = run(args.steps)
    st = a.stats()["edges"]["left"]
    print(json.dumps({"metric": "applied_updates_per_s", "impl": "ours, CPU node, loopback TCP", "value": args.steps / secs,
                      "elements": n, "steps": args.steps, "seconds": secs, "final_rel_err": rel, "converged": rel <= args.tol,
                      "late_join_state_transfer_s": join_s, "frames_sent": st["frames_sent"], "bytes_sent": st["bytes_sent"],
                      "tol": args.tol, "tcp_scale_mode": args.tcp_scale_mode, "tcp_bits": args.tcp_bits, "checked": f"every {SAMPLE}th element"}))
    b.close()
    a.close()


if __name__ == "__main__":
    main()
