"""One reference replica in a process of its own, driven over stdin/stdout (one JSON object per line).

The reference calls exit() on every socket error and when a peer disappears (src/sharedtensor.c:62,
80, 99, 421-430), so it is kept out of the test and benchmark processes.  ``RefWorker`` (below) is
the client side: it spawns this file with a stack limit large enough for the reference's
frame buffers, which live on thread stacks (src/sharedtensor.c:118, 144).

Operations: create, add (explicit values), add_seeded (torch.randn with a seed), pool (pre-generate
seeded deltas), add_pool, copy (all values), sample (strided subset of the values), digest (two numbers), quit.
"""
from __future__ import annotations

import ctypes
import json
import os
import resource
import select
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _serve() -> None:
    import torch

    torch.set_num_threads(max(1, int(os.environ.get("REF_WORKER_THREADS", "2"))))
    lib = ctypes.CDLL(str(HERE / "_ref" / "libsharedtensor_ref.so"))
    lib.ref_createOrFetch.restype = ctypes.c_void_p
    lib.ref_createOrFetch.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_long]
    lib.ref_copyToTensor.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]
    lib.ref_addFromTensor.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]
    if lib.ref_open() != 0:
        raise RuntimeError("reference module did not register its functions")
    out = sys.stdout
    z = None
    n = 0
    buf = None
    pool: dict[int, "torch.Tensor"] = {}

    def reply(**kw):
        out.write(json.dumps(kw) + "\n")
        out.flush()

    for line in sys.stdin:
        req = json.loads(line)
        op = req["op"]
        t0 = time.perf_counter()
        if op == "create":
            n = int(req["n"])
            if "values" in req:
                init = torch.tensor(req["values"], dtype=torch.float32)
            elif "seed" in req:
                g = torch.Generator().manual_seed(int(req["seed"]))
                init = torch.randn(n, generator=g, dtype=torch.float32) * float(req.get("std", 1.0))
            else:
                init = torch.zeros(n, dtype=torch.float32)
            z = lib.ref_createOrFetch(req["host"].encode(), int(req["port"]), init.data_ptr(), n)
            buf = torch.zeros(n, dtype=torch.float32)
            reply(ok=True, seconds=time.perf_counter() - t0)
        elif op == "add":
            d = torch.tensor(req["values"], dtype=torch.float32)
            lib.ref_addFromTensor(z, d.data_ptr(), n)
            reply(ok=True, seconds=time.perf_counter() - t0)
        elif op == "add_seeded":
            g = torch.Generator().manual_seed(int(req["seed"]))
            d = torch.randn(n, generator=g, dtype=torch.float32) * float(req["std"])
            t1 = time.perf_counter()
            lib.ref_addFromTensor(z, d.data_ptr(), n)
            reply(ok=True, seconds=time.perf_counter() - t1)
        elif op == "pool":
            for seed in req["seeds"]:
                g = torch.Generator().manual_seed(int(seed))
                pool[int(seed)] = torch.randn(n, generator=g, dtype=torch.float32) * float(req["std"])
            reply(ok=True, seconds=time.perf_counter() - t0)
        elif op == "add_pool":
            d = pool[int(req["seed"])]
            lib.ref_addFromTensor(z, d.data_ptr(), n)
            reply(ok=True, seconds=time.perf_counter() - t0)
        elif op == "copy":
            lib.ref_copyToTensor(z, buf.data_ptr(), n)
            reply(ok=True, values=buf.tolist(), seconds=time.perf_counter() - t0)
        elif op == "sample":
            lib.ref_copyToTensor(z, buf.data_ptr(), n)
            t1 = time.perf_counter()
            s = buf[:: int(req["stride"])]
            if "path" in req:  # large samples go through a file
                torch.save(s.clone(), req["path"])
                reply(ok=True, count=s.numel(), copy_seconds=t1 - t0)
            else:
                reply(ok=True, values=s.tolist(), copy_seconds=t1 - t0)
        elif op == "digest":
            # a 16-byte result of the replica's state, through the reference's only read call
            lib.ref_copyToTensor(z, buf.data_ptr(), n)
            s = buf[:: int(req["stride"])]
            reply(ok=True, digest=[float(s.double().sum()), float(s.numel())], seconds=time.perf_counter() - t0)
        elif op == "quit":
            reply(ok=True)
            out.flush()
            os._exit(0)  # the reference cannot be shut down in an orderly way
        else:
            reply(ok=False, error=f"unknown op {op}")


class RefWorker:
    """Client handle of one reference replica process."""

    def __init__(self, n: int, threads: int = 2, call_timeout: float = 600.0):
        self.call_timeout = call_timeout
        need = n // 8 + (64 << 20)
        soft, hard = resource.getrlimit(resource.RLIMIT_STACK)
        want = need if hard == resource.RLIM_INFINITY else min(need, hard)

        # The reference adds into four malloc()ed arrays it never clears (src/sharedtensor.c:367-370).
        # glibc's perturb tunable set to 255 makes malloc hand out zero-filled blocks (the thread
        # cache has to be off for it to apply to every block), which gives the unmodified binary the
        # start state its author assumed.
        env = dict(os.environ, REF_WORKER_THREADS=str(threads),
                   GLIBC_TUNABLES="glibc.malloc.tcache_count=0:glibc.malloc.perturb=255")
        # The stack limit has to be raised before the worker starts (its frame buffers are stack arrays of n/8
        # bytes, src/sharedtensor.c:118, 144, and glibc sizes thread stacks from the limit at program start).
        # A shell does it: a preexec_fn would run Python between fork and exec in a parent that has threads.
        cmd = [sys.executable, str(Path(__file__).resolve()), "--serve"]
        if soft != resource.RLIM_INFINITY and soft < want:
            cmd = ["bash", "-c", f'ulimit -s {want // 1024} 2>/dev/null; exec "$0" "$@"'] + cmd
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)

    def call(self, timeout: float | None = None, **req) -> dict:
        """One request, one reply line.  The reference can block for good (a joiner whose tree holds only zeros,
        src/sharedtensor.c:385): after `timeout` seconds without a reply the call raises instead of waiting on."""
        assert self.proc.stdin and self.proc.stdout
        self.proc.stdin.write(json.dumps(req) + "\n")
        self.proc.stdin.flush()
        timeout = self.call_timeout if timeout is None else timeout
        ready, _, _ = select.select([self.proc.stdout], [], [], timeout)
        if not ready:
            raise RuntimeError(f"reference worker did not answer {req.get('op')!r} within {timeout:.0f} s")
        line = self.proc.stdout.readline()
        if not line:
            raise RuntimeError(f"reference worker died (exit code {self.proc.poll()})")
        return json.loads(line)

    def kill(self) -> None:
        if self.proc.poll() is None:
            self.proc.kill()
        self.proc.wait()

    def alive(self) -> bool:
        return self.proc.poll() is None


if __name__ == "__main__":
    if "--serve" in sys.argv:
        _serve()
