"""T8 on CPU ranks: two processes train the same small model on a learnable task, once synchronously (gloo all-reduce)
and once through a shared tensor; both learn, and the asynchronous replicas end up with the same parameters."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent


def _run(world, port, mode, steps):
    procs = [subprocess.Popen([sys.executable, str(HERE / "train_worker.py"), str(r), str(world), str(port), mode, str(steps)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=150)
        except subprocess.TimeoutExpired:
            p.kill()
            out, err = p.communicate()
        outs.append((p.returncode, out, err))
    res = []
    for rc, out, err in outs:
        lines = [ln for ln in out.splitlines() if ln.startswith("{")]
        if not lines:
            raise AssertionError("a rank produced no result\n" + "\n".join(f"--- rc={o[0]}\n{o[2][-1500:]}" for o in outs))
        res.append(json.loads(lines[-1]))
    return res


@pytest.mark.parametrize("mode", ["sync", "async"])
def test_two_cpu_ranks_learn(free_port, mode):
    res = _run(2, free_port, mode, 120)
    for r in res:
        assert r["loss_last"] < 0.9 * r["loss_first"], r
    if mode == "async":
        (s0, n0), (s1, _) = res[0]["checksum"], res[1]["checksum"]
        assert abs(s0 - s1) <= 1e-3 * n0, res
