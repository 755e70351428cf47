"""T6: GPU replicas in separate processes on separate GPUs: TCP join, upgrade to peer-memory rings, snapshot on
join, convergence to the sum, and a rank that leaves (host-side failure: it exits between steps)."""
import json
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _run(world, port, n, scenario):
    sync_dir = tempfile.mkdtemp(prefix="st_multi_")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ST_TEST_SYNC_DIR=sync_dir)
    procs = [subprocess.Popen([sys.executable, str(HERE / "gpu_multi_worker.py"), str(r), str(world), str(port), str(n), scenario],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=150)
        except subprocess.TimeoutExpired:
            p.kill()
            out, err = p.communicate()
        outs.append((p.returncode, out, err))
    results = []
    for rc, out, err in outs:
        lines = [ln for ln in out.splitlines() if ln.startswith("{")]
        if not lines:
            report = "\n".join(f"--- rank {i}: rc={o[0]}\n{o[2][-1500:]}" for i, o in enumerate(outs))
            raise AssertionError(f"a worker produced no result\n{report}")
        results.append(json.loads(lines[-1]))
    shutil.rmtree(sync_dir, ignore_errors=True)
    # which physical GPUs the ranks ran on (pytest -s / -rP shows it): on a box with fewer GPUs than ranks some share one
    used = sorted({r.get("device_uuid", "?") for r in results})
    print(f"[{scenario}] {world} ranks on {len(used)} GPU(s): {used}")
    assert len(used) == min(world, torch.cuda.device_count()), "ranks are spread over the GPUs that exist"
    return results


def _need(k):
    """Ranks are spread over the GPUs that exist (rank % device_count).  Sharing a GPU is safe because no kernel of
    this framework ever waits for a neighbour; a box with one GPU still exercises the join, the fd exchange, the
    mapping of another process's memory and the rings."""
    if torch.cuda.device_count() < 1:
        pytest.skip("needs a GPU")


@pytest.mark.parametrize("world", [2, 4])
def test_tree_over_peer_memory(free_port, world):
    _need(world)
    res = _run(world, free_port, 5 * 4096 + 321, "sum")
    assert sum(r["master"] for r in res) == 1
    for r in res:
        assert r["joined_exact"], "a joiner starts from an exact snapshot of its parent"
        assert r["rel"] is not None and r["rel"] < 5e-5, r
        assert r["errors"] == 0
    assert res[1]["edges"]["up"] == "connected"


@pytest.mark.parametrize("world", [2, 4])
def test_mesh_group(free_port, world):
    _need(world)
    res = _run(world, free_port, 5 * 4096 + 321, "mesh")
    for r in res:
        assert r["joined_exact"], "every member starts from member 0's values"
        assert r["rel"] is not None and r["rel"] < 5e-5, r
        assert r["errors"] == 0
        assert r["members_alive"] == world


def test_rank_leaves_between_steps(free_port):
    _need(3)
    res = _run(3, free_port, 3 * 4096 + 5, "kill_leaf")
    assert res[2].get("exiting")
    for r in res[:2]:
        assert r["rel"] < 5e-5
        assert r["rel_after_loss"] < 5e-5, r
    assert res[0]["edge_failures"] == 1, "the master lost its right child and noticed it on the host"
    assert res[0]["edges"]["right"] == "free"


def test_trainers_that_queue_their_own_rounds(free_port):
    """T8 on GPUs: two async trainers, no engine thread, one sync round queued behind every update; the loss falls
    on both and the replicas end up equal."""
    _need(2)
    res = _run(2, free_port, 0, "train")
    for r in res:
        assert r["errors"] == 0
        assert r["loss_last"] < 0.9 * r["loss_first"], r
        assert r["rounds"] >= 120
    assert abs(res[0]["checksum"] - res[1]["checksum"]) <= 1e-3 * res[0]["norm"], res


def test_cut_up_edge_rejoins_without_losing_updates(free_port):
    """T7 on GPUs, failure made on the host: a replica's up connection is cut, it keeps adding while it re-joins,
    and every update (before, during and after) ends up on both replicas."""
    _need(2)
    res = _run(2, free_port, 3 * 4096 + 17, "rejoin")
    assert res[1]["rejoins"] == 1
    assert res[0]["edge_failures"] == 1
    for r in res:
        assert r["errors"] == 0
        assert r["rel"] < 5e-5, res


def test_master_leaves_and_a_child_takes_over(free_port):
    """T7 on GPUs: the master closes and exits between steps; one of its children becomes the master of the tensor's
    address, the other joins below it, and a later update reaches both."""
    _need(3)
    res = _run(3, free_port, 2 * 4096 + 9, "master_leaves")
    assert res[0].get("left")
    survivors = res[1:]
    assert sum(r["master"] for r in survivors) == 1, survivors
    for r in survivors:
        assert r["errors"] == 0
        assert r["rel_before"] < 5e-5 and r["rel_after"] < 5e-5, survivors
