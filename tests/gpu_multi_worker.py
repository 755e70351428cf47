"""Child process of test_gpu_multi.py: one GPU replica per process, joined through the TCP tree and upgraded
to peer-memory edges.  Prints one JSON line with what it observed."""
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

import sharedtensor  # noqa: E402



def emit(res: dict) -> None:
    """One result line per worker; it also says which physical GPU the rank ran on."""
    d = torch.cuda.current_device()
    res["device"] = d
    res["device_uuid"] = str(torch.cuda.get_device_properties(d).uuid)
    print(json.dumps(res), flush=True)

def _touch_and_wait(sync_dir, name, wanted, timeout=100.0):
    """File rendezvous between the worker processes: start-up time (first CUDA context on a fresh machine) varies by
    seconds, so ordering by sleeps alone is not enough."""
    (Path(sync_dir) / name).touch()
    deadline = time.time() + timeout
    while time.time() < deadline:
        if all((Path(sync_dir) / w).exists() for w in wanted):
            return
        time.sleep(0.01)
    raise RuntimeError(f"rendezvous timed out waiting for {wanted}")


def train(rank, world, port, sync_dir, dev):
    """Async trainers whose sync rounds are queued by the trainer itself (engine="manual", one round per step)."""
    from sharedtensor_b200.models import CharRNN, flatten_parameters
    from sharedtensor_b200.parallel.trainers import AsyncTrainer, structured_token_batches

    torch.manual_seed(5)
    model = CharRNN(vocab=13, hidden=24, layers=1).to(dev)
    init, _ = flatten_parameters(model, align=32)
    _touch_and_wait(sync_dir, f"up_{rank}", [f"joined_{r}" for r in range(rank)])
    st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.zeros_like(init), engine="manual", rel_bits=14)
    (Path(sync_dir) / f"joined_{rank}").touch()
    _touch_and_wait(sync_dir, f"in_{rank}", [f"in_{r}" for r in range(world)])
    tr = AsyncTrainer(model, st, lr=0.3, rounds_per_step=1)
    log = tr.run(structured_token_batches(13, 8, 10, dev, seed=10 + rank, period=1), steps=120, log_every=119)
    _touch_and_wait(sync_dir, f"trained_{rank}", [f"trained_{r}" for r in range(world)])
    # nobody has an engine thread: everybody keeps queueing rounds until all replicas have gone quiet
    deadline = time.time() + 20
    while time.time() < deadline:
        if st.flush(0.05):
            (Path(sync_dir) / f"quiet_{rank}").touch()
        if all((Path(sync_dir) / f"quiet_{r}").exists() for r in range(world)):
            break
    for _ in range(20):
        st.step(1)
    out = torch.empty_like(init)
    st.copyToTensor(out)
    torch.cuda.synchronize()
    s = st.stats()
    emit({"rank": rank, "loss_first": log.loss[0], "loss_last": log.loss[-1], "checksum": float(out.double().sum()),
                      "norm": float(out.double().norm()), "errors": s["device"]["errors"], "rounds": s["device"]["rounds"]})
    _touch_and_wait(sync_dir, f"done_{rank}", [f"done_{r}" for r in range(world)])
    time.sleep(0.2 + 0.3 * (world - rank))
    st.close()


def rejoin(rank, world, port, n, sync_dir, dev):
    """Host-side fault: rank 1 cuts its own up connection (both ends see EOF), goes on adding while it looks for a
    parent, and comes back below the master; nothing that was added anywhere may be lost."""
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    init = torch.randn(n, generator=g, device=dev)
    _touch_and_wait(sync_dir, f"up_{rank}", [f"joined_{r}" for r in range(rank)])
    st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.zeros(n, device=dev), rejoin_backoff_ms=50)
    (Path(sync_dir) / f"joined_{rank}").touch()
    d = []
    for i in range(3):
        g.manual_seed(50 + i)
        d.append(torch.randn(n, generator=g, device=dev) * 1e-2)
    _touch_and_wait(sync_dir, f"in_{rank}", [f"in_{r}" for r in range(world)])
    expect = init + d[0] + d[1] + d[2]
    res = {"rank": rank}
    if rank == 0:
        st.addFromTensor(d[0])
    else:
        st.addFromTensor(d[1])
        assert st.flush(10.0)             # everything said so far has been delivered
        st._b.inject_sever("up")
        for i in range(10):               # keeps adding while the edge is down and while it re-joins
            st.addFromTensor(d[2] / 10)
            time.sleep(0.02)
        deadline = time.time() + 20
        while time.time() < deadline and st.stats()["rejoins"] < 1:
            time.sleep(0.02)
        res["rejoins"] = st.stats()["rejoins"]
    out = torch.empty(n, device=dev)
    deadline = time.time() + 30
    rel = None
    while time.time() < deadline:
        st.copyToTensor(out)
        torch.cuda.synchronize()
        rel = ((out - expect).norm() / expect.norm()).item()
        if rel < 5e-5:
            break
        time.sleep(0.01)
    res["rel"] = rel
    s = st.stats()
    res["errors"] = s["device"]["errors"]
    res["edge_failures"] = s.get("edge_failures", 0)
    res["edges"] = {k: v["state"] for k, v in s["edges"].items()}
    emit(res)
    _touch_and_wait(sync_dir, f"done_{rank}", [f"done_{r}" for r in range(world)])
    time.sleep(0.2 + 0.3 * (world - rank))
    st.close()


def master_leaves(rank, world, port, n, sync_dir, dev):
    """Host-side failure: the master closes its replica between steps and exits.  Its two children notice on the
    host, one of them takes over the tensor's address, the other joins below it, and work goes on."""
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    init = torch.randn(n, generator=g, device=dev)
    _touch_and_wait(sync_dir, f"up_{rank}", [f"joined_{r}" for r in range(rank)])
    st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.zeros(n, device=dev), rejoin_backoff_ms=50)
    (Path(sync_dir) / f"joined_{rank}").touch()
    d = []
    for i in range(2):
        g.manual_seed(60 + i)
        d.append(torch.randn(n, generator=g, device=dev) * 1e-2)
    _touch_and_wait(sync_dir, f"in_{rank}", [f"in_{r}" for r in range(world)])
    out = torch.empty(n, device=dev)

    def wait_for(expect, seconds):
        deadline = time.time() + seconds
        rel = None
        while time.time() < deadline:
            st.copyToTensor(out)
            torch.cuda.synchronize()
            rel = ((out - expect).norm() / expect.norm()).item()
            if rel < 5e-5:
                break
            time.sleep(0.01)
        return rel

    if rank == 0:
        st.addFromTensor(d[0])
        st.flush(10.0)
        _touch_and_wait(sync_dir, "got_0", [f"got_{r}" for r in range(world)])  # the children hold the update
        time.sleep(0.3)
        st.close()  # nothing in flight: leaves between steps
        (Path(sync_dir) / "left").touch()
        emit({"rank": 0, "left": True})
        return
    res = {"rank": rank, "rel_before": wait_for(init + d[0], 30)}
    st.flush(10.0)
    _touch_and_wait(sync_dir, f"got_{rank}", [f"got_{r}" for r in range(world)] + ["left"])
    deadline = time.time() + 30
    while time.time() < deadline:  # a new home: either this replica is the master now or it has an up edge again
        s = st.stats()
        if s["master"] or s["edges"]["up"]["state"] == "connected":
            break
        time.sleep(0.02)
    _touch_and_wait(sync_dir, f"home_{rank}", [f"home_{r}" for r in range(1, world)])
    time.sleep(0.3)
    if rank == 1:
        st.addFromTensor(d[1])
    res["rel_after"] = wait_for(init + d[0] + d[1], 30)
    s = st.stats()
    res["master"] = bool(s["master"])
    res["errors"] = s["device"]["errors"]
    res["rejoins"] = s["rejoins"]
    emit(res)
    _touch_and_wait(sync_dir, f"done_{rank}", [f"done_{r}" for r in range(1, world)])
    time.sleep(0.2 + (0.0 if res["master"] else 0.0) + (0.6 if res["master"] else 0.0))  # the new master leaves last
    st.close()


def main():
    sync_dir = os.environ["ST_TEST_SYNC_DIR"]
    rank, world, port, n, scenario = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    torch.cuda.set_device(rank % torch.cuda.device_count())
    dev = torch.device("cuda", torch.cuda.current_device())
    if scenario == "train":
        return train(rank, world, port, sync_dir, dev)
    if scenario == "rejoin":
        return rejoin(rank, world, port, n, sync_dir, dev)
    if scenario == "master_leaves":
        return master_leaves(rank, world, port, n, sync_dir, dev)
    g = torch.Generator(device=dev)
    g.manual_seed(1234)
    init = torch.randn(n, generator=g, device=dev)
    if scenario == "mesh":
        st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.zeros(n, device=dev), topology="mesh",
                                        group_rank=rank, group_size=world)
    else:
        # the founder first, then the others in rank order (the tree's shape follows the join order)
        _touch_and_wait(sync_dir, f"up_{rank}", [f"joined_{r}" for r in range(rank)])
        st = sharedtensor.createOrFetch("127.0.0.1", port, init if rank == 0 else torch.zeros(n, device=dev), rejoin_backoff_ms=100)
        (Path(sync_dir) / f"joined_{rank}").touch()
    out = torch.empty(n, device=dev)
    st.copyToTensor(out)
    torch.cuda.synchronize()
    res = {"rank": rank, "master": st.is_master, "joined_exact": bool(torch.equal(out, init))}
    # every rank adds its own delta; all must reach the sum
    deltas = []
    for r in range(world):
        g.manual_seed(77 + r)
        deltas.append(torch.randn(n, generator=g, device=dev) * 1e-2)
    _touch_and_wait(sync_dir, f"in_{rank}", [f"in_{r}" for r in range(world)])  # everybody is in
    st.addFromTensor(deltas[rank])
    expect = init + sum(deltas)
    if scenario == "kill_leaf" and rank == world - 1:
        # leave between steps with nothing in flight: wait for own update to be delivered, then exit
        st.flush(10.0)
        time.sleep(0.5)
        res["exiting"] = True
        emit(res)
        os._exit(0)
    deadline = time.time() + 30
    rel = None
    while time.time() < deadline:
        st.copyToTensor(out)
        torch.cuda.synchronize()
        rel = ((out - expect).norm() / expect.norm()).item()
        if rel < 5e-5:
            break
        time.sleep(0.01)
    res["rel"] = rel
    if scenario == "kill_leaf":
        # survivors: the dead neighbour is noticed on the host, the edge is dropped, work goes on
        time.sleep(1.5)
        extra = torch.full((n,), 0.5, device=dev)
        if rank == 0:
            st.addFromTensor(extra)
        expect2 = expect + 0.5
        deadline = time.time() + 20
        while time.time() < deadline:
            st.copyToTensor(out)
            torch.cuda.synchronize()
            rel2 = ((out - expect2).norm() / expect2.norm()).item()
            if rel2 < 5e-5:
                break
            time.sleep(0.01)
        res["rel_after_loss"] = rel2
    s = st.stats()
    res["edges"] = {k: v["state"] for k, v in s["edges"].items()}
    res["edge_failures"] = s.get("edge_failures", 0)
    res["members_alive"] = s.get("members_alive")
    res["errors"] = s["device"]["errors"]
    res["frames_sent"] = s["device"]["frames_sent"]
    emit(res)
    alive = world - 1 if scenario == "kill_leaf" else world
    _touch_and_wait(sync_dir, f"done_{rank}", [f"done_{r}" for r in range(alive)])  # nobody leaves before all have looked
    time.sleep(0.2 + 0.3 * (world - rank))  # leaves first
    st.close()


if __name__ == "__main__":
    main()
