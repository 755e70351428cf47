"""T1/T4: sum consistency of CPU replicas over localhost TCP, including the 2-process, 240-element,
1000-adds-each configuration."""
import multiprocessing as mp
import time

import pytest
import torch

import sharedtensor


def _wait_equal(nodes, expect, tol_rel=1e-5, tol_inf=1e-4, timeout=30.0):
    t0 = time.time()
    out = torch.zeros_like(expect)
    worst = None
    while time.time() - t0 < timeout:
        worst = 0.0
        ok = True
        for n in nodes:
            n.copyToTensor(out)
            rel = ((out - expect).norm() / expect.norm()).item()
            inf = (out - expect).abs().max().item()
            worst = max(worst, rel)
            if rel > tol_rel or inf > tol_inf:
                ok = False
        if ok:
            return worst
        time.sleep(0.02)
    raise AssertionError(f"replicas did not converge: worst rel-L2 {worst}")


def _worker(port, seed, iters, q, ready):
    torch.manual_seed(seed)
    shape = (4, 5, 6, 2)
    init = torch.randn(shape)
    st = sharedtensor.createOrFetch("127.0.0.1", port, init)
    ready.wait()
    total = torch.zeros(shape)
    for _ in range(iters):
        d = torch.randn(shape) * 1e-2
        st.addFromTensor(d)
        total += d
    q.put((seed, init if st.is_master else None, total))
    # wait for the parent to tell us the expected sum
    expect = q_in[seed].get()
    out = torch.zeros(shape)
    t0 = time.time()
    ok = False
    while time.time() - t0 < 30:
        st.copyToTensor(out)
        rel = ((out - expect).norm() / expect.norm()).item()
        inf = (out - expect).abs().max().item()
        if rel <= 1e-5 and inf <= 1e-4:
            ok = True
            break
        time.sleep(0.02)
    q.put((seed, ok, rel, inf))
    done.wait()
    st.close()


q_in = {}
done = None


def test_config1_two_processes_1000_adds_each(free_port):
    """2 processes on localhost TCP, fp32 tensor of shape 4x5x6x2 from N(0,1), 1000 addFromTensor calls
    each with N(0,1e-2) deltas; both replicas must reach initial + sum of all deltas."""
    global done
    ctx = mp.get_context("fork")
    q = ctx.Queue()
    ready = ctx.Event()
    done = ctx.Event()
    q_in[1] = ctx.Queue()
    q_in[2] = ctx.Queue()
    p1 = ctx.Process(target=_worker, args=(free_port, 1, 1000, q, ready))
    p1.start()
    time.sleep(0.5)  # the first process founds the tensor
    p2 = ctx.Process(target=_worker, args=(free_port, 2, 1000, q, ready))
    p2.start()
    time.sleep(0.5)
    ready.set()
    res = [q.get(timeout=60), q.get(timeout=60)]
    init = [r[1] for r in res if r[1] is not None]
    assert len(init) == 1, "exactly one process is the master"
    expect = init[0] + res[0][2] + res[1][2]
    q_in[1].put(expect)
    q_in[2].put(expect)
    verdicts = [q.get(timeout=60), q.get(timeout=60)]
    done.set()
    p1.join(20)
    p2.join(20)
    for seed, ok, rel, inf in verdicts:
        assert ok, f"replica {seed}: rel-L2 {rel:.3g}, L-inf {inf:.3g}"


@pytest.mark.parametrize("n_nodes", [3, 6])
@pytest.mark.parametrize("tcp_scale_mode", ["tensor", "block32", "block32/8"])
def test_sum_consistency_tree(free_port, n_nodes, tcp_scale_mode):
    torch.manual_seed(n_nodes)
    n = 1000
    init = torch.randn(n)
    kw = {"tcp_scale_mode": tcp_scale_mode}
    if tcp_scale_mode.endswith("/8"):   # block scales with 8-bit integer frames
        kw = {"tcp_scale_mode": tcp_scale_mode[:-2], "tcp_bits": 8}
    nodes = [sharedtensor.createOrFetch("127.0.0.1", free_port, init, **kw)]
    try:
        for _ in range(n_nodes - 1):
            nodes.append(sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), **kw))
        expect = init.clone()
        for it in range(30):
            for i, node in enumerate(nodes):
                d = torch.randn(n) * 1e-2 * (1 + i)
                node.addFromTensor(d)
                expect += d
        _wait_equal(nodes, expect, tol_rel=2e-5 if tcp_scale_mode == "tensor" else 1e-5, tol_inf=5e-4)
    finally:
        for node in nodes:
            node.cfg.rejoin = False
        for node in reversed(nodes):
            node.close()


def test_push_update_and_late_joiner_with_history(free_port):
    n = 513
    torch.manual_seed(5)
    init = torch.randn(n)
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    try:
        cur = torch.zeros(n)
        a.copyToTensor(cur)
        new = cur + 0.5
        a.pushUpdate(new, cur)
        b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))
        _wait_equal([a, b], init + 0.5, tol_rel=2e-5, tol_inf=5e-4)
        assert b.flush(10.0)
        s = b.stats()
        assert s["edges"]["up"]["frames_recv"] > 0 and not s["master"]
        b.close()
    finally:
        a.close()


def test_state_dict_roundtrip(free_port):
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.arange(10.0))
    try:
        sd = a.state_dict()
        assert torch.equal(sd["values"], torch.arange(10.0))
        sd["values"] = sd["values"] * 2
        a.load_state_dict(sd)
        out = torch.zeros(10)
        a.copyToTensor(out)
        assert torch.equal(out, torch.arange(10.0) * 2)
    finally:
        a.close()


def test_rate_cap(free_port):
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.randn(64), max_frames_per_s=50.0)
    try:
        b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(64), ready_mode="first_frame")
        t0 = time.time()
        for _ in range(20):
            a.addFromTensor(torch.randn(64))
            time.sleep(0.02)
        time.sleep(0.2)
        sent = a.stats()["edges"]["left"]["frames_sent"]
        elapsed = time.time() - t0
        assert sent <= 50.0 * elapsed + 25, (sent, elapsed)
        b.close()
    finally:
        a.close()


def test_dropping_a_connected_tensor_and_using_a_closed_one(free_port):
    """Garbage-collecting a connected tensor closes it quietly (the reference calls exit(-1) there,
    src/sharedtensor.c:421-430); closing twice is fine; using a closed tensor raises."""
    import gc

    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.ones(100))
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(100))
    assert a.stats()["edges"]["left"]["state"] == "connected"
    del b
    gc.collect()
    t0 = time.time()
    while time.time() - t0 < 10 and a.stats()["edges"]["left"]["state"] != "free":
        time.sleep(0.02)
    assert a.stats()["edges"]["left"]["state"] == "free"
    a.close()
    a.close()
    with pytest.raises(RuntimeError, match="closed"):
        a.addFromTensor(torch.ones(100))


def test_membership_events_are_recorded(free_port):
    """stats()["events"]: what happened to this node's place in the tree, oldest first."""
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.ones(64))
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(64), rejoin_backoff_ms=50)
    try:
        assert [e["kind"] for e in a.stats()["events"]] == ["master", "adopted"]
        assert [e["kind"] for e in b.stats()["events"]] == ["joined"]
        b._b.inject_sever("up")
        t0 = time.time()
        while time.time() - t0 < 10 and b.stats()["rejoins"] < 1:
            time.sleep(0.02)
        kb = [e["kind"] for e in b.stats()["events"]]
        assert kb[:2] == ["joined", "edge_lost"] and kb[-1] == "rejoined", kb
        t0 = time.time()
        while time.time() - t0 < 10 and [e["kind"] for e in a.stats()["events"]].count("adopted") < 2:
            time.sleep(0.02)
        ka = [e["kind"] for e in a.stats()["events"]]
        assert "edge_lost" in ka and ka.count("adopted") == 2, ka
        ev = b.stats()["events"][-1]
        assert ev["ms"] > 1.6e12 and "below 127.0.0.1" in ev["detail"]
    finally:
        b.cfg.rejoin = False
        b.close()
        a.close()


def test_eight_bit_frames_deliver_an_update_in_one_frame(free_port):
    """CPU replicas over TCP with 8-bit integer frames: a fresh update is on the neighbour to under one percent after
    a single frame (sign frames need about ten), and the frame is one code byte per element plus the scale bytes."""
    n = 40000
    torch.manual_seed(8)
    init = torch.randn(n)
    kw = {"tcp_scale_mode": "block32", "tcp_bits": 8, "rejoin": False}
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone(), **kw)
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), **kw)
    try:
        out = torch.zeros(n)
        _wait_equal([a, b], init, tol_rel=1e-5, tol_inf=5e-4)
        time.sleep(0.3)
        before = b.stats()["edges"]["up"]
        d = torch.randn(n)
        a.addFromTensor(d)
        deadline = time.time() + 10
        while time.time() < deadline:
            b.copyToTensor(out)
            if ((out - init - d).norm() / d.norm()).item() < 1e-2:
                break
            time.sleep(0.001)
        assert ((out - init - d).norm() / d.norm()).item() < 1e-2
        _wait_equal([a, b], init + d, tol_rel=1e-5, tol_inf=5e-4)
        after = b.stats()["edges"]["up"]
        frames = after["frames_recv"] - before["frames_recv"]
        assert 1 <= frames <= 6, frames   # three frames carry the update down to the cut-off, one says "nothing more"
        assert (after["bytes_recv"] - before["bytes_recv"]) == frames * (n + n // 32)
    finally:
        b.close()
        a.close()


def test_eight_bit_frames_need_a_block_mode():
    with pytest.raises(ValueError):
        sharedtensor.Config(tcp_bits=8)
    with pytest.raises(ValueError):
        sharedtensor.Config(tcp_scale_mode="block32", tcp_bits=4)
