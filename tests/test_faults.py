"""T7: failure detection and recovery, with every failure made on the host: a cut socket, a killed
CPU process, frames dropped after they were read."""
import multiprocessing as mp
import os
import signal
import time

import pytest
import torch

import sharedtensor


def _poll(fn, timeout=20.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if fn():
            return True
        time.sleep(0.05)
    return False


def test_child_loss_frees_the_slot_and_a_new_child_is_adopted(free_port):
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.arange(32.0))
    try:
        b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(32), rejoin=False)
        assert a.stats()["edges"]["left"]["state"] == "connected"
        b.close()  # peer goes away: EOF on a's left edge
        assert _poll(lambda: a.stats()["edges"]["left"]["state"] == "free")
        assert a.stats()["edge_failures"] == 1
        a.addFromTensor(torch.ones(32))  # the master keeps working
        c = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(32), rejoin=False)
        out = torch.zeros(32)
        c.copyToTensor(out)
        assert torch.allclose(out, torch.arange(32.0) + 1, atol=1e-2)
        assert a.stats()["edges"]["left"]["state"] == "connected", "the freed slot is used again"
        c.close()
    finally:
        a.close()


def test_severed_up_edge_rejoins_and_keeps_unsent_updates(free_port):
    n = 128
    torch.manual_seed(2)
    init = torch.randn(n)
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50)
    try:
        assert b.flush(10.0)
        b._b.inject_sever("up")  # cut the socket under the edge
        assert _poll(lambda: b.stats()["rejoins"] == 1), b.stats()
        d = torch.randn(n) * 1e-2
        b.addFromTensor(d)
        expect = init + d
        out = torch.zeros(n)
        assert _poll(lambda: (a.copyToTensor(out) - expect).abs().max().item() < 1e-4)
        assert _poll(lambda: (b.copyToTensor(out) - expect).abs().max().item() < 1e-4)
    finally:
        b.cfg.rejoin = False
        b.close()
        a.close()


def _child(port, n):
    st = sharedtensor.createOrFetch("127.0.0.1", port, torch.zeros(n))
    st.addFromTensor(torch.ones(n))
    time.sleep(60)


def test_killed_process_is_detected_and_survivors_continue(free_port):
    n = 64
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))
    ctx = mp.get_context("fork")
    p = ctx.Process(target=_child, args=(free_port, n))
    p.start()
    try:
        out = torch.zeros(n)
        assert _poll(lambda: (a.copyToTensor(out) - 1).abs().max().item() < 1e-4), "child's update arrives"
        os.kill(p.pid, signal.SIGKILL)  # host-side failure: the rank simply dies
        p.join(10)
        assert _poll(lambda: a.stats()["edges"]["left"]["state"] == "free")
        a.addFromTensor(torch.ones(n))
        a.copyToTensor(out)
        assert torch.allclose(out, torch.full((n,), 2.0), atol=1e-4)
    finally:
        if p.is_alive():
            p.kill()
        a.close()


def test_dropped_frames_show_up_as_a_bounded_error(free_port):
    """A lost frame is a permanent offset of at most the frame's scale per element (the protocol has
    no sequence numbers, like the reference); the test checks the accounting and that later traffic
    is still applied."""
    n = 64
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))
    try:
        assert b.flush(10.0)
        b._b.inject_drop_frames("up", 1)
        a.addFromTensor(torch.ones(n))
        assert _poll(lambda: b.stats()["edges"]["up"]["dropped_by_injection"] == 1)
        assert a.flush(10.0) and b.flush(10.0)
        out = torch.zeros(n)
        b.copyToTensor(out)
        err = (out - 1).abs().max().item()
        assert 0 < err <= 1.0
        a.addFromTensor(torch.ones(n))
        assert _poll(lambda: abs((b.copyToTensor(out) - 2).abs().max().item() - err) < 1e-4)
    finally:
        b.cfg.rejoin = False
        b.close()
        a.close()


def test_master_leaves_and_a_child_takes_over_the_address(free_port):
    """The master closes; its two children notice, one of them becomes the master of host:port, the other joins
    below it, a newcomer can still join through host:port, and an update made afterwards reaches all of them."""
    n = 96
    torch.manual_seed(4)
    init = torch.randn(n)
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone())
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50)
    c = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50)
    e = None
    try:
        d0 = torch.randn(n) * 1e-2
        a.addFromTensor(d0)
        out = torch.zeros(n)
        for x in (b, c):
            assert _poll(lambda x=x: (x.copyToTensor(out) - (init + d0)).abs().max().item() < 1e-4)
        assert a.flush(10.0)
        a.close()
        assert _poll(lambda: sum(bool(x.stats()["master"]) for x in (b, c)) == 1), "exactly one child takes over"
        assert _poll(lambda: any(x.stats()["edges"]["up"]["state"] == "connected" for x in (b, c))), "the other joins below it"
        e = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin=False)  # a newcomer finds the tree
        d1 = torch.randn(n) * 1e-2
        b.addFromTensor(d1)
        for x in (b, c, e):
            assert _poll(lambda x=x: (x.copyToTensor(out) - (init + d0 + d1)).abs().max().item() < 1e-4), x.stats()
    finally:
        for x in (e, c, b):
            if x is not None:
                x.cfg.rejoin = False
                x.close()


def test_closing_while_a_node_rejoins_never_blocks(free_port):
    """Five nodes; one cuts its up connection; after a random short while all are closed, in either order.  Every
    close has to come back promptly whatever the re-joining node is doing at that moment (a close that set its
    stop flag between the supervisor's check and its wait used to leave the supervisor asleep for good)."""
    import random
    import socket

    from sharedtensor_b200 import _native

    core = _native.core()
    rnd = random.Random(7)
    n = 500

    def node():
        c = core.NodeConfig()
        c.rejoin_backoff_ms = 50
        return core.CpuNode(n, c)

    for it in range(40):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        init = torch.randn(n)
        nodes = [node()]
        nodes[0].start("127.0.0.1", port, init.data_ptr())
        for _ in range(4):
            nd = node()
            nd.start("127.0.0.1", port, 0)
            assert nd.wait_ready(20000)
            nodes.append(nd)
        nodes[rnd.choice([1, 2, 3, 4])].inject_sever(0)
        time.sleep(rnd.choice([0.0, 0.01, 0.05, 0.1, 0.3]))
        t0 = time.time()
        for nd in (reversed(nodes) if rnd.random() < 0.5 else nodes):
            nd.close()
        assert time.time() - t0 < 10.0, f"iteration {it}: closing five nodes took {time.time() - t0:.1f} s"


def test_churn_between_quiet_rounds_keeps_the_exact_sum(free_port):
    """Five replicas; every round all of them add, the tree goes quiet, one random replica (the master included)
    leaves, the survivors find each other again through host:port, and a newcomer joins.  Every replica holds
    initial + all updates after every step."""
    import random

    rnd = random.Random(3)
    torch.manual_seed(3)
    n = 256
    init = torch.randn(n)
    nodes = [sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone(), rejoin_backoff_ms=50)]
    for _ in range(4):
        nodes.append(sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50))
    expect = init.clone()
    out = torch.zeros(n)

    def converged():
        return max(float((nd.copyToTensor(out) - expect).abs().max()) for nd in nodes) < 2e-4

    def reformed():
        st = [nd.stats() for nd in nodes]
        return sum(bool(s["master"]) for s in st) == 1 and all(s["master"] or s["edges"]["up"]["state"] == "connected" for s in st)

    try:
        for r in range(8):
            for nd in nodes:
                d = torch.randn(n) * 1e-2
                nd.addFromTensor(d)
                expect += d
            assert _poll(converged), f"round {r}: updates"
            for nd in nodes:
                nd.flush(5.0)
            gone = nodes.pop(rnd.randrange(len(nodes)))
            gone.cfg.rejoin = False
            gone.close()
            assert _poll(reformed), f"round {r}: one master, everybody else attached"
            assert _poll(converged), f"round {r}: after the leave"
            nodes.append(sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50))
            assert _poll(converged), f"round {r}: after the join"
    finally:
        for nd in nodes:
            nd.cfg.rejoin = False
        for nd in reversed(nodes):
            nd.close()


@pytest.mark.parametrize("fmt", [{}, {"tcp_scale_mode": "block32"}, {"tcp_scale_mode": "block32", "tcp_bits": 8}],
                         ids=["tensor", "block32", "block32-8bit"])
def test_cut_edge_under_continuous_traffic_loses_nothing_on_loopback(free_port, fmt):
    """A child adds without pause while its up connection is cut five times.  What it had written before a cut still
    reaches the parent (the FIN follows the queued data), a frame whose write failed is taken back, the rest is
    carried over the re-join: both replicas end up with every update.  In every frame format of the TCP edges."""
    import threading

    n = 4096
    torch.manual_seed(0)
    init = torch.randn(n)
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone(), **fmt)
    b = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=20, **fmt)
    expect = init.clone()
    stop = threading.Event()

    def adder():
        g = torch.Generator().manual_seed(1)
        while not stop.is_set():
            d = torch.randn(n, generator=g) * 1e-2
            b.addFromTensor(d)
            expect.add_(d)
            time.sleep(0.002)

    t = threading.Thread(target=adder)
    t.start()
    try:
        for i in range(5):
            time.sleep(0.15)
            b._b.inject_sever("up")
            assert _poll(lambda: b.stats()["rejoins"] >= i + 1, timeout=10.0)
        stop.set()
        t.join()
        out = torch.zeros(n)
        assert _poll(lambda: float((a.copyToTensor(out) - expect).abs().max()) < 1e-4)
        assert _poll(lambda: float((b.copyToTensor(out) - expect).abs().max()) < 1e-4)
    finally:
        stop.set()
        t.join()
        b.cfg.rejoin = False
        b.close()
        a.close()


def test_abrupt_churn_under_traffic_leaves_the_survivors_in_agreement(free_port):
    """Replicas are closed without warning while updates keep coming in at random places, and newcomers join.  What a
    closed replica had not passed on is gone for everybody, so the sum is not checked; but once the churn stops, one
    tree is left and all its replicas hold the same values."""
    import random
    import threading

    rnd = random.Random(5)
    torch.manual_seed(5)
    n = 256

    def mk(t):
        return sharedtensor.createOrFetch("127.0.0.1", free_port, t, rejoin_backoff_ms=30)

    nodes = [mk(torch.randn(n))] + [mk(torch.zeros(n)) for _ in range(5)]
    lock = threading.Lock()
    stop = threading.Event()

    def adder():
        g = torch.Generator().manual_seed(6)
        while not stop.is_set():
            with lock:
                nd = rnd.choice(nodes)
            try:
                nd.addFromTensor(torch.randn(n, generator=g) * 1e-2)
            except RuntimeError:  # closed in between
                pass
            time.sleep(0.001)

    t = threading.Thread(target=adder)
    t.start()
    try:
        for _ in range(6):
            time.sleep(rnd.choice([0.02, 0.05, 0.1]))
            with lock:
                gone = nodes.pop(rnd.randrange(len(nodes)))
            gone.cfg.rejoin = False
            gone.close()
            time.sleep(rnd.choice([0.0, 0.05, 0.2]))
            with lock:
                nodes.append(mk(torch.zeros(n)))
        stop.set()
        t.join()
        ref, out = torch.zeros(n), torch.zeros(n)

        def settled():
            st = [nd.stats() for nd in nodes]
            if sum(bool(s["master"]) for s in st) != 1:
                return False
            if not all(s["master"] or s["edges"]["up"]["state"] == "connected" for s in st):
                return False
            nodes[0].copyToTensor(ref)
            return max(float((nd.copyToTensor(out) - ref).abs().max()) for nd in nodes) < 2e-4

        assert _poll(settled, timeout=40.0)
    finally:
        stop.set()
        t.join()
        for nd in nodes:
            nd.cfg.rejoin = False
        for nd in reversed(nodes):
            nd.close()
