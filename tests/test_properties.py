"""T1: sum consistency as a property.  For random tree sizes, join orders interleaved with updates, update
magnitudes and wire formats, every replica ends at initial + sum of all deltas."""
import socket
import time

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

import sharedtensor


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@settings(max_examples=6, deadline=None, suppress_health_check=list(HealthCheck))
@given(n_nodes=st.integers(2, 7), n=st.sampled_from([1, 33, 240, 1025]), mode=st.sampled_from(["tensor", "block32", "block256", "block32/8", "block256/8"]),
       schedule=st.lists(st.tuples(st.integers(0, 6), st.floats(1e-4, 1.0)), min_size=3, max_size=12), seed=st.integers(0, 10_000))
def test_every_replica_reaches_the_exact_sum(n_nodes, n, mode, schedule, seed):
    torch.manual_seed(seed)
    port = _port()
    init = torch.randn(n)
    expect = init.double().clone()
    kw = {"tcp_scale_mode": mode}
    if mode.endswith("/8"):   # block scales with 8-bit integer frames
        kw = {"tcp_scale_mode": mode[:-2], "tcp_bits": 8}
    nodes = [sharedtensor.createOrFetch("127.0.0.1", port, init, **kw)]
    try:
        joins_left = n_nodes - 1
        for who, mag in schedule:
            if joins_left and who % 2 == 0:  # joins interleave with updates: late joiners must receive history
                nodes.append(sharedtensor.createOrFetch("127.0.0.1", port, torch.zeros(n), **kw))
                joins_left -= 1
            d = torch.randn(n) * mag
            nodes[who % len(nodes)].addFromTensor(d)
            expect += d.double()
        while joins_left:
            nodes.append(sharedtensor.createOrFetch("127.0.0.1", port, torch.zeros(n), **kw))
            joins_left -= 1
        out = torch.zeros(n)
        scale = max(1.0, float(expect.abs().max()))
        deadline = time.time() + 60
        worst = None
        while time.time() < deadline:
            worst = 0.0
            for nd in nodes:
                nd.copyToTensor(out)
                worst = max(worst, float((out.double() - expect).abs().max()) / scale)
            if worst < 5e-5:
                break
            time.sleep(0.02)
        assert worst < 5e-5, worst
    finally:
        for nd in reversed(nodes):
            nd.close()
