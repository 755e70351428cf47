"""The GPU replicas' protocol on the host model of a replica (tests/replica_model.py, the model the kernel tests
compare the device with): who is told what, forwarding through a chain, silence once everything has been said."""
import pytest
import torch

from replica_model import Oracle
from sharedtensor_b200 import _native


@pytest.fixture(scope="module")
def core():
    return _native.core()


def _run_chain(nodes, links, rounds, updates=None):
    """nodes: list of Oracle; links: list of (a, link of a, b, link of b).  Every round each node makes one pass, in
    order, and finds what its neighbours sent since its last pass.  Returns the frames sent per node and round."""
    inbox = {(i, l): [] for i, o in enumerate(nodes) for l in range(len(o.k))}
    peer = {}
    for a, la, b, lb in links:
        peer[(a, la)] = (b, lb)
        peer[(b, lb)] = (a, la)
    sent = [[0] * len(nodes) for _ in range(rounds)]
    for r in range(rounds):
        for i, d in (updates or {}).get(r, []):
            nodes[i].v += d
            nodes[i].mark()
        for i, o in enumerate(nodes):
            arrived = {l: inbox[(i, l)] for l in range(len(o.k))}
            for l in arrived:
                inbox[(i, l)] = []
            out = o.visit(arrived)
            for l, frame in out.items():
                inbox[peer[(i, l)]].append(frame)
                sent[r][i] += int(o.tiles_of(frame).sum())
    return sent


@pytest.mark.parametrize("bits", [1, 8])
def test_chain_forwards_and_falls_silent(core, bits):
    """A - B - C: updates made at both ends reach the other end through B, every replica ends at the exact sum to
    within the cut-off, and once everything has been said nobody sends any more."""
    n = 3 * 4096 + 57
    torch.manual_seed(3)
    A, B, C = Oracle(core, n, 32, 1, bits), Oracle(core, n, 32, 2, bits), Oracle(core, n, 32, 1, bits)
    init = torch.randn(n)
    for o in (A, B, C):     # a common start, mirrors included: nothing to say
        o.v = init.clone()
        o.k = [init.clone() for _ in o.k]
    da, dc = torch.randn(n), torch.randn(n) * 1e-2
    rounds = 80 if bits == 1 else 16
    sent = _run_chain([A, B, C], [(0, 0, 1, 0), (1, 1, 2, 0)], rounds, {1: [(0, da), (2, dc)]})
    assert sum(sent[0]) == 0, "nothing to say before the first update"
    expect = init + da + dc
    for o in (A, B, C):
        assert ((o.v - expect).norm() / expect.norm()).item() < 5e-6
    assert sum(sent[-1]) == 0 and sum(sent[-2]) == 0, "silent once everything has been said"


def test_a_receiver_does_not_answer(core):
    """B's values and its mirror of A differ in their low bits (B made an update earlier).  A then sends a large update:
    it moves B's values and B's mirror of A alike, the two sums round differently and the cut-off of many blocks moves,
    and B still sends nothing back; the update goes on to C in the same pass."""
    n = 8 * 4096
    torch.manual_seed(5)
    A, B, C = Oracle(core, n, 32, 1), Oracle(core, n, 32, 2), Oracle(core, n, 32, 1)
    init = torch.randn(n)
    for o in (A, B, C):
        o.v = init.clone()
        o.k = [init.clone() for _ in o.k]
    links = [(0, 0, 1, 0), (1, 1, 2, 0)]
    _run_chain([A, B, C], links, 12, {0: [(1, torch.randn(n))]})          # B's own update, drained
    assert not bool(B.dirty.any())
    assert bool((B.v != B.k[0]).any()), "values and mirror agree to the cut-off, not to the bit"
    # the whole tensor, old rule: how many blocks B would send back to A after receiving A's update
    da = torch.randn(n)
    A.v += da
    A.mark()
    fa = A.visit()[0]
    shadow = Oracle(core, n, 32, 2)
    shadow.v, shadow.k = B.v.clone(), [k.clone() for k in B.k]
    shadow.decode(0, fa)
    shadow.mark()
    assert int(shadow.encode(0)[1].ne(0).sum()) > 0, "the case is not vacuous: an unconditional answer would say something"
    out = B.visit({0: [fa]})
    assert 0 not in out, "B answers a frame it only received"
    assert 1 in out and int(B.tiles_of(out[1]).sum()) == n // 4096, "and passes it on to C at once"
    C.visit({0: [out[1]]})
    assert ((C.v - (B.v)).norm() / da.norm()).item() < 1e-2, "one 8-bit frame per hop delivers the update to under 1 %"


def test_mesh_group_one_hop_no_forwarding(core):
    """Four replicas as a fully connected group: one link and one mirror each, a member's frame goes to every peer and
    what arrives from the peers is not passed on.  Everybody ends at the exact sum, and a member that only received
    sends nothing."""
    n = 2 * 4096 + 300
    torch.manual_seed(9)
    members = [Oracle(core, n, 32, 1) for _ in range(4)]
    init = torch.randn(n)
    for o in members:
        o.v = init.clone()
        o.k = [init.clone()]
    deltas = {0: torch.randn(n), 2: torch.randn(n) * 1e-3}
    inbox = [[] for _ in members]
    sent = [0] * 4
    for r in range(12):
        if r == 1:
            for i, d in deltas.items():
                members[i].v += d
                members[i].mark()
        for i, o in enumerate(members):
            arrived, inbox[i] = inbox[i], []
            out = o.visit({0: arrived})
            if 0 in out:
                sent[i] += 1
                for j in range(4):
                    if j != i:
                        inbox[j].append(out[0])
    expect = init + deltas[0] + deltas[2]
    for o in members:
        assert ((o.v - expect).norm() / expect.norm()).item() < 5e-6
    assert sent[1] == 0 and sent[3] == 0 and sent[0] >= 3 and sent[2] >= 1
