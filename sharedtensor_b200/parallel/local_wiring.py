"""Wiring of several GPU replicas that live in ONE process (tests, single-GPU emulation of a tree).

Across processes the same rings are exchanged as file descriptors (see ``csrc/cuda/gpu_node.cpp``); here
both ends are in the same address space, so each side simply hands the other the address of its edge block.
Rounds of such replicas are launched one after the other on their streams; since no kernel ever waits for
a neighbour this is safe on a single GPU.
"""
from __future__ import annotations


def connect_local(a, b):
    """Creates one tree edge between replicas ``a`` and ``b``.  Returns ``(link_a, link_b)``."""
    la, lb = a.add_link(), b.add_link()
    if la < 0 or lb < 0:
        raise RuntimeError("no free link")
    ba, bb = a.alloc_edge_block(), b.alloc_edge_block()
    a.attach_peer(la, ba, b.edge_block_ptr(bb))
    b.attach_peer(lb, bb, a.edge_block_ptr(ba))
    return la, lb


def connect_mesh(replicas):
    """Fully connects the replicas as one mesh group: one link (one mirror) per replica, one ring pair per
    ordered pair of replicas.  Returns the link id of each replica."""
    links = [r.add_link() for r in replicas]
    blocks = {}
    for i, ri in enumerate(replicas):
        for j in range(len(replicas)):
            if i != j:
                blocks[(i, j)] = ri.alloc_edge_block()  # block at i that j stores into
    for i, ri in enumerate(replicas):
        for j, rj in enumerate(replicas):
            if i != j:
                ri.attach_peer(links[i], blocks[(i, j)], rj.edge_block_ptr(blocks[(j, i)]))
    return links
