"""T3: wire compatibility with the unmodified reference (built from its own C file, hosted by
baseline/ref_host.c, one process per replica)."""
import sys
import time
from pathlib import Path

import pytest
import torch

import sharedtensor

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "baseline"))
import build_ref  # noqa: E402
from ref_worker import RefWorker  # noqa: E402

pytestmark = pytest.mark.skipif(build_ref.build() is None, reason="reference source not available")


def _close_to(values, expect, tol):
    return (torch.tensor(values) - expect).abs().max().item() <= tol


def _poll(fn, timeout=20.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if fn():
            return True
        time.sleep(0.05)
    return False


def test_our_node_below_reference_master(free_port):
    n = 240
    torch.manual_seed(0)
    init = torch.randn(n)
    ref = RefWorker(n, call_timeout=60.0)
    ours = None
    try:
        ref.call(op="create", host="127.0.0.1", port=free_port, n=n, values=init.tolist())
        ours = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))
        out = torch.zeros(n)
        ours.copyToTensor(out)
        assert (out - init).abs().max() < 5e-3  # ready after the scale fell by 2^-12
        d_ours = torch.randn(n) * 1e-2
        d_ref = torch.randn(n) * 1e-2
        ours.addFromTensor(d_ours)
        ref.call(op="add", values=d_ref.tolist())
        expect = init + d_ours + d_ref
        # the reference sleeps one second whenever its residual is exactly zero (src/sharedtensor.c:163)
        assert _poll(lambda: _close_to(ref.call(op="copy")["values"], expect, 2e-4)), "reference replica"
        assert _poll(lambda: (ours.copyToTensor(out) - expect).abs().max().item() <= 2e-4), "our replica"
    finally:
        if ours is not None:
            ours.cfg.rejoin = False
            ours.close()
        ref.kill()


def test_reference_nodes_below_our_master_with_redirect(free_port):
    """Our master adopts two reference joiners and redirects a third one to its right child, which is
    a reference process: the 'N' + sockaddr_in reply must be understood by the reference client."""
    n = 64
    torch.manual_seed(1)
    init = torch.randn(n)
    ours = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    refs = [RefWorker(n, call_timeout=60.0) for _ in range(3)]
    try:
        # One phase at a time: the reference updates its arrays from several threads without any synchronisation
        # (src/sharedtensor.c:106-111 against 166-174), so a joiner that arrives while its reference parent is
        # still receiving its own state can lose increments for good.  Every replica is checked before the next
        # process joins or speaks.
        for r in refs:
            r.call(op="create", host="127.0.0.1", port=free_port, n=n)
            assert _poll(lambda r=r: _close_to(r.call(op="copy")["values"], init, 2e-4)), "state transfer to a reference joiner"
        st = ours.stats()
        assert st["edges"]["left"]["state"] == "connected" and st["edges"]["right"]["state"] == "connected"
        assert st["redirects"] == 1
        d = torch.randn(n) * 1e-2
        refs[2].call(op="add", values=d.tolist())  # the redirected grandchild speaks up
        expect = init + d
        out = torch.zeros(n)
        assert _poll(lambda: (ours.copyToTensor(out) - expect).abs().max().item() <= 2e-4)
        for r in refs:
            assert _poll(lambda r=r: _close_to(r.call(op="copy")["values"], expect, 2e-4))
    finally:
        ours.close()
        for r in refs:
            r.kill()


def test_our_node_survives_the_death_of_a_reference_master(free_port):
    """The reference master is killed (host-side failure).  Our child notices the closed connection, finds nobody at
    host:port, takes the address over and serves newcomers with the state it held."""
    n = 96
    torch.manual_seed(5)
    init = torch.randn(n)
    ref = RefWorker(n, call_timeout=60.0)
    ours = newcomer = None
    try:
        ref.call(op="create", host="127.0.0.1", port=free_port, n=n, values=init.tolist())
        ours = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin_backoff_ms=50)
        out = torch.zeros(n)
        assert _poll(lambda: (ours.copyToTensor(out) - init).abs().max().item() <= 2e-4)
        ref.kill()
        assert _poll(lambda: bool(ours.stats()["master"])), ours.stats()
        d = torch.randn(n) * 1e-2
        ours.addFromTensor(d)
        newcomer = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin=False)
        assert _poll(lambda: (newcomer.copyToTensor(out) - (init + d)).abs().max().item() <= 2e-4)
    finally:
        for x in (newcomer, ours):
            if x is not None:
                x.cfg.rejoin = False
                x.close()
        ref.kill()
