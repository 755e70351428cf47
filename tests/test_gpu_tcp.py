"""Mixed trees: a GPU replica with TCP edges to CPU nodes of this framework and to the unmodified reference.
Frames on those edges are the reference's wire format, encoded and decoded on the device."""
import sys
import time
from pathlib import Path

import pytest
import torch

import sharedtensor

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _poll(fn, timeout=30.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if fn():
            return True
        time.sleep(0.05)
    return False


def _rel(st, expect, out):
    st.copyToTensor(out)
    if out.is_cuda:
        torch.cuda.synchronize()
    return ((out.cpu() - expect).norm() / expect.norm()).item()


def test_gpu_master_with_cpu_child_and_back(free_port):
    n = 3 * 4096 + 50
    torch.manual_seed(0)
    init = torch.randn(n)
    g = sharedtensor.createOrFetch("127.0.0.1", free_port, init.cuda())
    c = None
    try:
        c = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n))  # CPU node below a GPU master
        out_c, out_g = torch.zeros(n), torch.zeros(n, device="cuda")
        assert _poll(lambda: _rel(c, init, out_c) < 1e-5), "state streamed to the CPU child through the 1-bit codec"
        dg, dc = torch.randn(n) * 1e-2, torch.randn(n) * 1e-2
        g.addFromTensor(dg.cuda())
        c.addFromTensor(dc)
        expect = init + dg + dc
        assert _poll(lambda: _rel(c, expect, out_c) < 1e-5)
        assert _poll(lambda: _rel(g, expect, out_g) < 1e-5)
        s = g.stats()
        assert s["edges"]["left"]["transport"] == "tcp" and s["edges"]["left"]["frames_sent"] > 0
    finally:
        if c is not None:
            c.close()
        g.close()


def test_gpu_child_below_cpu_master(free_port):
    n = 5000
    torch.manual_seed(1)
    init = torch.randn(n)
    m = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    g = None
    try:
        g = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n, device="cuda"))
        out_g, out_m = torch.zeros(n, device="cuda"), torch.zeros(n)
        assert _rel(g, init, out_g) < 5e-3  # ready once the stream's scale fell by 2^-12
        d = torch.randn(n) * 1e-2
        g.addFromTensor(d.cuda())
        assert _poll(lambda: _rel(m, init + d, out_m) < 1e-5)
        assert _poll(lambda: _rel(g, init + d, out_g) < 1e-5)
        assert g.stats()["edges"]["up"]["transport"] == "tcp"
    finally:
        if g is not None:
            g.close()
        m.close()


def test_gpu_child_below_reference_master(free_port):
    sys.path.insert(0, str(ROOT / "baseline"))
    import build_ref
    from ref_worker import RefWorker

    if build_ref.build() is None:
        pytest.skip("reference source not available")
    n = 240
    torch.manual_seed(2)
    init = torch.randn(n)
    ref = RefWorker(n, call_timeout=60.0)
    g = None
    try:
        ref.call(op="create", host="127.0.0.1", port=free_port, n=n, values=init.tolist())
        g = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n, device="cuda"))
        d = torch.randn(n) * 1e-2
        g.addFromTensor(d.cuda())
        expect = init + d
        out_g = torch.zeros(n, device="cuda")
        assert _poll(lambda: (torch.tensor(ref.call(op="copy")["values"]) - expect).abs().max().item() < 2e-4)
        assert _poll(lambda: _rel(g, expect, out_g) < 1e-4)
    finally:
        if g is not None:
            g.close()
        ref.kill()


def test_gpu_child_rejoins_a_cpu_master_over_tcp(free_port):
    """Host-side failure on a TCP edge: the GPU replica's connection to its CPU parent is cut; it keeps what the
    parent had not been told (updates made during the outage included), joins again and both sides end up with
    every update."""
    n = 6000
    torch.manual_seed(2)
    init = torch.randn(n)
    m = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    g = None
    try:
        g = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n, device="cuda"), rejoin_backoff_ms=50)
        out_g, out_m = torch.zeros(n, device="cuda"), torch.zeros(n)
        d1, d2 = torch.randn(n) * 1e-2, torch.randn(n) * 1e-2
        g.addFromTensor(d1.cuda())
        assert _poll(lambda: _rel(m, init + d1, out_m) < 1e-5)
        g._b.inject_sever("up")
        for _ in range(5):
            g.addFromTensor((d2 / 5).cuda())
            time.sleep(0.02)
        assert _poll(lambda: g.stats()["rejoins"] == 1), g.stats()
        expect = init + d1 + d2
        assert _poll(lambda: _rel(m, expect, out_m) < 1e-5), _rel(m, expect, out_m)
        assert _poll(lambda: _rel(g, expect, out_g) < 1e-5), _rel(g, expect, out_g)
    finally:
        if g is not None:
            g.cfg.rejoin = False
            g.close()
        m.close()
