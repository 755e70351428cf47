"""T2: the tree-join wire protocol, byte for byte (reference src/sharedtensor.c:192-242, 244-332)."""
import math
import socket
import struct
import time

import torch

import sharedtensor


def _connect(port):
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.settimeout(5)
    return s


def _recv_exact(s, n):
    buf = b""
    while len(buf) < n:
        chunk = s.recv(n - len(buf))
        assert chunk, "peer closed"
        buf += chunk
    return buf


def test_handshake_bytes_and_redirect_alternation(free_port):
    master = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.arange(8.0))
    try:
        # the first two inbound connections are adopted: exactly one byte 'Y', then frames
        c1 = _connect(free_port)
        assert _recv_exact(c1, 1) == b"Y"
        c2 = _connect(free_port)
        assert _recv_exact(c2, 1) == b"Y"
        a1 = c1.getsockname()
        a2 = c2.getsockname()
        # every later one gets 'N' + a raw 16-byte sockaddr_in, alternating right, left, right
        got = []
        for _ in range(3):
            c = _connect(free_port)
            msg = _recv_exact(c, 17)
            assert msg[:1] == b"N"
            family, port_be = struct.unpack("<H", msg[1:3])[0], struct.unpack(">H", msg[3:5])[0]
            ip = socket.inet_ntoa(msg[5:9])
            assert family == socket.AF_INET
            assert msg[9:17] == b"\0" * 8
            got.append((ip, port_be))
            assert c.recv(1) == b""  # server closes after the redirect
            c.close()
        assert got == [a2, a1, a2], "redirect targets are the children's own source addresses: right, left, right"
        # the adopted connections carry tensor-scale frames: 4-byte scale + ceil(8/8) sign bytes
        frame = _recv_exact(c1, 5)
        scale = struct.unpack("<f", frame[:4])[0]
        assert scale == 4.0  # rms of 0..7 is 4.18 -> 2^2
        assert frame[4] == 0b00000001  # only element 0 (value 0) is "not positive"
        c1.close()
        c2.close()
    finally:
        master.close()


def test_tree_shape_of_sequential_joins(free_port):
    """Joiner 1 -> master.left, 2 -> master.right, 3 -> under right, 4 -> under left (2.2 of the protocol)."""
    nodes = [sharedtensor.createOrFetch("127.0.0.1", free_port, torch.arange(4.0) + 1)]
    try:
        for _ in range(4):
            nodes.append(sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(4)))
        st = [n.stats() for n in nodes]
        m = st[0]
        assert m["master"] and m["edges"]["up"]["state"] == "free"
        assert m["edges"]["left"]["peer"] == st[1]["listen_addr"]
        assert m["edges"]["right"]["peer"] == st[2]["listen_addr"]
        assert m["redirects"] == 2
        # third joiner was sent to the right child first, fourth to the left child
        assert st[2]["edges"]["left"]["peer"] == st[3]["listen_addr"]
        assert st[1]["edges"]["left"]["peer"] == st[4]["listen_addr"]
        out = torch.zeros(4)
        for n in nodes:
            n.copyToTensor(out)
            assert torch.allclose(out, torch.arange(4.0) + 1, atol=2e-3)  # ready once the stream's scale fell by 2^-12
    finally:
        for n in reversed(nodes):
            n.cfg.rejoin = False
        for n in reversed(nodes):
            n.close()


def test_late_joiner_receives_state_and_all_zero_state_does_not_hang(free_port):
    master = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(16))
    try:
        t0 = time.time()
        j = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.ones(16))  # joiner's values are ignored
        assert time.time() - t0 < 5, "an all-zero shared state must not block the joiner (the reference spins forever)"
        out = torch.ones(16)
        j.copyToTensor(out)
        assert torch.equal(out, torch.zeros(16))
        j.close()
    finally:
        master.close()


def test_size_mismatch_is_an_error(free_port):
    st = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(4, 5, 6, 2))
    try:
        import pytest

        with pytest.raises(ValueError, match="Not the right size!"):
            st.addFromTensor(torch.zeros(10))
        with pytest.raises(ValueError, match="Not the right size!"):
            st.copyToTensor(torch.zeros(241))
        with pytest.raises(TypeError):
            st.addFromTensor(torch.zeros(240, dtype=torch.float64))
        st.addFromTensor(torch.ones(240))
        out = torch.empty(4, 5, 6, 2)
        st.copyToTensor(out)
        assert torch.equal(out, torch.ones(4, 5, 6, 2))
    finally:
        st.close()


def test_frames_of_the_reference_binary_decode_with_our_codec(free_port):
    """T0/T2 against the real thing: a raw socket joins an unmodified reference master, gets the one byte 'Y', and the
    frames the reference then streams (4-byte scale + ceil(n/8) sign bytes, src/sharedtensor.c:156-177), decoded by
    our codec into a zeroed buffer, add up to the reference's values."""
    import sys
    from pathlib import Path

    import pytest

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "baseline"))
    import build_ref
    from ref_worker import RefWorker

    from sharedtensor_b200 import _native

    if build_ref.build() is None:
        pytest.skip("reference source not available")
    core = _native.core()
    n = 240
    torch.manual_seed(3)
    init = torch.randn(n)
    ref = RefWorker(n, call_timeout=60.0)
    try:
        ref.call(op="create", host="127.0.0.1", port=free_port, n=n, values=init.tolist())
        c = _connect(free_port)
        assert _recv_exact(c, 1) == b"Y"
        got = torch.zeros(n)
        nbytes = (n + 7) // 8
        prev_scale = None
        err = float("inf")
        for i in range(4000):
            frame = _recv_exact(c, 4 + nbytes)
            scale = struct.unpack("<f", frame[:4])[0]
            assert scale >= 0.0 and scale == scale
            if scale > 0.0:  # every scale is a power of two, and the stream's scales never grow
                m, _ = math.frexp(scale)
                assert m == 0.5
                assert prev_scale is None or scale <= prev_scale
                prev_scale = scale
            bits = torch.frombuffer(bytearray(frame[4:]), dtype=torch.uint8)
            core.decode_tensor_add(bits.data_ptr(), scale, n, got.data_ptr(), 0)
            err = (got - init).abs().max().item()
            if err <= 1e-3:
                break
        assert err <= 1e-3, f"after {i + 1} frames the decoded stream is still {err} away"
        c.close()
    finally:
        ref.kill()


def test_garbage_from_a_peer_costs_only_that_edge(free_port):
    """A connection that is adopted and then sends a frame with a NaN scale, a negative scale, or nothing at all
    before it closes: the node drops that edge, frees the slot and keeps serving (the reference adds whatever
    arrives into its arrays, src/sharedtensor.c:106-127, or exits)."""
    n = 64
    init = torch.arange(float(n))
    master = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone())
    try:
        nbytes = (n + 7) // 8
        for bad in (struct.pack("<f", float("nan")), struct.pack("<f", -1.0), None):
            c = _connect(free_port)
            assert _recv_exact(c, 1) == b"Y"
            if bad is not None:
                c.sendall(bad + b"\xff" * nbytes)
                deadline = time.time() + 10
                while time.time() < deadline and master.stats()["edges"]["left"]["state"] == "connected":
                    time.sleep(0.02)
            c.close()
            deadline = time.time() + 10
            while time.time() < deadline and master.stats()["edges"]["left"]["state"] != "free":
                time.sleep(0.02)
            assert master.stats()["edges"]["left"]["state"] == "free"
        out = torch.zeros(n)
        master.copyToTensor(out)
        assert torch.equal(out, init), "nothing of the garbage reached the values"
        child = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.zeros(n), rejoin=False)
        child.copyToTensor(out)
        assert torch.allclose(out, init, atol=1e-1)
        child.close()
    finally:
        master.close()


def test_garbage_scale_code_in_block_mode_costs_only_that_edge(free_port):
    """The same in block-scale mode: a frame whose scale bytes hold the code no encoder emits (255, which would
    decode to infinity) ends that edge and leaves the values alone."""
    n = 64
    init = torch.arange(float(n))
    master = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone(), tcp_scale_mode="block32")
    try:
        c = _connect(free_port)
        assert _recv_exact(c, 1) == b"Y"
        c.sendall(b"\xff" * (n // 32) + b"\x00" * (4 * (n // 32)))   # scale bytes, then sign words
        deadline = time.time() + 10
        while time.time() < deadline and master.stats()["edges"]["left"]["state"] != "free":
            time.sleep(0.02)
        assert master.stats()["edges"]["left"]["state"] == "free"
        c.close()
        out = torch.zeros(n)
        master.copyToTensor(out)
        assert torch.equal(out, init), "nothing of the garbage reached the values"
    finally:
        master.close()


def test_garbage_scale_code_in_eight_bit_mode_costs_only_that_edge(free_port):
    """... and with 8-bit integer frames (scale bytes, then one code byte per element)."""
    n = 64
    init = torch.arange(float(n))
    master = sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone(), tcp_scale_mode="block32", tcp_bits=8)
    try:
        c = _connect(free_port)
        assert _recv_exact(c, 1) == b"Y"
        c.sendall(b"\xff" * (n // 32) + b"\x81" * n)
        deadline = time.time() + 10
        while time.time() < deadline and master.stats()["edges"]["left"]["state"] != "free":
            time.sleep(0.02)
        assert master.stats()["edges"]["left"]["state"] == "free"
        c.close()
        out = torch.zeros(n)
        master.copyToTensor(out)
        assert torch.equal(out, init), "nothing of the garbage reached the values"
    finally:
        master.close()


def test_simultaneous_founders_end_up_in_one_tree(free_port):
    """Six callers reach createOrFetch at the same moment with nobody serving host:port yet: exactly one becomes the
    master, the others lose the race for the address, try again and join below it with the master's values."""
    import threading

    n = 64
    for _ in range(3):
        nodes, errs = [None] * 6, []

        def go(i):
            try:
                nodes[i] = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.full((n,), float(i + 1)), rejoin=False)
            except Exception as e:  # noqa: BLE001
                errs.append(repr(e))

        ts = [threading.Thread(target=go, args=(i,)) for i in range(6)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        try:
            assert not errs, errs
            masters = [i for i, x in enumerate(nodes) if x.stats()["master"]]
            assert len(masters) == 1
            want = float(masters[0] + 1)
            out = torch.zeros(n)
            for x in nodes:
                deadline = time.time() + 10
                while time.time() < deadline and abs(float(x.copyToTensor(out).mean()) - want) > 1e-3:
                    time.sleep(0.02)
                assert abs(float(out.mean()) - want) <= 1e-3
        finally:
            for x in reversed([x for x in nodes if x is not None]):
                x.close()
        time.sleep(0.1)
