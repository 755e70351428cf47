"""T5: every sm_100a kernel against the host codec / a plain PyTorch fp32 statement of the same operation.
Two or three replicas live in one process on one GPU and are wired to each other directly."""
import pytest
import torch

from sharedtensor_b200 import _native
from sharedtensor_b200.parallel.local_wiring import connect_local, connect_mesh

from replica_model import Oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cu():
    mod = _native.cuda()
    assert torch.cuda.is_available()
    return mod


@pytest.fixture(scope="module")
def core():
    return _native.core()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _replica(cu, n, block=32, slots=4, shareable=True, rel_bits=22, bits=8, deadline_us=1000, window=0):
    cfg = cu.GpuConfig()
    cfg.window_tiles = window
    cfg.bits = bits
    cfg.poll_deadline_us = deadline_us
    cfg.block = block
    cfg.ring_slots = slots
    cfg.shareable = shareable
    cfg.rel_bits = rel_bits
    return cu.GpuReplica(0, n, cfg)


def _read(ptr_fn, n, rep):
    out = torch.empty(n, device="cuda")
    rep.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    return out


def _dev_view(ptr, n):
    """Copies n floats from a raw device address."""
    out = torch.empty(n, device="cuda")
    _native.cuda().memcpy_d2d(out.data_ptr(), ptr, n * 4)
    torch.cuda.synchronize()
    return out


# --------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 4097, 1 << 20, (1 << 22) + 5])
def test_snapshot_add_sub_add(cu, n):
    torch.manual_seed(n)
    rep = _replica(cu, n)
    init = torch.randn(n, device="cuda")
    rep.load_values(init.data_ptr(), _stream())
    out = torch.empty(n, device="cuda")
    rep.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert torch.equal(out, init)
    d = torch.randn(n, device="cuda") * 1e-2
    rep.add(d.data_ptr(), _stream())
    rep.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert torch.equal(out, init + d)
    new, old = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    rep.sub_add(new.data_ptr(), old.data_ptr(), _stream())
    rep.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert torch.equal(out, (init + d) + (new - old))
    bf = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rep.snapshot_bf16(bf.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert torch.equal(bf, out.to(torch.bfloat16))


def test_unaligned_user_tensors(cu):
    n = 10001
    rep = _replica(cu, n)
    base = torch.randn(n + 3, device="cuda")
    d = base[1:n + 1]  # 4-byte aligned only
    assert d.data_ptr() % 16 != 0
    rep.add(d.data_ptr(), _stream())
    outbuf = torch.zeros(n + 3, device="cuda")
    out = outbuf[3:n + 3]
    rep.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert torch.equal(out, d)


def test_atomic_add_kernels(cu):
    n = 100003
    torch.manual_seed(1)
    v = torch.randn(n, device="cuda")
    d = torch.randn(n, device="cuda")
    ref = v + d
    cu.add(v.data_ptr(), d.data_ptr(), n, True, _stream())
    torch.cuda.synchronize()
    assert torch.equal(v, ref)
    a, b = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    ref = v + (a - b)
    cu.sub_add(v.data_ptr(), a.data_ptr(), b.data_ptr(), n, True, _stream())
    torch.cuda.synchronize()
    assert torch.equal(v, ref)
    g16 = torch.randn(n, device="cuda").to(torch.bfloat16)
    ref = v + (-0.5) * g16.float()
    cu.add_scaled_bf16(v.data_ptr(), g16.data_ptr(), -0.5, n, True, _stream())
    torch.cuda.synchronize()
    assert torch.equal(v, ref)


def test_table_scales(cu):
    torch.manual_seed(3)
    sizes = [5, 70000, 1, 300000, 4096, 0, 65536]
    offs = [0]
    for s in sizes:
        offs.append(offs[-1] + s)
    total = offs[-1]
    x = torch.cat([torch.randn(s, device="cuda") * (10.0 ** (i - 3)) for i, s in enumerate(sizes)])
    off_d = torch.tensor(offs, dtype=torch.int64, device="cuda")
    scratch = torch.empty(cu.table_scales_scratch_doubles(len(sizes), total), dtype=torch.float64, device="cuda")
    out = torch.empty(len(sizes), dtype=torch.float64, device="cuda")
    exps = torch.empty(len(sizes), dtype=torch.int8, device="cuda")
    cu.table_scales(x.data_ptr(), off_d.data_ptr(), len(sizes), total, scratch.data_ptr(), out.data_ptr(), exps.data_ptr(), _stream())
    torch.cuda.synchronize()
    for i, s in enumerate(sizes):
        seg = x[offs[i]:offs[i + 1]].double()
        ref = float((seg * seg).sum())
        assert abs(float(out[i]) - ref) <= 1e-9 * max(ref, 1e-30)
        if s:
            rms = (ref / s) ** 0.5
            import math

            assert int(exps[i]) == math.floor(math.log2(rms))
        else:
            assert int(exps[i]) == -128


def test_sample_sqerr_and_delay(cu):
    n = 1 << 20
    a = torch.randn(n, device="cuda")
    stride = 16
    b = a[::stride].clone() + 0.5
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    cu.sample_sqerr(a.data_ptr(), stride, b.data_ptr(), b.numel(), out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert abs(float(out[0]) - 0.25 * b.numel()) < 1e-3 * b.numel()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    cu.delay(2_000_000, _stream())
    e1.record()
    torch.cuda.synchronize()
    assert 1.9 <= e0.elapsed_time(e1) < 10.0


# --------------------------------------------------------------------------------------------------
def _state(cu, rep, link):
    n = rep.size()
    v = torch.empty(n, device="cuda")
    rep.snapshot(v.data_ptr(), _stream())
    torch.cuda.synchronize()
    k = _dev_view(rep.mirror_ptr(link), n)
    return v.cpu(), k.cpu()


def _dev_bytes(ptr, nbytes):
    out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _native.cuda().memcpy_d2d(out.data_ptr(), ptr, nbytes)
    torch.cuda.synchronize()
    return out.cpu()


def _cases():
    out = []
    for bits in (1, 2, 4, 8):
        for block in ((32, 64, 128, 256, 1024, 2048, 4096) if bits in (1, 8) else (32, 256, 4096)):
            for n in (1, 31, 4096, 4097, 10000, 3 * 4096 + 77):
                out.append((bits, block, n))
    return out


@pytest.mark.parametrize("bits,block,n", _cases())
def test_round_bit_exact_two_replicas(cu, core, bits, block, n):
    """A -> B streaming of A's state plus updates on both sides, compared bit for bit with the host codec: values,
    mirrors, and the code words and scale bytes in the ring slots."""
    torch.manual_seed(n * 13 + block + bits)
    A, B = _replica(cu, n, block, bits=bits), _replica(cu, n, block, bits=bits)
    la, lb = connect_local(A, B)
    oa, ob = Oracle(core, n, block, 1, bits), Oracle(core, n, block, 1, bits)
    init = torch.randn(n) * torch.logspace(-2, 1, n)
    oa.v = init.clone()
    A.load_values(init.cuda().data_ptr(), _stream())
    lay = B.edge_layout()
    pb = bits * 512 + max(16, 4096 // block)
    slots = 4
    sent_a = 0  # frames A has produced so far
    rounds = 24 if bits == 1 else 10
    for it in range(rounds):
        if it in (3, 7):
            da, db = torch.randn(n) * 1e-2, torch.randn(n) * 1e-1
            oa.v += da
            ob.v += db
            oa.mark()
            ob.mark()
            A.add(da.cuda().data_ptr(), _stream())
            B.add(db.cuda().data_ptr(), _stream())
            torch.cuda.synchronize()
        # A's sweep: receives B's previous frame (if any), sends; then B's sweep
        A.round()
        A.sync()
        # host model, same order: A decodes what B sent last time, encodes
        if it > 0:
            oa.decode(0, frame_b)
        frame_a = oa.encode(0)
        words, sc, loud = oa.payload_of_tile(frame_a, 0)
        if bool(sc.any()):
            # what A just pushed into B's ring: tile 0 of the frame, in the slot the tile's sequence number selects
            raw = _dev_bytes(B.edge_block_ptr(0) + lay["off_payload"] + ((sent_a % slots) * B.tiles() + 0) * pb, pb)
            got_words = raw[:bits * 512].view(torch.int32).reshape(128, bits)
            assert torch.equal(got_words[loud], words.reshape(128, bits)[loud]), f"code words differ in round {it}"
            assert torch.equal(raw[bits * 512:bits * 512 + sc.numel()], sc), f"scale bytes differ in round {it}"
            sent_a += 1
        B.round()
        B.sync()
        ob.decode(0, frame_a)
        frame_b = ob.encode(0)
        va, ka = _state(cu, A, la)
        vb, kb = _state(cu, B, lb)
        assert torch.equal(va, oa.v), f"A values differ in round {it}"
        assert torch.equal(ka, oa.k[0]), f"A mirror differs in round {it}"
        assert torch.equal(vb, ob.v), f"B values differ in round {it}"
        assert torch.equal(kb, ob.k[0]), f"B mirror differs in round {it}"
    st = A.status()
    assert st[5] == 0, "no error bits"
    assert A.check_guards() == 0 and B.check_guards() == 0


@pytest.mark.parametrize("bits", [1, 8])
def test_one_frame_of_eight_bits_delivers_an_update(cu, bits):
    """A fresh N(0,1) update: relative error after one 8-bit frame is under one percent; sign frames need many."""
    n = 64 * 4096
    torch.manual_seed(2)
    A, B = _replica(cu, n, bits=bits), _replica(cu, n, bits=bits)
    connect_local(A, B)
    d = torch.randn(n, device="cuda")
    A.add(d.data_ptr(), _stream())
    torch.cuda.synchronize()
    A.round()
    A.sync()
    B.round()
    B.sync()
    out = torch.empty(n, device="cuda")
    B.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    rel = ((out - d).norm() / d.norm()).item()
    if bits == 8:
        assert rel < 1e-2, rel
    else:
        assert rel > 0.3, rel


def test_a_received_frame_is_not_answered(cu):
    """A frame moves the receiver's values and its mirror of the sender by the same step, so it leaves nothing to say
    to the sender; the two additions round differently and the cut-off moves with the values, which must not make
    the receiver send a frame back for every tile it received."""
    n = 16 * 4096
    torch.manual_seed(31)
    A, B = _replica(cu, n), _replica(cu, n)
    connect_local(A, B)
    names = cu.status_names()
    i_sent = names.index("frames_sent")
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    db = torch.randn(n, device="cuda")
    B.add(db.data_ptr(), _stream())     # B's values and its mirror of A differ in their low bits from here on
    torch.cuda.synchronize()
    for _ in range(12):
        A.round(); A.sync(); B.round(); B.sync()
    da = torch.randn(n, device="cuda")  # large enough to move the cut-off of many blocks
    A.add(da.data_ptr(), _stream())
    torch.cuda.synchronize()
    sent_b = B.status()[i_sent]
    for _ in range(6):
        A.round(); A.sync(); B.round(); B.sync()
    assert B.status()[i_sent] == sent_b, "the receiver answered frames it had only received"
    out = torch.empty(n, device="cuda")
    expect = init + db + da
    for r in (A, B):
        r.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        assert ((out - expect).norm() / expect.norm()).item() < 1e-5


def test_several_passes_in_one_launch(cu):
    """One launch can make several passes over the tensor: the second and third frame of an update follow the first
    without the host, and a receiver's launch takes all of them."""
    n = 9 * 4096 + 100
    torch.manual_seed(17)
    A, B = _replica(cu, n), _replica(cu, n)
    connect_local(A, B)
    names = cu.status_names()
    d = torch.randn(n, device="cuda")
    A.add(d.data_ptr(), _stream())
    torch.cuda.synchronize()
    before = A.launches()
    A.round(True, True, 6)
    A.sync()
    assert A.launches() - before == 1
    st = A.status()
    sent = st[names.index("frames_sent")]
    assert sent >= 3 * A.tiles() - 3, "it takes three frames per tile to bring fp32 values below the cut-off"
    B.round(True, True, 6)
    B.sync()
    A.round()
    A.sync()
    assert A.status()[names.index("frames_sent")] == sent, "the one launch had said everything"
    out = torch.empty(n, device="cuda")
    B.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert ((out - d).norm() / d.norm()).item() < 1e-6
    assert A.status()[names.index("errors")] == 0 and B.status()[names.index("errors")] == 0


def test_several_frames_per_round_and_ring_full(cu, core):
    """The sender runs ahead: the receiver takes up to three frames per sweep in order; once the ring is full the
    sender skips (nothing is lost, the residual simply stays) and counts it."""
    n, block, slots, bits = 2 * 4096 + 5, 32, 4, 1
    torch.manual_seed(7)
    A, B = _replica(cu, n, block, slots, bits=bits), _replica(cu, n, block, slots, bits=bits)
    la, lb = connect_local(A, B)
    oa, ob = Oracle(core, n, block, 1, bits), Oracle(core, n, block, 1, bits)
    init = torch.randn(n)
    oa.v = init.clone()
    A.load_values(init.cuda().data_ptr(), _stream())
    frames = []
    for _ in range(slots + 3):  # three rounds more than the ring holds
        A.round()
        A.sync()
    for _ in range(slots):
        frames.append(oa.encode(0))
    va, ka = _state(cu, A, la)
    assert torch.equal(ka, oa.k[0]), "only ring_slots frames were produced"
    st = A.status()
    names = cu.status_names()
    assert st[names.index("blocked_no_credit")] == 3 * A.tiles()
    assert st[names.index("frames_sent")] == slots * A.tiles()
    # B drains up to three frames per sweep, in order
    taken = 0
    for take in (3, 1):
        B.round(True, False)  # receiver-only rounds
        B.sync()
        ob.decode(0, frames[taken:taken + take])
        taken += take
        vb, kb = _state(cu, B, lb)
        assert torch.equal(vb, ob.v) and torch.equal(kb, ob.k[0])
    # credits are back: A can send again
    A.round()
    A.sync()
    oa.encode(0)
    va, ka = _state(cu, A, la)
    assert torch.equal(ka, oa.k[0])
    assert A.check_guards() == 0 and B.check_guards() == 0


@pytest.mark.parametrize("bits", [1, 8])
def test_unacknowledged_frames_are_taken_back(cu, bits):
    """A sender whose neighbour never consumed (never acknowledged) two frames takes their steps off its mirror again
    and its ring counters fall back, so that what the frames said counts as not yet told."""
    n = 3 * 4096 + 70
    torch.manual_seed(21)
    A, B = _replica(cu, n, bits=bits), _replica(cu, n, bits=bits)
    la, lb = connect_local(A, B)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    for _ in range(2):
        A.round()
        A.sync()
    k = _dev_view(A.mirror_ptr(la), n)
    assert float(k.abs().max()) > 0.0
    assert A.unsend_unacknowledged(0) == 2 * A.tiles()
    k = _dev_view(A.mirror_ptr(la), n)
    assert float(k.abs().max()) == 0.0, "the mirror is back where it was before the two frames"
    names = cu.status_names()
    sent_before = A.status()[names.index("frames_sent")]
    A.round()
    A.sync()
    assert A.status()[names.index("frames_sent")] == sent_before + A.tiles(), "the ring has room again"
    assert A.check_guards() == 0 and B.check_guards() == 0


def test_updates_commute_with_rounds(cu):
    """One stream adds 200 deltas while the engine threads run rounds: both replicas end at the exact fp32 sum
    (every delta is a multiple of 2^-10 and all partial sums are exactly representable, so any order gives it)."""
    n = 40 * 4096 + 11
    torch.manual_seed(9)
    A, B = _replica(cu, n), _replica(cu, n)
    connect_local(A, B)
    init = torch.randint(-1000, 1000, (n,), device="cuda").float() / 16.0
    A.load_values(init.data_ptr(), _stream())
    A.start_engine()
    B.start_engine()
    side = torch.cuda.Stream()
    deltas = [torch.randint(-64, 64, (n,), device="cuda").float() / 1024.0 for _ in range(8)]
    expect = init.clone()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for i in range(200):
            (A if i % 2 == 0 else B).add(deltas[i % 8].data_ptr(), side.cuda_stream)
    for i in range(200):
        expect += deltas[i % 8]
    side.synchronize()
    import time

    out = torch.empty(n, device="cuda")
    ok = False
    deadline = time.time() + 20
    while time.time() < deadline and not ok:
        ok = True
        for r in (A, B):
            r.snapshot(out.data_ptr(), _stream())
            torch.cuda.synchronize()
            ok = ok and torch.equal(out, expect)
        time.sleep(0.01)
    A.stop_engine()
    B.stop_engine()
    assert ok, float((out - expect).abs().max())
    assert A.status()[5] == 0 and B.status()[5] == 0
    assert A.check_guards() == 0 and B.check_guards() == 0


def test_windowed_launches_cover_the_tensor(cu):
    """A tensor that is covered in several launches per pass (windows of 16 tiles here): manual rounds make whole
    passes, the engine thread goes from window to window, and both see every tile."""
    n = 40 * 4096 + 11
    torch.manual_seed(31)
    A, B = _replica(cu, n, window=16), _replica(cu, n, window=16)
    connect_local(A, B)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    out = torch.empty(n, device="cuda")
    for _ in range(4):
        A.round()
        A.sync()
        B.round()
        B.sync()
    B.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert ((out - init).norm() / init.norm()).item() < 1e-5
    names = cu.status_names()
    quiet = False
    for _ in range(10):     # the refinements die down: a pass that finds nothing to do on either side
        A.round()
        A.sync()
        B.round()
        B.sync()
        sa, sb = A.status(), B.status()
        if all(s[names.index(k)] == 0 for s in (sa, sb) for k in ("last_work_count", "pending_tiles")):
            quiet = True
            break
    assert quiet, "the counters of a whole pass (all windows) are zero once nothing moves"
    assert A.status()[names.index("tiles_processed")] >= A.tiles()
    A.start_engine()
    B.start_engine()
    d = torch.randn(n, device="cuda")
    B.add(d.data_ptr(), _stream())
    import time

    deadline = time.time() + 10
    ok = False
    while time.time() < deadline and not ok:
        A.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        ok = ((out - (init + d)).norm() / init.norm()).item() < 1e-5
        time.sleep(0.005)
    A.stop_engine()
    B.stop_engine()
    assert ok
    assert A.status()[5] == 0 and B.status()[5] == 0


def test_join_while_the_default_stream_is_busy(cu):
    """Links, edge blocks and sequence counters are created while the legacy default stream holds a long queue:
    they are zeroed on the streams that use them, not behind that queue, so the first rounds see clean memory and
    nothing is wiped after the fact."""
    n = 3 * 4096 + 5
    torch.manual_seed(12)
    A, B = _replica(cu, n), _replica(cu, n)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    torch.cuda.synchronize()
    for _ in range(60):
        cu.delay(5_000_000, _stream())          # 0.3 s of queued work on the default stream
    side = torch.cuda.Stream()
    connect_local(A, B)
    out = torch.empty(n, device="cuda")
    for _ in range(6):
        A.round()
        A.sync()
        B.round()
        B.sync()
    B.snapshot(out.data_ptr(), side.cuda_stream)
    side.synchronize()
    still_busy = not torch.cuda.current_stream().query()
    assert ((out - init).norm() / init.norm()).item() < 1e-5
    assert still_busy, "the default stream was meant to be busy for the whole test"
    torch.cuda.synchronize()
    for _ in range(3):                           # nothing is zeroed late: the replicas stay where they are
        A.round()
        A.sync()
        B.round()
        B.sync()
    B.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert ((out - init).norm() / init.norm()).item() < 1e-5
    assert A.status()[5] == 0 and B.status()[5] == 0


def test_bounded_wait_runs_out_and_the_replica_recovers(cu):
    """The copy barrier of one tile is told to expect more bytes than are copied: the group that owns the tile gives
    up after the configured limit, stores nothing of that tile, reports it, and the next ordinary round converges."""
    n = 2 * 4096
    torch.manual_seed(3)
    A, B = _replica(cu, n, deadline_us=200), _replica(cu, n, deadline_us=200)
    la, lb = connect_local(A, B)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    A.set_test_stall_tile(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cs = torch.cuda.ExternalStream(A.comm_stream())
    e0.record(cs)
    A.round()
    e1.record(cs)
    A.sync()
    assert e0.elapsed_time(e1) < 50.0, "the kernel returned"
    names = cu.status_names()
    st = A.status()
    assert st[names.index("wait_timeouts")] >= 1
    assert st[names.index("errors")] & 1
    k = _dev_view(A.mirror_ptr(la), n)
    assert float(k[4096:].abs().max()) == 0.0, "nothing of the stalled tile was stored"
    A.set_test_stall_tile(-1)
    out = torch.empty(n, device="cuda")
    for _ in range(6):
        A.round()
        A.sync()
        B.round()
        B.sync()
    B.snapshot(out.data_ptr(), _stream())
    torch.cuda.synchronize()
    assert ((out - init).norm() / init.norm()).item() < 1e-5
    assert A.check_guards() == 0 and B.check_guards() == 0


@pytest.mark.parametrize("bits", [8, 1])
def test_chain_bit_exact_with_the_host_model(cu, core, bits):
    """A - B - C with B forwarding: values and every mirror of all three replicas, pass by pass, against the host model
    (what arrives on one link is passed on over the other in the same pass, is not answered on its own link, and two
    links that deliver in the same pass are added up before they go into the values)."""
    n = 2 * 4096 + 333
    torch.manual_seed(40 + bits)
    reps = [_replica(cu, n, bits=bits) for _ in range(3)]
    la, lb0 = connect_local(reps[0], reps[1])
    lb1, lc = connect_local(reps[1], reps[2])
    links = [[la], [lb0, lb1], [lc]]
    models = [Oracle(core, n, 32, 1, bits), Oracle(core, n, 32, 2, bits), Oracle(core, n, 32, 1, bits)]
    init = torch.randn(n)
    models[0].v = init.clone()
    reps[0].load_values(init.cuda().data_ptr(), _stream())     # B and C start from zero and are streamed the state
    peer = {(0, 0): (1, 0), (1, 0): (0, 0), (1, 1): (2, 0), (2, 0): (1, 1)}
    inbox = {key: [] for key in peer}
    for it in range(12 if bits == 8 else 30):
        if it in (3, 8):
            for i, scale in ((0, 1e-1), (2, 1.0)):
                d = torch.randn(n) * scale
                models[i].v += d
                models[i].mark()
                reps[i].add(d.cuda().data_ptr(), _stream())
            torch.cuda.synchronize()
        for i in range(3):
            reps[i].round()
            reps[i].sync()
            arrived = {l: inbox[(i, l)] for l in range(len(models[i].k))}
            for l in arrived:
                inbox[(i, l)] = []
            for l, frame in models[i].visit(arrived).items():
                inbox[peer[(i, l)]].append(frame)
            for l, dev_link in enumerate(links[i]):
                v, k = _state(cu, reps[i], dev_link)
                assert torch.equal(v, models[i].v), f"values of replica {i} differ in pass {it}"
                assert torch.equal(k, models[i].k[l]), f"mirror {l} of replica {i} differs in pass {it}"
    for r in reps:
        assert r.status()[5] == 0 and r.check_guards() == 0


def test_chain_forwarding_converges_to_the_sum(cu):
    """A - B - C: updates made at the ends reach the other end through B's forwarding."""
    n = 5 * 4096 + 123
    torch.manual_seed(11)
    reps = [_replica(cu, n) for _ in range(3)]
    connect_local(reps[0], reps[1])
    connect_local(reps[1], reps[2])
    init = torch.randn(n, device="cuda")
    reps[0].load_values(init.data_ptr(), _stream())
    # late-join emulation: B and C start from zero and are streamed the state
    expect = init.clone()
    for it in range(60):
        if it in (10, 20, 30):
            for i, r in enumerate(reps):
                d = torch.randn(n, device="cuda") * 1e-2 * (i + 1)
                r.add(d.data_ptr(), _stream())
                expect += d
        for r in reps:
            r.round()
        for r in reps:
            r.sync()
    out = torch.empty(n, device="cuda")
    for r in reps:
        r.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        rel = ((out - expect).norm() / expect.norm()).item()
        assert rel < 5e-5, rel  # two hops, each with its own 2^-22 relative cut-off
    # quiescent: an idle round lists no tile
    for r in reps:
        r.round()
        r.sync()
    names = cu.status_names()
    for r in reps:
        st = r.status()
        assert st[names.index("last_work_count")] == 0
        assert st[names.index("errors")] == 0


def test_mesh_group_no_forwarding(cu):
    """Four replicas as one mesh group: one mirror each, every update crosses exactly one hop."""
    n = 3 * 4096 + 9
    torch.manual_seed(5)
    reps = [_replica(cu, n) for _ in range(4)]
    connect_mesh(reps)
    init = torch.randn(n, device="cuda")
    for r in reps:  # a mesh group starts from a common state
        r.load_values(init.data_ptr(), _stream())
        r.copy_mirror_from_values(0)
    expect = init.clone()
    for it in range(40):
        if it in (0, 7, 19):
            for i, r in enumerate(reps):
                d = torch.randn(n, device="cuda") * 1e-2 * (i + 1)
                r.add(d.data_ptr(), _stream())
                expect += d
        for r in reps:
            r.round()
        for r in reps:
            r.sync()
    out = torch.empty(n, device="cuda")
    for r in reps:
        r.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        rel = ((out - expect).norm() / expect.norm()).item()
        assert rel < 1e-5, rel


def test_engine_thread_free_running(cu):
    n = 8 * 4096
    torch.manual_seed(4)
    A, B = _replica(cu, n), _replica(cu, n)
    connect_local(A, B)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    A.start_engine()
    B.start_engine()
    import time

    out = torch.empty(n, device="cuda")
    deadline = time.time() + 10
    ok = False
    while time.time() < deadline:
        B.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        if ((out - init).norm() / init.norm()).item() < 1e-5:
            ok = True
            break
        time.sleep(0.01)
    d = torch.randn(n, device="cuda")
    B.add(d.data_ptr(), _stream())
    ok2 = False
    deadline = time.time() + 10
    while time.time() < deadline:
        A.snapshot(out.data_ptr(), _stream())
        torch.cuda.synchronize()
        if ((out - (init + d)).norm() / init.norm()).item() < 1e-5:
            ok2 = True
            break
        time.sleep(0.01)
    A.stop_engine()
    B.stop_engine()
    assert ok and ok2


def test_trace_ring_records_rounds(cu):
    n = 2 * 4096
    A, B = _replica(cu, n), _replica(cu, n)
    connect_local(A, B)
    init = torch.randn(n, device="cuda")
    A.load_values(init.data_ptr(), _stream())
    for _ in range(5):
        A.round()
        B.round()
    st = A.status()
    assert len(st) == cu.STATUS_WORDS + cu.TRACE_ENTRIES * cu.TRACE_WORDS
    recs = [st[cu.STATUS_WORDS + i * cu.TRACE_WORDS: cu.STATUS_WORDS + (i + 1) * cu.TRACE_WORDS] for i in range(5)]
    assert [r[1] for r in recs] == [0, 1, 2, 3, 4], "round numbers"
    assert all(r[0] > 0 for r in recs) and recs[4][0] > recs[0][0], "GPU clock stamps increase"
    assert recs[0][2] >= 1, "tiles handled by the recording group"


def test_vmm_blocks_when_available(cu):
    rep = _replica(cu, 4096, shareable=True)
    b = rep.alloc_edge_block()
    if cu.vmm_available():
        assert rep.edge_block_is_vmm(b)
