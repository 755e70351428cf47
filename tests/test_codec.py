"""T0: the host codec against a numpy restatement of the reference's loops
(encoder src/sharedtensor.c:156-174, decoder 106-111)."""
import numpy as np
import pytest
import torch

from sharedtensor_b200 import _native

core = _native.core()


def np_ref_encode(r: np.ndarray):
    """Sequential fp32 model of the reference sender loop; returns (scale, bits, new residual)."""
    r = r.astype(np.float32).copy()
    acc = np.float32(0)
    for x in r:
        acc = np.float32(acc + np.float32(x * x))
    mean = np.float32(acc / np.float32(len(r)))
    s = np.float32(np.sqrt(np.float64(mean)))
    if s > 0 and np.isfinite(s):
        scale = np.float32(2.0 ** np.floor(np.log2(np.float64(s))))
    else:
        scale = np.float32(0)
    bits = np.zeros((len(r) + 7) // 8, dtype=np.uint8)
    for i in range(len(r)):
        if r[i] > 0:
            r[i] = np.float32(r[i] - scale)
        else:
            bits[i // 8] |= 1 << (i % 8)
            r[i] = np.float32(r[i] + scale)
    return scale, bits, r


def np_ref_decode(bits, scale, n):
    i = np.arange(n)
    b = (bits[i // 8] >> (i % 8)) & 1
    return (np.float32(scale) - b.astype(np.float32) * np.float32(scale) * 2).astype(np.float32)


@pytest.mark.parametrize("n", [1, 2, 7, 8, 9, 31, 32, 33, 240, 1000])
@pytest.mark.parametrize("kind", ["normal", "zeros", "tiny", "mixed"])
def test_reference_encoder_bit_exact(n, kind):
    rng = np.random.default_rng(n * 7 + len(kind))
    if kind == "normal":
        r = rng.standard_normal(n)
    elif kind == "zeros":
        r = np.zeros(n)
    elif kind == "tiny":
        r = rng.standard_normal(n) * 1e-30
    else:
        r = rng.standard_normal(n) * 10.0 ** rng.integers(-6, 3, n)
        r[::3] = 0.0
        r[1::5] = -0.0
    r = r.astype(np.float32)
    scale_np, bits_np, r_np = np_ref_encode(r)
    t = torch.from_numpy(r.copy())
    bits = torch.zeros(core.sign_bytes(n), dtype=torch.uint8)
    scale = core.encode_residual_ref(t.data_ptr(), n, bits.data_ptr())
    assert np.float32(scale) == scale_np
    assert np.array_equal(bits.numpy(), bits_np)
    assert np.array_equal(t.numpy(), r_np)
    # scale is zero or an exact power of two
    if scale:
        m, _ = np.frexp(scale)
        assert m == 0.5


@pytest.mark.parametrize("n", [1, 5, 64, 240, 1001])
def test_decoder_matches_reference(n):
    rng = np.random.default_rng(n)
    bits = rng.integers(0, 256, (n + 7) // 8, dtype=np.uint8)
    dst = rng.standard_normal(n).astype(np.float32)
    expect = dst + np_ref_decode(bits, 0.25, n)
    t = torch.from_numpy(dst.copy())
    t2 = torch.from_numpy(dst.copy())
    b = torch.from_numpy(bits)
    core.decode_tensor_add(b.data_ptr(), 0.25, n, t.data_ptr(), t2.data_ptr())
    assert np.array_equal(t.numpy(), expect)
    assert np.array_equal(t2.numpy(), expect)
    # scale 0 is a no-op whatever the bits say
    core.decode_tensor_add(b.data_ptr(), 0.0, n, t.data_ptr(), 0)
    assert np.array_equal(t.numpy(), expect)


def test_mirror_form_tracks_residual_form():
    """Quantising v - k and stepping k produces the reference's residual stream.  The two forms
    round differently in the last bit (the mirror form subtracts two exact numbers each frame, the
    residual form accumulates roundings), so signs may differ for elements within an ulp of zero."""
    n = 240
    rng = np.random.default_rng(3)
    v = torch.from_numpy(rng.standard_normal(n).astype(np.float32))
    k = torch.zeros(n)
    resid = v.clone()
    bits_a = torch.zeros(core.sign_bytes(n), dtype=torch.uint8)
    bits_b = torch.zeros_like(bits_a)
    for it in range(40):
        sa = core.encode_tensor(v.data_ptr(), k.data_ptr(), n, bits_a.data_ptr(), 0.0, 0)  # rule 0: the reference's
        sb = core.encode_residual_ref(resid.data_ptr(), n, bits_b.data_ptr())
        if it < 12:
            assert sa == sb
            assert torch.equal(bits_a, bits_b)
        assert torch.allclose(v - k, resid, atol=1e-6)
    assert (v - k).norm() / v.norm() < 2e-2  # the tensor-wide scale drains outliers slowly


def test_tensor_stream_converges_to_fp32_floor():
    n = 240
    torch.manual_seed(0)
    v = torch.randn(n)
    k = torch.zeros(n)
    peer = torch.zeros(n)
    bits = torch.zeros(core.sign_bytes(n), dtype=torch.uint8)
    for _ in range(400):
        s = core.encode_tensor(v.data_ptr(), k.data_ptr(), n, bits.data_ptr(), 2.0 ** -21)
        core.decode_tensor_add(bits.data_ptr(), s, n, peer.data_ptr(), 0)
    assert torch.equal(peer, k)
    assert ((peer - v).norm() / v.norm()) < 1e-5
    assert (peer - v).abs().max() < 1e-4


@pytest.mark.parametrize("block", [32, 64, 256, 4096])
@pytest.mark.parametrize("n", [1, 31, 32, 33, 100, 4096, 5000])
def test_block_roundtrip_and_convergence(block, n):
    torch.manual_seed(n + block)
    v = torch.randn(n) * torch.logspace(-3, 1, n)  # heterogeneous magnitudes
    k = torch.zeros(n)
    peer = torch.zeros(n)
    words = torch.zeros(core.block_words(n), dtype=torch.int32)
    scales = torch.zeros(core.block_scales(n, block), dtype=torch.uint8)
    prev = None
    for it in range(120):
        ss = core.encode_block(v.data_ptr(), k.data_ptr(), n, block, -60, 22, words.data_ptr(), scales.data_ptr())
        core.decode_block_add(words.data_ptr(), scales.data_ptr(), n, block, peer.data_ptr(), 0)
        assert torch.equal(peer, k), "decoder and encoder-side mirror must agree bit for bit"
        prev = ss
    rel = ((peer - v).norm() / v.norm()).item()
    # larger blocks share one scale among more heterogeneous elements and drain more slowly
    assert rel < {32: 1e-5, 64: 1e-5, 256: 1e-3, 4096: 5e-2}[block], rel
    assert prev is not None


def test_block_silent_when_converged():
    n = 256
    v = torch.randn(n)
    k = v.clone()
    words = torch.zeros(core.block_words(n), dtype=torch.int32)
    scales = torch.ones(core.block_scales(n, 32), dtype=torch.uint8)
    ss = core.encode_block(v.data_ptr(), k.data_ptr(), n, 32, -60, 22, words.data_ptr(), scales.data_ptr())
    assert ss == 0.0
    assert int(scales.sum()) == 0
    assert torch.equal(k, v)


def test_block_scale_is_pow2_floor_of_two_thirds_of_the_largest_residual():
    n = 32
    v = torch.full((n,), 3.0)
    k = torch.zeros(n)
    words = torch.zeros(1, dtype=torch.int32)
    scales = torch.zeros(1, dtype=torch.uint8)
    core.encode_block(v.data_ptr(), k.data_ptr(), n, 32, -60, 22, words.data_ptr(), scales.data_ptr())
    assert int(scales[0]) - 127 == 1  # largest residual 3 -> 2/3 of it is 2 -> 2^1
    assert int(words[0]) == 0          # all positive -> bit 0
    assert torch.equal(k, torch.full((n,), 2.0))


def test_bisection_shrinks_the_error_bound_every_frame():
    """The largest outstanding residual falls to at most 2/3 with every frame, and by about half on average."""
    n = 4096
    torch.manual_seed(9)
    v = torch.randn(n) * torch.exp(torch.randn(n))  # heavy-tailed
    k = torch.zeros(n)
    words = torch.zeros(core.block_words(n), dtype=torch.int32)
    scales = torch.zeros(core.block_scales(n, 32), dtype=torch.uint8)
    worst = []
    for _ in range(14):
        worst.append(core.encode_block(v.data_ptr(), k.data_ptr(), n, 32, -60, 22, words.data_ptr(), scales.data_ptr()))
    for a, b in zip(worst[:10], worst[1:11]):
        assert b <= a * (2.0 / 3.0) * (1 + 1e-6)
    assert worst[10] <= worst[0] * 0.56 ** 10
    assert ((v - k).norm() / v.norm()) < 1e-3


def test_segment_sumsq():
    x = torch.arange(10, dtype=torch.float32)
    out = core.segment_sumsq(x.data_ptr(), [0, 3, 3, 10])
    assert out == [5.0, 0.0, float((x[3:] ** 2).sum())]


@pytest.mark.parametrize("n", [1, 7, 8, 9, 1000, 65537, 2_100_003])
def test_fast_paths_are_bit_identical_to_the_plain_codec(n):
    """The AVX2 / multi-threaded host paths (the sizes cover the scalar tail, one thread and several threads) give
    exactly the bits, the scale and the mirror of the plain loops, NaNs and exact zeros included."""
    P = lambda t: t.data_ptr()  # noqa: E731
    g = torch.Generator().manual_seed(n)
    v = torch.randn(n, generator=g)
    k = torch.randn(n, generator=g) * 0.5
    if n > 100:
        v[5] = float("nan")
        v[17] = 0.0
        k[17] = 0.0
    k1, k2 = k.clone(), k.clone()
    b1 = torch.zeros((n + 7) // 8, dtype=torch.uint8)
    b2 = torch.full_like(b1, 0xAA)
    vmax = float(torch.nan_to_num(v.abs(), nan=0.0).max())
    s1 = core.encode_tensor(P(v), P(k1), n, P(b1), vmax * 2.0 ** -22, 1)
    s2 = core.encode_tensor_fast(P(v), P(k2), n, P(b2), 0.0, 2.0 ** -22)
    assert s1 == s2 and s1 > 0
    assert torch.equal(b1, b2)
    assert torch.equal(torch.nan_to_num(k1, nan=7.0), torch.nan_to_num(k2, nan=7.0))
    # a frame below the cut-off: bits only, the mirror stays
    k3 = k.clone()
    assert core.encode_tensor_fast(P(v), P(k3), n, P(b2), 1e9, 0.0) == 0.0
    assert torch.equal(torch.nan_to_num(k3, nan=7.0), torch.nan_to_num(k, nan=7.0))
    k4 = k.clone()
    core.encode_tensor(P(v), P(k4), n, P(b1), 1e9, 1)
    assert torch.equal(b1, b2)
    # decode
    d1 = torch.randn(n, generator=g)
    d2, m1, m2 = d1.clone(), torch.zeros(n), torch.zeros(n)
    core.decode_tensor_add(P(b1), 0.25, n, P(d1), P(m1))
    core.decode_tensor_add_fast(P(b1), 0.25, n, P(d2), P(m2))
    assert torch.equal(d1, d2) and torch.equal(m1, m2)
    # block format: whole blocks vectorised, the ragged tail through the plain loop, pieces over threads
    for B in (32, 64, 256, 4096):
        v = torch.randn(n, generator=g)
        if n > 100:
            v[3] = float("nan")
            v[40] = 0.0
        k1, k2 = k.clone(), k.clone()
        w1 = torch.zeros((n + 31) // 32, dtype=torch.int32)
        w2 = torch.full_like(w1, 0x5A5A5A5A)
        c1 = torch.zeros((n + B - 1) // B, dtype=torch.uint8)
        c2 = torch.full_like(c1, 7)
        r1 = core.encode_block(P(v), P(k1), n, B, -100, 22, P(w1), P(c1))
        r2 = core.encode_block_fast(P(v), P(k2), n, B, -100, 22, P(w2), P(c2))
        assert r1 == r2 and torch.equal(w1, w2) and torch.equal(c1, c2), B
        assert torch.equal(torch.nan_to_num(k1, nan=7.0), torch.nan_to_num(k2, nan=7.0)), B
        a1, a2, m1, m2 = torch.zeros(n), torch.zeros(n), torch.ones(n), torch.ones(n)
        core.decode_block_add(P(w1), P(c1), n, B, P(a1), P(m1))
        core.decode_block_add_fast(P(w1), P(c1), n, B, P(a2), P(m2))
        assert torch.equal(a1, a2) and torch.equal(m1, m2), B


@pytest.mark.parametrize("n", [1, 31, 1000, 65537, 2_100_003])
def test_fast_eight_bit_frames_are_bit_identical_to_the_plain_codec(n):
    """8-bit integer frames as the TCP edges carry them (one code byte per element): the AVX2 + FMA / multi-threaded
    path against the plain loops, with a NaN and exact zeros in the data; taking a frame back undoes its step."""
    P = lambda t: t.data_ptr()  # noqa: E731
    g = torch.Generator().manual_seed(n + 1)
    for B in (32, 256, 4096):
        v = torch.randn(n, generator=g) * torch.logspace(-3, 2, n)
        k = v + torch.randn(n, generator=g) * 1e-2 * v.abs()
        if n > 100:
            v[3] = float("nan")
            v[40] = 0.0
            k[40] = 0.0
        k1, k2 = k.clone(), k.clone()
        ns = (n + B - 1) // B
        c1, c2 = torch.zeros(n, dtype=torch.uint8), torch.full((n,), 7, dtype=torch.uint8)
        s1, s2 = torch.zeros(ns, dtype=torch.uint8), torch.full((ns,), 9, dtype=torch.uint8)
        r1 = core.encode_block_int(P(v), P(k1), n, B, -100, 22, 8, P(c1), P(s1))
        r2 = core.encode_block_int8_fast(P(v), P(k2), n, B, -100, 22, P(c2), P(s2))
        assert r1 == r2 and torch.equal(s1, s2), B
        loud = s1.ne(0).repeat_interleave(B)[:n]
        assert torch.equal(c1[loud], c2[loud]), B          # (codes of a silent block's NaN are not looked at)
        assert torch.equal(torch.nan_to_num(k1, nan=7.0), torch.nan_to_num(k2, nan=7.0)), B
        steps = torch.zeros(n)
        core.block_int_steps(P(c1), P(s1), n, B, 8, P(steps))
        a1, a2, m1, m2 = torch.zeros(n), torch.zeros(n), torch.ones(n), torch.ones(n)
        core.decode_block_int_add(P(c1), P(s1), n, B, 8, 1.0, P(a1), P(m1))
        core.decode_block_int8_add_fast(P(c1), P(s1), n, B, 1.0, P(a2), P(m2))
        assert torch.equal(a1, a2) and torch.equal(m1, m2) and torch.equal(a1, steps), B
        core.decode_block_int8_add_fast(P(c1), P(s1), n, B, -1.0, P(a2), 0)
        assert torch.equal(a2, torch.zeros(n)), B
