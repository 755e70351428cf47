"""The allocation-free table-scales entry point, called through its exported C symbol.

Some callers cannot allocate device memory at the moment they need per-tensor energies (their pool owns
the whole GPU, or a cudaMalloc would stall a latency-critical loop); for them the library carries its own
scratch array.  This test calls that entry point twice in a row with different tables and checks both
results against the ordinary entry point, which takes its scratch from the caller.  The file name makes
pytest collect it last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _table(seed, sizes):
    torch.manual_seed(seed)
    offs = [0]
    for s in sizes:
        offs.append(offs[-1] + s)
    x = torch.cat([torch.randn(s, device="cuda") * (3.0 ** (i - 2)) for i, s in enumerate(sizes)]) if offs[-1] else torch.empty(0, device="cuda")
    return x, torch.tensor(offs, dtype=torch.int64, device="cuda"), offs[-1]


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    from sharedtensor_b200 import _build, _native

    cu = _native.cuda()
    lib = ctypes.CDLL(str(_build.target_path("_cuda")))
    fn = lib.st_table_scales_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.st_noalloc_strerror.restype = ctypes.c_char_p
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream

    for seed, sizes in ((1, [5, 70000, 1, 300000, 4096, 0, 65536]), (2, [200000, 3, 131072])):
        x, offs, total = _table(seed, sizes)
        n_seg = len(sizes)
        # ordinary entry point: scratch allocated by the caller
        scratch = torch.empty(cu.table_scales_scratch_doubles(n_seg, total), dtype=torch.float64, device="cuda")
        ref_sum = torch.empty(n_seg, dtype=torch.float64, device="cuda")
        ref_exp = torch.empty(n_seg, dtype=torch.int8, device="cuda")
        cu.table_scales(x.data_ptr(), offs.data_ptr(), n_seg, total, scratch.data_ptr(), ref_sum.data_ptr(), ref_exp.data_ptr(), stream)
        # allocation-free entry point: outputs are still ours, scratch is the library's
        out_sum = torch.full((n_seg,), -1.0, dtype=torch.float64, device="cuda")
        out_exp = torch.full((n_seg,), 99, dtype=torch.int8, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(x.data_ptr(), offs.data_ptr(), n_seg, total, out_sum.data_ptr(), out_exp.data_ptr(), stream)
        assert rc == 0, lib.st_noalloc_strerror(rc)
        torch.cuda.synchronize()
        if seed == 2:  # (the first call on a device may load the library's device image; the second must leave memory alone)
            assert torch.cuda.mem_get_info()[0] == free_before, "the call allocated device memory"
        assert torch.allclose(out_sum, ref_sum, rtol=1e-9, atol=0.0)
        assert torch.equal(out_exp, ref_exp)
        seg = [float((x[offs[i]:offs[i + 1]].double() ** 2).sum()) for i in range(n_seg)]
        assert torch.allclose(out_sum.cpu(), torch.tensor(seg, dtype=torch.float64), rtol=1e-9)

    # sizes beyond the built-in scratch are refused with a message, nothing is launched
    x, offs, total = _table(3, [16])
    o1 = torch.empty(1, dtype=torch.float64, device="cuda")
    o2 = torch.empty(1, dtype=torch.int8, device="cuda")
    assert fn(x.data_ptr(), offs.data_ptr(), 5000, total, o1.data_ptr(), o2.data_ptr(), stream) == -1
    assert fn(x.data_ptr(), offs.data_ptr(), 1, (1 << 31) + 1, o1.data_ptr(), o2.data_ptr(), stream) == -2
    assert b"scratch" in lib.st_noalloc_strerror(-2)

    # a table whose offsets go further than the total the caller gave: no read past the scratch array, NaN instead
    x, offs, total = _table(4, [70000, 200000])
    o1 = torch.zeros(2, dtype=torch.float64, device="cuda")
    o2 = torch.zeros(2, dtype=torch.int8, device="cuda")
    assert fn(x.data_ptr(), offs.data_ptr(), 2, 65536, o1.data_ptr(), o2.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert bool(torch.isnan(o1[1]))
