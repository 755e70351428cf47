"""Table sync on CPU replicas: tensors of very different magnitudes converge independently."""
import time

import torch

import sharedtensor


def test_table_sync_heterogeneous_magnitudes(free_port):
    torch.manual_seed(0)
    tensors = {"big": torch.randn(7, 11) * 100.0, "small": torch.randn(50) * 1e-4, "one": torch.randn(1)}
    a = sharedtensor.createOrFetchTable("127.0.0.1", free_port, tensors)
    b = sharedtensor.createOrFetchTable("127.0.0.1", free_port, {k: torch.zeros_like(v) for k, v in tensors.items()})
    try:
        d = {"big": torch.randn(7, 11), "small": torch.randn(50) * 1e-6, "one": torch.ones(1)}
        b.addFromTensors(d)
        expect = {k: tensors[k] + d[k] for k in tensors}
        out = {k: torch.zeros_like(v) for k, v in tensors.items()}
        ok = False
        t0 = time.time()
        while time.time() - t0 < 20 and not ok:
            ok = True
            for t in (a, b):
                t.copyToTensors(out)
                for k in tensors:
                    rel = ((out[k] - expect[k]).norm() / expect[k].norm()).item()
                    ok = ok and rel < 1e-4  # relative PER TENSOR: the small one is not drowned by the big one
            time.sleep(0.02)
        assert ok
        sc = a.scales()
        assert sc["big"]["rms_exp"] > sc["small"]["rms_exp"] + 15
        assert abs(sc["one"]["sumsq"] - float(expect["one"] ** 2)) < 1e-3
    finally:
        b.close()
        a.close()


def test_table_layout_alignment():
    from sharedtensor_b200.ops.table import TableLayout

    lay = TableLayout({"a": torch.Size([3]), "b": torch.Size([2, 40]), "c": torch.Size([])}, 32)
    assert lay.offsets == {"a": 0, "b": 32, "c": 128}
    assert lay.numel == 160
    flat = torch.arange(160.0)
    v = lay.views(flat)
    assert v["b"].shape == (2, 40) and v["b"][0, 0] == 32.0 and v["c"].item() == 128.0
