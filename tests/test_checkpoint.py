import torch

import sharedtensor
from sharedtensor_b200.utils import checkpoint


def test_save_refound_and_restore(tmp_path, free_port):
    a = sharedtensor.createOrFetch("127.0.0.1", free_port, torch.arange(24.0).view(2, 3, 4))
    a.addFromTensor(torch.ones(2, 3, 4))
    path = str(tmp_path / "ckpt.pt")
    checkpoint.save(a, path, extra={"step": 7})
    a.close()
    v, extra = checkpoint.load_values(path)
    assert extra == {"step": 7} and v.shape == (2, 3, 4)
    assert torch.equal(v, torch.arange(24.0).view(2, 3, 4) + 1)
    b = sharedtensor.createOrFetch("127.0.0.1", free_port + 1 if free_port < 65000 else free_port - 1, v)
    try:
        out = torch.zeros(2, 3, 4)
        b.copyToTensor(out)
        assert torch.equal(out, v)
        b.addFromTensor(torch.ones(2, 3, 4))
        checkpoint.restore_into(b, path)
        b.copyToTensor(out)
        assert torch.equal(out, v)
    finally:
        b.close()


def test_cpu_affinity_helper_is_a_no_op_without_a_gpu():
    import os

    from sharedtensor_b200.utils.affinity import bind_to_gpu

    before = os.sched_getaffinity(0)
    assert bind_to_gpu(0) == sorted(before)     # no NVML device here: nothing to intersect with
    assert os.sched_getaffinity(0) == before
